/* C ABI of libmb200_hybrid.so: kernels of layered decoders (a list of layers, each with its own kind of token mixer),
 * with an fp32 residual stream and bf16 or fp32 storage of activations and weights.
 *
 * Conventions: pointers are device pointers; `dt` = 0 (bf16) or 1 (fp32) is the storage type of every `void*` activation
 * and weight operand; index tensors are int32 unless said otherwise; `stream` is a cudaStream_t.  Every call returns 0 or
 * an error code and leaves the text in mbh_last_error().  No call synchronises or allocates.
 */
#ifndef MISTRAL_B200_HYBRID_H
#define MISTRAL_B200_HYBRID_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MBH_ABI_VERSION 1

int mbh_abi_version(void);
const char* mbh_last_error(void);

/* x32[t, :] = table[tokens[t], :] * scale.  tokens: int64 [T]; table [V, D]; x32: fp32 [T, D]. */
int mbh_embed_scale(const void* tokens, const void* table, float scale, void* x32, int64_t T, int64_t D, int dt, void* stream);

/* y[t, :] = x32[t, :] / sqrt(mean(x32[t]^2) + eps) * w.  x32 fp32 [T, D] (the residual stream); y, w: storage type. */
int mbh_rmsnorm(const void* x32, const void* w, void* y, int64_t T, int64_t D, float eps, int dt, void* stream);

/* Linear x[M, K] W[N, K]^T (+ bias[N]) with an epilogue:
 *   0  out[M, N] = act(.)      SiLU on columns < n_act, identity elsewhere
 *   1  out32[M, N] += .        in-place add into the fp32 residual stream
 *   2  out[M, N/2]             rows of W interleaved (2c gate, 2c+1 up): g = min(gate, limit), u = clamp(up, -limit, limit),
 *                              out = g * sigmoid(alpha * g) * (u + 1)
 *   3  out32[M, N] = .         fp32 result (logits)
 * Any M, N, K.  M <= 8 runs the weight-streaming kernel, larger M the tiled one (tensor cores for bf16). */
int mbh_linear(const void* x, const void* w, const void* bias, void* out, void* out32, int64_t M, int64_t N, int64_t K, int epi, int64_t n_act,
               float limit, float alpha, int dt, void* stream);

/* The epilogues of mbh_linear alone, applied to y[M, N] (storage type, N even) that another GEMM produced. */
int mbh_linear_epilogue(const void* y, const void* bias, void* out, void* out32, int64_t M, int64_t N, int epi, int64_t n_act, float limit, float alpha,
                        int dt, void* stream);

/* Splits qkv[T, H*d + G*d + G*e]; RMS-norms every q and k head over d with the shared weights qnorm / knorm [d] (null: no
 * norm); multiplies q at position p by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) (temp_every = 0: no temperature);
 * value mixing: vmix_mode 0 none, 1 copy v to v_first[T, G*e], 2 v <- (1 - *vmix) v + *vmix v_first; then scatters k and v to
 * row cache_rows[t] of cache_k [rows, G, d] / cache_v [rows, G, e] (-1: not cached) and writes q_out [T, H*d]. */
int mbh_attn_prep(const void* qkv, const void* qnorm, const void* knorm, const void* positions, const void* cache_rows, void* q_out, void* cache_k,
                  void* cache_v, void* v_first, const void* vmix, int vmix_mode, int64_t T, int64_t H, int64_t G, int64_t d, int64_t e, float eps,
                  float temp_coef, int64_t temp_every, int dt, void* stream);

/* Causal softmax attention of q[T, H*d] over the ring: token t of sequence b (q_start[B+1]) at position positions[t] sees keys
 * 0..position of cache block slots[b] (W rows each, key j in row j % W); score = q.k * scale + bias_tab[min(distance, n_tab-1), h]
 * (fp32 [n_tab, H]).  out [T, H*e].
 * n_tiles > 0 (prompts): the number of 64-query tiles, sum over sequences of ceil(len / 64); with bf16 storage and key/value
 * sizes among {32, 64, 128} the tensor-core kernel runs (P rounded to bf16 before P V).  n_tiles = 0: the exact fp32 kernel,
 * with `splits` > 1 CTAs per (token, head) along the keys (decode) and their partial results in scratch (fp32 [T*H, splits, 2 + e]). */
int mbh_attn_bias(const void* q, const void* cache_k, const void* cache_v, const void* bias_tab, int64_t n_tab, const void* positions,
                  const void* q_start, const void* slots, void* out, int64_t T, int64_t B, int64_t W, int64_t H, int64_t G, int64_t d, int64_t e,
                  float scale, int64_t n_tiles, int64_t splits, void* scratch, int dt, void* stream);

/* Decayed linear attention.  qkvg [T, 2*H*d + 2*H*e] = q | k | v | gate; per head S <- decay[h] S + k v^T, o = S^T q, fp32;
 * state fp32 [slots, H, d, e] is read (unless seqpos[b] == 0: starts at zero) and written back; o32 fp32 [T, H*e]. */
int mbh_lightning_scan(const void* qkvg, void* state, const void* decay, const void* q_start, const void* seqpos, const void* slots, void* o32,
                       int64_t B, int64_t H, int64_t d, int64_t e, int dt, void* stream);

/* y[t, :] = rms_norm(o32[t, :N]; eps) * w * sigmoid(g[t * g_pitch + g_off + :N]). */
int mbh_gated_headnorm(const void* o32, const void* w, const void* g, int64_t g_pitch, int64_t g_off, void* y, int64_t T, int64_t N, float eps,
                       int dt, void* stream);

#ifdef __cplusplus
}
#endif
#endif
