// Latent attention: queries, keys and values are linear maps of small per-token latents, and the cache keeps one row per
// token, [c (kv_rank) | rotated key part (rot_dim)], shared by all heads.
//
//   latent_prep     from the packed input projection y = [W_dq h | W_dkv h | W_g h]: RMS norm of the query latent -> cq;
//                   RMS norm of the key/value latent c and the rotated shared key part -> the token's ring row
//   latent_absorb   per head: rotates the rotated part of q and folds the key up-projection into the query,
//                   qa = [W_uk[h]^T q_plain | rot(q_rot)], so that q.k = qa . [c | k_rot] and attention runs over the latent rows
//                   (attn_bias_kernel with one key/value head, key size kv_rank + rot_dim, value = the row's first kv_rank entries)
//   latent_vup      per head: out = W_uv[h] o_latent, times the sigmoid of the head's output-gate logit
//   attn_latent_decode  one token per sequence: a CTA takes a span of one sequence's latent rows for ALL heads, so a row is read
//                   from memory once per step instead of once per head; partial (max, sum, acc) per head go to attn_merge_kernel
//   latent_expand   whole prompts in bf16 take the other form: keys [W_uk c | rot(k_r)] and values W_uv c of the prompt's own tokens
//                   are written out per head (two Linears, then this scatter into a temporary ring) and the tensor-core prompt
//                   kernel runs ordinary multi-head attention on them; latent_absorb without W_uk only rotates q; head_gate
//                   applies the output gate
//
// Rotation: interleaved pairs (2i, 2i+1) of the first rot_dims entries, angle = position * freq[i] evaluated in double
// precision (the table of frequencies comes from the host, any frequency scaling already applied), cos and sin multiplied by `mag`.
#pragma once
#include "hybrid_common.cuh"

namespace mbh {

struct LatentPrepArgs {
    const void* y;           // [T, q_rank + kv_rank + rot_dim + n_extra]
    const void* qnorm;       // [q_rank]
    const void* cnorm;       // [kv_rank]
    const double* freq;      // [rot_dims / 2]
    const int* positions;    // [T]
    const int* cache_rows;   // [T] ring row or -1
    void* cq;                // [T, q_rank]
    void* ring;              // [rows, kv_rank + rot_dim]
    int q_rank, kv_rank, rot_dim, rot_dims, pitch;
    float eps, mag;
};

__device__ __forceinline__ void rot_pair(float u, float v, int pos, double f, float mag, float& ou, float& ov) {
    double sn, cs;
    sincos((double)pos * f, &sn, &cs);
    const float c = (float)cs * mag, s = (float)sn * mag;
    ou = u * c - v * s;
    ov = v * c + u * s;
}

template <typename T>
__global__ void __launch_bounds__(128) latent_prep_kernel(LatentPrepArgs a) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const T* row = static_cast<const T*>(a.y) + (size_t)t * a.pitch;
    const int pos = a.positions[t], crow = a.cache_rows ? a.cache_rows[t] : -1;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.q_rank; i += blockDim.x) { const float v = to_f(row[i]); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float inv_q = 1.f / sqrtf(ss / (float)a.q_rank + a.eps);
    T* cq = static_cast<T*>(a.cq) + (size_t)t * a.q_rank;
    const T* qn = static_cast<const T*>(a.qnorm);
    for (int i = threadIdx.x; i < a.q_rank; i += blockDim.x) cq[i] = from_f<T>(to_f(row[i]) * inv_q * to_f(qn[i]));
    if (crow < 0) return;
    const T* kv = row + a.q_rank;
    ss = 0.f;
    for (int i = threadIdx.x; i < a.kv_rank; i += blockDim.x) { const float v = to_f(kv[i]); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float inv_c = 1.f / sqrtf(ss / (float)a.kv_rank + a.eps);
    T* dst = static_cast<T*>(a.ring) + (size_t)crow * (a.kv_rank + a.rot_dim);
    const T* cn = static_cast<const T*>(a.cnorm);
    for (int i = threadIdx.x; i < a.kv_rank; i += blockDim.x) dst[i] = from_f<T>(to_f(kv[i]) * inv_c * to_f(cn[i]));
    const T* kr = kv + a.kv_rank;
    T* dr = dst + a.kv_rank;
    for (int i = threadIdx.x; i < a.rot_dims / 2; i += blockDim.x) {
        float u, v;
        rot_pair(to_f(kr[2 * i]), to_f(kr[2 * i + 1]), pos, a.freq[i], a.mag, u, v);
        dr[2 * i] = from_f<T>(u);
        dr[2 * i + 1] = from_f<T>(v);
    }
    for (int i = a.rot_dims + threadIdx.x; i < a.rot_dim; i += blockDim.x) dr[i] = kr[i];
}

struct LatentAbsorbArgs {
    const void* q;           // [T, H, dn + rot_dim]
    const void* w_uk;        // [H * dn, kv_rank]
    const double* freq;
    const int* positions;
    void* qa;                // [T, H, kv_rank + rot_dim]
    int H, dn, rot_dim, rot_dims, kv_rank;
    float mag;
};

// grid (token * head, blocks of 128 latent columns); thread r owns one latent column: W_uk[h] is read row by row, coalesced over r,
// four rows in flight
template <typename T>
__global__ void __launch_bounds__(128) latent_absorb_kernel(LatentAbsorbArgs a) {
    extern __shared__ float qs[];  // [dn]
    const int t = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const T* q = static_cast<const T*>(a.q) + ((size_t)t * a.H + h) * (a.dn + a.rot_dim);
    T* qa = static_cast<T*>(a.qa) + ((size_t)t * a.H + h) * (a.kv_rank + a.rot_dim);
    for (int i = threadIdx.x; i < a.dn; i += blockDim.x) qs[i] = to_f(q[i]);
    __syncthreads();
    T* dr = qa + a.kv_rank;
    if (a.w_uk) {
        const T* W = static_cast<const T*>(a.w_uk) + (size_t)h * a.dn * a.kv_rank;
        const int r = blockIdx.y * blockDim.x + threadIdx.x;
        if (r < a.kv_rank) {
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            int i = 0;
            for (; i + 4 <= a.dn; i += 4) {
                a0 = fmaf(qs[i], to_f(W[(size_t)i * a.kv_rank + r]), a0);
                a1 = fmaf(qs[i + 1], to_f(W[(size_t)(i + 1) * a.kv_rank + r]), a1);
                a2 = fmaf(qs[i + 2], to_f(W[(size_t)(i + 2) * a.kv_rank + r]), a2);
                a3 = fmaf(qs[i + 3], to_f(W[(size_t)(i + 3) * a.kv_rank + r]), a3);
            }
            for (; i < a.dn; ++i) a0 = fmaf(qs[i], to_f(W[(size_t)i * a.kv_rank + r]), a0);
            qa[r] = from_f<T>((a0 + a1) + (a2 + a3));
        }
        if (blockIdx.y != 0) return;  // the rotated part is written once
    } else {  // no folding: qa [T, H, dn + rot_dim] = [q plain | rot(q rotated)]
        qa = static_cast<T*>(a.qa) + ((size_t)t * a.H + h) * (a.dn + a.rot_dim);
        dr = qa + a.dn;
        for (int i = threadIdx.x; i < a.dn; i += blockDim.x) qa[i] = q[i];
    }
    const T* qr = q + a.dn;
    const int pos = a.positions[t];
    for (int i = threadIdx.x; i < a.rot_dims / 2; i += blockDim.x) {
        float u, v;
        rot_pair(to_f(qr[2 * i]), to_f(qr[2 * i + 1]), pos, a.freq[i], a.mag, u, v);
        dr[2 * i] = from_f<T>(u);
        dr[2 * i + 1] = from_f<T>(v);
    }
    for (int i = a.rot_dims + threadIdx.x; i < a.rot_dim; i += blockDim.x) dr[i] = qr[i];
}

struct LatentVupArgs {
    const void* o_lat;       // [T, H, kv_rank]
    const void* w_uv;        // [H * dv, kv_rank]
    const void* gate;        // gate logit of (t, h) at gate[t * g_pitch + g_off + h]; null: no gate
    void* out;               // [T, H * dv]
    int H, dv, kv_rank, g_pitch, g_off;
};

// grid (token * head, blocks of value columns); a warp per value column: dot product over the latent, lanes along it
template <typename T>
__global__ void __launch_bounds__(128) latent_vup_kernel(LatentVupArgs a) {
    extern __shared__ float os[];  // [kv_rank]
    const int t = blockIdx.x / a.H, h = blockIdx.x % a.H, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const T* o = static_cast<const T*>(a.o_lat) + ((size_t)t * a.H + h) * a.kv_rank;
    for (int i = threadIdx.x; i < a.kv_rank; i += blockDim.x) os[i] = to_f(o[i]);
    __syncthreads();
    float gate = 1.f;
    if (a.gate) gate = sigmoid_exact(to_f(static_cast<const T*>(a.gate)[(size_t)t * a.g_pitch + a.g_off + h]));
    const T* W = static_cast<const T*>(a.w_uv) + (size_t)h * a.dv * a.kv_rank;
    T* out = static_cast<T*>(a.out) + ((size_t)t * a.H + h) * a.dv;
    for (int j = blockIdx.y * nw + warp; j < a.dv; j += nw * gridDim.y) {
        const T* wr = W + (size_t)j * a.kv_rank;
        float acc = 0.f;
        for (int i = lane; i < a.kv_rank; i += 32) acc = fmaf(os[i], to_f(wr[i]), acc);
        acc = warp_sum(acc);
        if (lane == 0) out[j] = from_f<T>(rnd<T>(acc) * gate);
    }
}

// four consecutive entries of a shared-memory row (4-byte aligned for bf16: even pitch, offset a multiple of 4 entries)
template <typename T> __device__ __forceinline__ void load4_smem(const T* p, float* o);
template <> __device__ __forceinline__ void load4_smem<float>(const float* p, float* o) { o[0] = p[0]; o[1] = p[1]; o[2] = p[2]; o[3] = p[3]; }
template <> __device__ __forceinline__ void load4_smem<bf16>(const bf16* p, float* o) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + 2));
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}

struct LatentDecodeArgs {
    const void* qa;          // [B, H, kv_rank + rot_dim]
    const void* ring;        // [rows, kv_rank + rot_dim]
    const int* positions;    // [B]
    const int* slots;        // [B]
    float* scratch;          // [B * H, splits, 2 + kv_rank]
    int B, W, H, kv_rank, rot_dim;
    float scale;
    int splits;
};

constexpr int LD_WARPS = 8, LD_KT = 32, LD_CPL = 16;  // kv_rank <= 32 * LD_CPL; heads <= LD_WARPS * HPW

// grid (B, splits).  Shared memory: q of all heads (fp32, scaled) | a tile of LD_KT latent rows (row pitch padded against bank
// conflicts) | the tile's probabilities per head.  Warp w owns heads w*HPW .. w*HPW + HPW - 1: scores with a lane per row, then the
// weighted sum of the rows with a lane per LD_CPL strided columns.
template <typename T, int HPW>
__global__ void __launch_bounds__(LD_WARPS * 32) attn_latent_decode_kernel(LatentDecodeArgs a) {
    extern __shared__ __align__(16) unsigned char ld_smem[];
    const int d = a.kv_rank + a.rot_dim, e = a.kv_rank;
    const int kp = d + (sizeof(T) == 2 ? 2 : 1);
    float* qs = reinterpret_cast<float*>(ld_smem);                  // [H][d]
    float* ps = qs + (size_t)a.H * d;                               // [H][LD_KT]
    T* ks = reinterpret_cast<T*>(ps + (size_t)a.H * LD_KT);         // [LD_KT][kp]
    const int b = blockIdx.x, split = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = a.positions[b] + 1;
    int span = (n + a.splits - 1) / a.splits;
    span = (span + LD_KT - 1) / LD_KT * LD_KT;
    const int c0 = split * span, c1 = min(n, c0 + span);
    const T* q = static_cast<const T*>(a.qa) + (size_t)b * a.H * d;
    {
        constexpr int V = Vec<T>::N;
        const int nq = a.H * d;
        if (nq % V == 0 && reinterpret_cast<uintptr_t>(q) % 16 == 0) {
            for (int i = threadIdx.x * V; i < nq; i += blockDim.x * V) {
                float qv[V];
                Vec<T>::load(q + i, qv);
#pragma unroll
                for (int u = 0; u < V; ++u) qs[i + u] = qv[u] * a.scale;
            }
        } else {
            for (int i = threadIdx.x; i < nq; i += blockDim.x) qs[i] = to_f(q[i]) * a.scale;
        }
    }
    const T* ring = static_cast<const T*>(a.ring) + (size_t)a.slots[b] * a.W * d;
    float m[HPW], l[HPW], acc[HPW][LD_CPL];
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        m[hh] = -INFINITY; l[hh] = 0.f;
#pragma unroll
        for (int k = 0; k < LD_CPL; ++k) acc[hh][k] = 0.f;
    }
    const bool words = (d * sizeof(T)) % 4 == 0;
    const bool quads = (d * sizeof(T)) % 16 == 0 && reinterpret_cast<uintptr_t>(ring) % 16 == 0;  // 16-byte loads, 4-byte stores (padded pitch)
    for (int j0 = c0; j0 < c1; j0 += LD_KT) {
        const int cn = min(LD_KT, c1 - j0);
        __syncthreads();
        if (quads) {
            const int nq4 = d * (int)sizeof(T) / 16, pw = kp * (int)sizeof(T) / 4;
            uint32_t* dst = reinterpret_cast<uint32_t*>(ks);
#pragma unroll 4
            for (int idx = threadIdx.x; idx < cn * nq4; idx += blockDim.x) {
                const int r = idx / nq4, i = idx - r * nq4;
                const uint4 v = reinterpret_cast<const uint4*>(ring + (size_t)((j0 + r) % a.W) * d)[i];
                uint32_t* o = dst + r * pw + 4 * i;
                o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
            }
        } else if (words) {
            const int nw = d * (int)sizeof(T) / 4, pw = kp * (int)sizeof(T) / 4;
            uint32_t* dst = reinterpret_cast<uint32_t*>(ks);
            for (int idx = threadIdx.x; idx < cn * nw; idx += blockDim.x) {
                const int r = idx / nw, i = idx - r * nw;
                dst[r * pw + i] = reinterpret_cast<const uint32_t*>(ring + (size_t)((j0 + r) % a.W) * d)[i];
            }
        } else {
            for (int idx = threadIdx.x; idx < cn * d; idx += blockDim.x) {
                const int r = idx / d, i = idx - r * d;
                ks[r * kp + i] = ring[(size_t)((j0 + r) % a.W) * d + i];
            }
        }
        __syncthreads();
        // scores: a lane per row; the row's entries are read once for the warp's HPW heads, q four entries at a time
        float sv[HPW];
#pragma unroll
        for (int hh = 0; hh < HPW; ++hh) sv[hh] = 0.f;
        if (lane < cn) {
            const T* kr = ks + lane * kp;
            int i = 0;
            if (d % 4 == 0) {
                for (; i < d; i += 4) {
                    float k4[4];
                    load4_smem<T>(kr + i, k4);
#pragma unroll
                    for (int hh = 0; hh < HPW; ++hh) {
                        const float4 q4 = *reinterpret_cast<const float4*>(qs + (size_t)min(warp * HPW + hh, a.H - 1) * d + i);
                        sv[hh] = fmaf(q4.x, k4[0], sv[hh]); sv[hh] = fmaf(q4.y, k4[1], sv[hh]);
                        sv[hh] = fmaf(q4.z, k4[2], sv[hh]); sv[hh] = fmaf(q4.w, k4[3], sv[hh]);
                    }
                }
            }
            for (; i < d; ++i) {
                const float kv1 = to_f(kr[i]);
#pragma unroll
                for (int hh = 0; hh < HPW; ++hh) sv[hh] = fmaf(qs[(size_t)min(warp * HPW + hh, a.H - 1) * d + i], kv1, sv[hh]);
            }
        }
#pragma unroll
        for (int hh = 0; hh < HPW; ++hh) {
            const int h = warp * HPW + hh;
            if (h >= a.H) break;
            const float sc = (lane < cn) ? sv[hh] : -INFINITY;
            const float m_new = fmaxf(m[hh], warp_max(sc));
            const float p = (lane < cn) ? expf(sc - m_new) : 0.f;
            const float corr = (m[hh] == -INFINITY) ? 0.f : expf(m[hh] - m_new);
            l[hh] = l[hh] * corr + warp_sum(p);
            m[hh] = m_new;
            ps[h * LD_KT + lane] = p;
#pragma unroll
            for (int k = 0; k < LD_CPL; ++k) acc[hh][k] *= corr;
        }
        __syncwarp();
        for (int r = 0; r < cn; ++r) {
            float kv[LD_CPL];
#pragma unroll
            for (int k = 0; k < LD_CPL; ++k) kv[k] = (lane + 32 * k < e) ? to_f(ks[r * kp + lane + 32 * k]) : 0.f;
#pragma unroll
            for (int hh = 0; hh < HPW; ++hh) {
                const int h = warp * HPW + hh;
                if (h >= a.H) break;
                const float p = ps[h * LD_KT + r];
#pragma unroll
                for (int k = 0; k < LD_CPL; ++k) acc[hh][k] = fmaf(p, kv[k], acc[hh][k]);
            }
        }
    }
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        const int h = warp * HPW + hh;
        if (h >= a.H) break;
        float* part = a.scratch + (((size_t)b * a.H + h) * a.splits + split) * (2 + e);
        if (lane == 0) { part[0] = m[hh]; part[1] = l[hh]; }
#pragma unroll
        for (int k = 0; k < LD_CPL; ++k)
            if (lane + 32 * k < e) part[2 + lane + 32 * k] = acc[hh][k];
    }
}

struct LatentExpandArgs {
    const void* kn;          // [T, H * dn]   W_uk c
    const void* v;           // [T, H * dv]   W_uv c
    const void* ring;        // [rows, kv_rank + rot_dim]; the rotated key part of token t is in row cache_rows[t]
    const int* positions; const int* cache_rows; const int* q_start;
    void* kfull;             // [B * Wt, H, dn + rot_dim]: token at position p of sequence b in row b * Wt + p
    void* vfull;             // [B * Wt, H, dv]
    int B, Wt, H, dn, rot_dim, dv, kv_rank;
};

template <typename T>
__global__ void __launch_bounds__(128) latent_expand_kernel(LatentExpandArgs a) {
    const int t = blockIdx.x;
    int b = 0;
    while (b + 1 < a.B && a.q_start[b + 1] <= t) ++b;
    const size_t row = (size_t)b * a.Wt + a.positions[t];
    const int d = a.dn + a.rot_dim;
    const T* kn = static_cast<const T*>(a.kn) + (size_t)t * a.H * a.dn;
    const T* kr = static_cast<const T*>(a.ring) + (size_t)a.cache_rows[t] * (a.kv_rank + a.rot_dim) + a.kv_rank;
    T* kf = static_cast<T*>(a.kfull) + row * a.H * d;
    for (int i = threadIdx.x; i < a.H * d; i += blockDim.x) {
        const int h = i / d, c = i % d;
        kf[i] = c < a.dn ? kn[h * a.dn + c] : kr[c - a.dn];
    }
    const T* v = static_cast<const T*>(a.v) + (size_t)t * a.H * a.dv;
    T* vf = static_cast<T*>(a.vfull) + row * a.H * a.dv;
    for (int i = threadIdx.x; i < a.H * a.dv; i += blockDim.x) vf[i] = v[i];
}

// out[t, h, :] *= sigmoid(gate[t * g_pitch + g_off + h])
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ out, const T* __restrict__ gate, int g_pitch, int g_off, int H, int dv) {
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < H * dv; i += blockDim.x) {
        const float g = sigmoid_exact(to_f(gate[(size_t)t * g_pitch + g_off + i / dv]));
        out[(size_t)t * H * dv + i] = from_f<T>(to_f(out[(size_t)t * H * dv + i]) * g);
    }
}

}  // namespace mbh
