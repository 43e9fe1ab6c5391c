// Latent attention: queries, keys and values are linear maps of small per-token latents, and the cache keeps one row per
// token, [c (kv_rank) | rotated key part (rot_dim)], shared by all heads.
//
//   latent_prep     from the packed input projection y = [W_dq h | W_dkv h | W_g h]: RMS norm of the query latent -> cq;
//                   RMS norm of the key/value latent c and the rotated shared key part -> the token's ring row
//   latent_absorb   per head: rotates the rotated part of q and folds the key up-projection into the query,
//                   qa = [W_uk[h]^T q_plain | rot(q_rot)], so that q.k = qa . [c | k_rot] and attention runs over the latent rows
//                   (attn_bias_kernel with one key/value head, key size kv_rank + rot_dim, value = the row's first kv_rank entries)
//   latent_vup      per head: out = W_uv[h] o_latent, times the sigmoid of the head's output-gate logit
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

// one CTA per (token, head); thread r owns latent columns r, r + blockDim, ...: W_uk[h] is read row by row, coalesced over r
template <typename T>
__global__ void __launch_bounds__(128) latent_absorb_kernel(LatentAbsorbArgs a) {
    extern __shared__ float qs[];  // [dn]
    const int t = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const T* q = static_cast<const T*>(a.q) + ((size_t)t * a.H + h) * (a.dn + a.rot_dim);
    T* qa = static_cast<T*>(a.qa) + ((size_t)t * a.H + h) * (a.kv_rank + a.rot_dim);
    for (int i = threadIdx.x; i < a.dn; i += blockDim.x) qs[i] = to_f(q[i]);
    __syncthreads();
    const T* W = static_cast<const T*>(a.w_uk) + (size_t)h * a.dn * a.kv_rank;
    for (int r = threadIdx.x; r < a.kv_rank; r += blockDim.x) {
        float acc = 0.f;
        for (int i = 0; i < a.dn; ++i) acc = fmaf(qs[i], to_f(W[(size_t)i * a.kv_rank + r]), acc);
        qa[r] = from_f<T>(acc);
    }
    const T* qr = q + a.dn;
    T* dr = qa + a.kv_rank;
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

// one CTA per (token, head); a warp per value column: dot product over the latent, lanes along it
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
    for (int j = warp; j < a.dv; j += nw) {
        const T* wr = W + (size_t)j * a.kv_rank;
        float acc = 0.f;
        for (int i = lane; i < a.kv_rank; i += 32) acc = fmaf(os[i], to_f(wr[i]), acc);
        acc = warp_sum(acc);
        if (lane == 0) out[j] = from_f<T>(rnd<T>(acc) * gate);
    }
}

}  // namespace mbh
