/*
 * Q / K preparation ahead of the append and the attention: per-head RMSNorm (optional weight),
 * interleaved-pair RoPE on the first n_rot dims, and for Q the split of the packed [q | gate]
 * projection.  Restates qsa_q_prep_k / qsa_k_prep_k (src/q4_rocm.cu:6229-6294) and their launchers
 * (:6296-6343): one block per (head, token), position = pos0 + t or the device position word + t.
 */
#include "q4_internal.h"

namespace {

__device__ __forceinline__ float block_sum_128(float v, float *sh) {
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    return sh[0] + sh[1] + sh[2] + sh[3];
}

/* src == dst is allowed (K is prepared in place). */
__device__ __forceinline__ void norm_rope(const float *src, float *dst, const float *wn, uint32_t hd,
                                          uint32_t n_rot, int32_t pos, float base, float eps, float *sh) {
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < hd; i += blockDim.x) ss += src[i] * src[i];
    ss = block_sum_128(ss, sh);
    const float scale = 1.0f / sqrtf(ss / (float)hd + eps);
    const uint32_t np = n_rot / 2;
    /* each thread normalises and rotates whole pairs, so in-place operation needs no barrier */
    for (uint32_t p = threadIdx.x; p < hd / 2; p += blockDim.x) {
        float x0 = src[2 * p] * scale * (wn ? wn[2 * p] : 1.f);
        float x1 = src[2 * p + 1] * scale * (wn ? wn[2 * p + 1] : 1.f);
        if (p < np) {
            const float freq = powf(base, -(float)p / (float)np);
            const float ang = (float)pos * freq;
            const float c = cosf(ang), si = sinf(ang);
            const float y0 = x0 * c - x1 * si, y1 = x0 * si + x1 * c;
            x0 = y0;
            x1 = y1;
        }
        dst[2 * p] = x0;
        dst[2 * p + 1] = x1;
    }
}

__global__ void q4_q_prep_k(const float *qg, const float *wn, float *q, float *g, uint32_t hd, uint32_t n_rot,
                            int32_t pos0, float base, float eps, uint32_t n_head, const int32_t *pp) {
    __shared__ float sh[4];
    const uint32_t h = blockIdx.x, t = blockIdx.y;
    const int32_t pos = (pp ? *pp : pos0) + (int32_t)t;
    const float *src = qg + ((size_t)t * n_head + h) * hd * 2;
    float *qd = q + ((size_t)t * n_head + h) * hd, *gd = g + ((size_t)t * n_head + h) * hd;
    for (uint32_t i = threadIdx.x; i < hd; i += blockDim.x) gd[i] = src[hd + i];
    norm_rope(src, qd, wn, hd, n_rot, pos, base, eps, sh);
}
__global__ void q4_k_prep_k(float *k, const float *wn, uint32_t hd, uint32_t n_rot, int32_t pos0, float base,
                            float eps, uint32_t n_kvh, const int32_t *pp) {
    __shared__ float sh[4];
    const uint32_t h = blockIdx.x, t = blockIdx.y;
    const int32_t pos = (pp ? *pp : pos0) + (int32_t)t;
    float *kh = k + ((size_t)t * n_kvh + h) * hd;
    norm_rope(kh, kh, wn, hd, n_rot, pos, base, eps, sh);
}

}  // namespace

extern "C" bool q4_hip_qsa_q_prep_n(const float *d_qg, const float *d_wn, float *d_q, float *d_g, uint32_t n_head,
                                    uint32_t hd, uint32_t n_rot, int32_t pos0, float base, float eps,
                                    uint32_t n_tok) {
    if (!g_q4.ok || !d_qg || !d_q || !d_g || n_head == 0 || n_tok == 0 || hd == 0 || (hd & 1) || n_rot > hd)
        return false;
    q4_q_prep_k<<<dim3(n_head, n_tok), 128, 0, g_q4.stream>>>(d_qg, d_wn, d_q, d_g, hd, n_rot, pos0, base, eps,
                                                             n_head, nullptr);
    return q4i_check(cudaGetLastError(), "q_prep launch");
}
extern "C" bool q4_hip_qsa_q_prep_d(const float *qg, const float *wn, float *q, float *g, uint32_t n_head,
                                    uint32_t hd, uint32_t n_rot, float base, float eps) {
    if (!g_q4.ok || !g_q4.pos_d || !qg || !q || !g || n_head == 0 || hd == 0 || (hd & 1) || n_rot > hd)
        return false;
    q4_q_prep_k<<<dim3(n_head, 1), 128, 0, g_q4.stream>>>(qg, wn, q, g, hd, n_rot, 0, base, eps, n_head,
                                                         g_q4.pos_d);
    return q4i_check(cudaGetLastError(), "q_prep_d launch");
}
extern "C" bool q4_hip_qsa_q_prep(const float *d_qg, const float *d_wn, float *d_q, float *d_g, uint32_t n_head,
                                  uint32_t hd, uint32_t n_rot, int32_t pos, float base, float eps) {
    return q4_hip_qsa_q_prep_n(d_qg, d_wn, d_q, d_g, n_head, hd, n_rot, pos, base, eps, 1);
}
extern "C" bool q4_hip_qsa_k_prep_n(float *d_k, const float *d_wn, uint32_t n_kvh, uint32_t hd, uint32_t n_rot,
                                    int32_t pos0, float base, float eps, uint32_t n_tok) {
    if (!g_q4.ok || !d_k || n_kvh == 0 || n_tok == 0 || hd == 0 || (hd & 1) || n_rot > hd) return false;
    q4_k_prep_k<<<dim3(n_kvh, n_tok), 128, 0, g_q4.stream>>>(d_k, d_wn, hd, n_rot, pos0, base, eps, n_kvh, nullptr);
    return q4i_check(cudaGetLastError(), "k_prep launch");
}
extern "C" bool q4_hip_qsa_k_prep_d(float *k, const float *wn, uint32_t n_kvh, uint32_t hd, uint32_t n_rot,
                                    float base, float eps) {
    if (!g_q4.ok || !g_q4.pos_d || !k || n_kvh == 0 || hd == 0 || (hd & 1) || n_rot > hd) return false;
    q4_k_prep_k<<<dim3(n_kvh, 1), 128, 0, g_q4.stream>>>(k, wn, hd, n_rot, 0, base, eps, n_kvh, g_q4.pos_d);
    return q4i_check(cudaGetLastError(), "k_prep_d launch");
}
extern "C" bool q4_hip_qsa_k_prep(float *d_k, const float *d_wn, uint32_t n_kvh, uint32_t hd, uint32_t n_rot,
                                  int32_t pos, float base, float eps) {
    return q4_hip_qsa_k_prep_n(d_k, d_wn, n_kvh, hd, n_rot, pos, base, eps, 1);
}
