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

/* ---- K prep fused into the append: RMSNorm + RoPE of the new K rows, q8_0 quantisation (or fp16 /
 * fp32 conversion) of K and V, and the scatter into the store, in one launch -- replaces
 * q4_hip_qsa_k_prep_d + q4_hip_kv_append_d (src/q4_fwd.c:884,891) and the prefill pair
 * q4_hip_qsa_k_prep_n + 2 x kv_write (:1734,1738-1741).  The normalised, rotated K row is built in
 * shared memory with exactly the arithmetic of q4_k_prep_k, then quantised with the append kernel's
 * arithmetic, so the cache bytes equal those of the two-launch sequence. */
namespace {

struct PrepAppendParams {
    Q4Cache C;
    int layout;
    uint32_t layer, n_kvh, hd, n_rot, n_tok;
    const float *k, *v, *wn;
    const int32_t *pos;      /* device position word or null */
    int32_t pos0;
    float base, eps;
    uint32_t *err;
};

__global__ void q4_prep_append_k(const PrepAppendParams P) {
    __shared__ float sh[4];
    __shared__ __align__(16) float row_s[256];
    const uint32_t kh = blockIdx.x, t = blockIdx.y;
    const bool which = blockIdx.z != 0;
    const int32_t pos = (P.pos ? *P.pos : P.pos0) + (int32_t)t;
    const float *src = (which ? P.v : P.k) + ((size_t)t * P.n_kvh + kh) * P.hd;
    if (!which) norm_rope(src, row_s, P.wn, P.hd, P.n_rot, pos, P.base, P.eps, sh);
    else for (uint32_t i = threadIdx.x; i < P.hd; i += blockDim.x) row_s[i] = src[i];
    __syncthreads();
    if (pos < 0 || (uint32_t)pos >= P.C.max_kv) {
        if (threadIdx.x == 0) atomicOr(P.err, (uint32_t)Q4E_RANGE);
        return;
    }
    /* 8 lanes per 32-value block, as the append kernel: hd / 4 lanes are busy */
    const uint32_t nb = P.hd / 32u, sub = threadIdx.x & 7u, b = threadIdx.x >> 3;
    const bool live = b < nb;
    const float4 x = live ? *reinterpret_cast<const float4 *>(row_s + b * 32 + sub * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    float d, id;
    q4d_block_scale(x, d, id);
    if (!live) return;
    uint8_t *row = const_cast<uint8_t *>(which ? P.C.v : P.C.k) + (uint64_t)P.layer * P.C.layer_stride +
                   (uint64_t)kh * P.C.kvh_stride + (uint64_t)pos * P.C.tok_stride;
    if (P.layout == LAY_Q8P) {
        *reinterpret_cast<uint32_t *>(row + b * 32 + sub * 4) = q4d_quant4(x, id);
        if (sub == 0) {
            uint8_t *srow = const_cast<uint8_t *>(P.C.s) + (uint64_t)P.layer * P.C.s_layer_stride +
                            (uint64_t)kh * P.C.s_kvh_stride + (uint64_t)pos * P.C.s_tok_stride;
            reinterpret_cast<__half *>(srow)[(which ? nb : 0u) + b] = __float2half_rn(d);
        }
    } else if (P.layout == LAY_F16) {
        __half2 *o = reinterpret_cast<__half2 *>(row + (b * 32 + sub * 4) * 2);
        o[0] = __floats2half2_rn(x.x, x.y);
        o[1] = __floats2half2_rn(x.z, x.w);
    } else {
        *reinterpret_cast<float4 *>(row + (b * 32 + sub * 4) * 4) = x;
    }
}

bool prep_append(q4_gpu_kv *kv, uint32_t layer, const float *k, const float *v, const float *wn, uint32_t n_rot,
                 float base, float eps, const int32_t *pos_dev, int32_t pos0, uint32_t n_tok) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "kv_prep_append: library not initialised");
    Q4_REQUIRE(kv && k && v && n_tok && layer < kv->n_layers && n_rot <= kv->hd && !(n_rot & 1), "kv_prep_append: bad argument");
    Q4_REQUIRE(pos_dev || (pos0 >= 0 && (uint64_t)pos0 + n_tok <= kv->max_kv), "kv_prep_append: rows beyond max_kv");
    PrepAppendParams p;
    p.C = kv->view;
    p.layout = kv->kind == Q4K_Q8 ? LAY_Q8P : kv->kind == Q4K_F16 ? LAY_F16 : LAY_F32;
    p.layer = layer; p.n_kvh = kv->n_kvh; p.hd = kv->hd; p.n_rot = n_rot; p.n_tok = n_tok;
    p.k = k; p.v = v; p.wn = wn; p.pos = pos_dev; p.pos0 = pos0; p.base = base; p.eps = eps; p.err = g_q4.err_d;
    q4_prep_append_k<<<dim3(kv->n_kvh, n_tok, 2), 128, 0, g_q4.stream>>>(p);
    return q4i_check(cudaGetLastError(), "kv_prep_append launch");
}

}  // namespace

extern "C" bool q4_gpu_kv_prep_append(q4_gpu_kv *kv, uint32_t layer, const float *k_raw, const float *v, const float *k_norm_w,
                                      uint32_t n_rot, float rope_base, float eps, uint32_t pos0, uint32_t n_tok) {
    return prep_append(kv, layer, k_raw, v, k_norm_w, n_rot, rope_base, eps, nullptr, (int32_t)pos0, n_tok);
}
extern "C" bool q4_gpu_kv_prep_append_d(q4_gpu_kv *kv, uint32_t layer, const float *k_raw, const float *v,
                                        const float *k_norm_w, uint32_t n_rot, float rope_base, float eps) {
    if (!g_q4.ok || !g_q4.pos_d) return q4i_fail(Q4E_INIT, "kv_prep_append_d: library not initialised");
    return prep_append(kv, layer, k_raw, v, k_norm_w, n_rot, rope_base, eps, g_q4.pos_d, 0, 1);
}
