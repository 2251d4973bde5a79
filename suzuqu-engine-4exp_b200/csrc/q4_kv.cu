/*
 * KV store (allocator + record layout), the fused K/V append with q8_0 quantisation, conversion
 * to / from the reference layout, bulk prefix save / restore, and the host entry points of the
 * decode attention (reference ABI and store-based).
 *
 * Quantiser contract (f32_to_q8_k, src/q4_rocm.cu:7221-7238; kv_append_k, :7962-7999):
 *   amax = max |x| over 32 values; d = amax / 127.f; id = d > 0 ? 1.f / d : 0;
 *   code = clamp(rintf(x * id), -127, 127); scale = fp16(d) (round to nearest even)
 * evaluated in IEEE fp32 (explicit _rn intrinsics: no reciprocal-multiply rewrite, no FMA
 * contraction), so codes and scales are bit-exact with the C evaluation of that source.
 *
 * The work is 8 lanes per 32-value block: one 16-byte load per lane, amax by three shuffles, one
 * 4-byte store of codes per lane -- rows are read and written fully coalesced.
 */
#include <stdlib.h>
#include <string.h>

#include "q4_internal.h"

namespace {

struct AppendParams {
    Q4Cache one;
    const Q4Cache *many;          /* one cache view per row (batched sessions), device array */
    uint32_t layer, n_rows, n_kvh, hd;
    const float *k, *v;           /* [n_rows][n_kvh*hd] */
    const int32_t *pos;           /* device positions (per row if many, else one word) or null */
    uint32_t pos0;
    uint32_t *err;
};

__device__ __forceinline__ float4 load4(const float *p, bool aligned) {
    if (aligned) return *reinterpret_cast<const float4 *>(p);
    return make_float4(p[0], p[1], p[2], p[3]);
}

/* n floats -> n/32 reference blocks {fp16 scale, 32 x int8} at dst (2-byte aligned stores). */
__global__ void q4_f32_to_q8_k(const float *src, uint8_t *dst, uint64_t nblocks, bool aligned) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t b = i >> 3;
    const uint32_t sub = (uint32_t)i & 7u;
    const bool live = b < nblocks;
    const float4 x = live ? load4(src + b * 32 + sub * 4, aligned) : make_float4(0.f, 0.f, 0.f, 0.f);
    float d, id;
    q4d_block_scale(x, d, id);
    if (!live) return;
    const uint32_t c = q4d_quant4(x, id);
    uint8_t *o = dst + b * 34;
    if (sub == 0) *reinterpret_cast<__half *>(o) = __float2half_rn(d);
    uint16_t *cp = reinterpret_cast<uint16_t *>(o + 2 + sub * 4);
    cp[0] = (uint16_t)(c & 0xffffu);
    cp[1] = (uint16_t)(c >> 16);
}

__global__ void q4_f32_to_f16_k(const float *src, __half *dst, uint64_t n, const int32_t *pos,
                                uint32_t stride) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (pos) dst += (size_t)(uint32_t)*pos * stride;
    if (i < n) dst[i] = __float2half_rn(src[i]);
}

/* fp16 / fp32 rows of any length and alignment at the slot held in the device position word (the
 * reference's kv_append_k takes any n for these kinds, src/q4_rocm.cu:7986-7999): one element per
 * thread, blockIdx.y: 0 = K, 1 = V. */
template <bool F16>
__global__ void q4_append_flat_k(uint8_t *kc, uint8_t *vc, const float *k, const float *v, uint32_t n, uint32_t bpt,
                                 const int32_t *pos) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint8_t *row = (blockIdx.y ? vc : kc) + (uint64_t)(uint32_t)*pos * bpt;
    const float x = (blockIdx.y ? v : k)[i];
    if (F16) reinterpret_cast<__half *>(row)[i] = __float2half_rn(x);
    else reinterpret_cast<float *>(row)[i] = x;
}

/* Fused K+V append into a cache view.  blockIdx.y: 0 = K, 1 = V.  8 lanes per 32 values. */
template <int LAY>
__global__ void q4_append_k(const AppendParams P) {
    const uint32_t nb = P.hd / 32u;
    const uint32_t per_row = P.n_kvh * nb * 8u;
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t r = (uint32_t)(i / per_row);
    const uint32_t w = (uint32_t)(i % per_row);
    const uint32_t sub = w & 7u, blk = w >> 3, kh = blk / nb, b = blk % nb;
    const bool which = blockIdx.y != 0;
    bool live = r < P.n_rows;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) x = *reinterpret_cast<const float4 *>((which ? P.v : P.k) + (size_t)r * P.n_kvh * P.hd +
                                                     (size_t)blk * 32 + sub * 4);
    float d = 0.f, id = 0.f;
    if (LAY == LAY_Q8P || LAY == LAY_Q8R) q4d_block_scale(x, d, id);
    if (!live) return;
    const Q4Cache C = P.many ? P.many[r] : P.one;
    const uint32_t p = P.pos ? (uint32_t)P.pos[P.many ? r : 0] + (P.many ? 0u : r) : P.pos0 + r;
    if (p >= C.max_kv) {
        if (w == 0) atomicOr(P.err, (uint32_t)Q4E_RANGE);
        return;
    }
    uint8_t *row = const_cast<uint8_t *>(which ? C.v : C.k) + (uint64_t)P.layer * C.layer_stride +
                   (uint64_t)kh * C.kvh_stride + (uint64_t)p * C.tok_stride;
    if (LAY == LAY_Q8P) {
        *reinterpret_cast<uint32_t *>(row + b * 32 + sub * 4) = q4d_quant4(x, id);
        if (sub == 0) {
            uint8_t *srow = const_cast<uint8_t *>(C.s) + (uint64_t)P.layer * C.s_layer_stride +
                            (uint64_t)kh * C.s_kvh_stride + (uint64_t)p * C.s_tok_stride;
            reinterpret_cast<__half *>(srow)[(which ? nb : 0u) + b] = __float2half_rn(d);
        }
    } else if (LAY == LAY_Q8R) {
        const uint32_t c = q4d_quant4(x, id);
        uint8_t *o = row + b * 34;
        if (sub == 0) *reinterpret_cast<__half *>(o) = __float2half_rn(d);
        uint16_t *cp = reinterpret_cast<uint16_t *>(o + 2 + sub * 4);
        cp[0] = (uint16_t)(c & 0xffffu);
        cp[1] = (uint16_t)(c >> 16);
    } else if (LAY == LAY_F16) {
        __half2 *o = reinterpret_cast<__half2 *>(row + (b * 32 + sub * 4) * 2);
        o[0] = __floats2half2_rn(x.x, x.y);
        o[1] = __floats2half2_rn(x.z, x.w);
    } else {
        *reinterpret_cast<float4 *>(row + (b * 32 + sub * 4) * 4) = x;
    }
}

/* Planar store <-> reference layout, rows [tok0, tok0+n_tok) of one plane.  Bytes only. */
template <int LAY, bool TO_REF>
__global__ void q4_relayout_k(Q4Cache C, uint32_t layer, int which, uint32_t n_kvh, uint32_t hd,
                              uint32_t tok0, uint32_t n_tok, uint8_t *ref) {
    const uint32_t nb = hd / 32u;
    const uint32_t per_row = n_kvh * nb * 8u;
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t r = (uint32_t)(i / per_row);
    if (r >= n_tok) return;
    const uint32_t w = (uint32_t)(i % per_row);
    const uint32_t sub = w & 7u, blk = w >> 3, kh = blk / nb, b = blk % nb;
    uint8_t *row = const_cast<uint8_t *>(which ? C.v : C.k) + (uint64_t)layer * C.layer_stride +
                   (uint64_t)kh * C.kvh_stride + (uint64_t)(tok0 + r) * C.tok_stride;
    if (LAY == LAY_Q8P) {
        uint8_t *o = ref + (((size_t)r * n_kvh + kh) * nb + b) * 34;
        __half *sc = reinterpret_cast<__half *>(const_cast<uint8_t *>(C.s) + (uint64_t)layer * C.s_layer_stride +
                                                (uint64_t)kh * C.s_kvh_stride +
                                                (uint64_t)(tok0 + r) * C.s_tok_stride) +
                     (which ? nb : 0u) + b;
        uint32_t *cw = reinterpret_cast<uint32_t *>(row + b * 32 + sub * 4);
        uint16_t *cp = reinterpret_cast<uint16_t *>(o + 2 + sub * 4);
        if (TO_REF) {
            const uint32_t c = *cw;
            cp[0] = (uint16_t)(c & 0xffffu);
            cp[1] = (uint16_t)(c >> 16);
            if (sub == 0) *reinterpret_cast<__half *>(o) = *sc;
        } else {
            *cw = (uint32_t)cp[0] | ((uint32_t)cp[1] << 16);
            if (sub == 0) *sc = *reinterpret_cast<__half *>(o);
        }
    } else {
        const uint32_t es = LAY == LAY_F16 ? 2u : 4u;
        uint8_t *o = ref + (((size_t)r * n_kvh + kh) * hd + b * 32 + sub * 4) * es;
        uint8_t *s = row + (b * 32 + sub * 4) * es;
        if (LAY == LAY_F16) {
            if (TO_REF) *reinterpret_cast<uint2 *>(o) = *reinterpret_cast<uint2 *>(s);
            else *reinterpret_cast<uint2 *>(s) = *reinterpret_cast<uint2 *>(o);
        } else {
            if (TO_REF) *reinterpret_cast<uint4 *>(o) = *reinterpret_cast<uint4 *>(s);
            else *reinterpret_cast<uint4 *>(s) = *reinterpret_cast<uint4 *>(o);
        }
    }
}
/* 32-byte aligned records (288 B) were measured: no faster than 16-byte alignment (272 B) */
inline uint32_t q8_record_bytes(uint32_t hd) { return (2u * hd + hd / 8u + 15u) & ~15u; }   /* 272 at hd 128 */
inline uint32_t row_bytes(uint32_t hd, int kind) {
    return kind == Q4K_Q8 ? hd : hd * (kind == Q4K_F16 ? 2u : 4u);   /* q8_0: the code part of a record */
}
inline int store_layout(int kind) { return kind == Q4K_Q8 ? LAY_Q8P : kind == Q4K_F16 ? LAY_F16 : LAY_F32; }
inline bool hd_ok(uint32_t hd) { return hd == 32 || hd == 64 || hd == 128 || hd == 256; }

/* A caller-owned cache in the reference layout (src/q4_fwd.c:644-655) as a kernel view. */
Q4Cache ref_view(const void *kc, const void *vc, uint32_t n_kvh, uint32_t hd, uint32_t max_kv, int kind) {
    Q4Cache c;
    memset(&c, 0, sizeof(c));
    const uint32_t rb = kind == Q4K_Q8 ? (hd / 32u) * 34u : hd * (kind == Q4K_F16 ? 2u : 4u);
    c.k = (const uint8_t *)kc;
    c.v = (const uint8_t *)vc;
    c.kvh_stride = rb;
    c.tok_stride = n_kvh * rb;
    c.max_kv = max_kv;
    return c;
}
inline int ref_layout(int kind) { return kind == Q4K_Q8 ? LAY_Q8R : kind == Q4K_F16 ? LAY_F16 : LAY_F32; }

bool launch_append(const AppendParams &p, int layout) {
    const uint64_t threads = (uint64_t)p.n_rows * p.n_kvh * (p.hd / 32u) * 8u;
    dim3 grid((unsigned)((threads + 255) / 256), 2);
    switch (layout) {
    case LAY_Q8P: q4_append_k<LAY_Q8P><<<grid, 256, 0, g_q4.stream>>>(p); break;
    case LAY_Q8R: q4_append_k<LAY_Q8R><<<grid, 256, 0, g_q4.stream>>>(p); break;
    case LAY_F16: q4_append_k<LAY_F16><<<grid, 256, 0, g_q4.stream>>>(p); break;
    default: q4_append_k<LAY_F32><<<grid, 256, 0, g_q4.stream>>>(p); break;
    }
    return q4i_check(cudaGetLastError(), "append launch");
}

}  // namespace

/* ======================================================================= reference ABI ===== */

extern "C" bool q4_hip_f32_to_q8(void *dst_q8, const float *src, uint64_t n) {
    if (!g_q4.ok || !dst_q8 || !src || n == 0 || (n % 32u) != 0) return false;
    const uint64_t nb = n / 32u;
    const uint64_t threads = nb * 8u;
    q4_f32_to_q8_k<<<(unsigned)((threads + 255) / 256), 256, 0, g_q4.stream>>>(
        src, (uint8_t *)dst_q8, nb, ((uintptr_t)src & 15u) == 0);
    return q4i_check(cudaGetLastError(), "f32_to_q8 launch");
}
extern "C" bool q4_hip_f32_to_f16(void *dst_f16, const float *src, uint64_t n) {
    if (!g_q4.ok || !dst_f16 || !src || !n) return false;
    q4_f32_to_f16_k<<<(unsigned)((n + 255) / 256), 256, 0, g_q4.stream>>>(src, (__half *)dst_f16, n, nullptr, 0);
    return q4i_check(cudaGetLastError(), "f32_to_f16 launch");
}
extern "C" bool q4_hip_f32_to_f16_d(void *dst_base, uint32_t stride_elems, const float *src, uint64_t n) {
    if (!g_q4.ok || !g_q4.pos_d || !dst_base || !src || !n) return false;
    q4_f32_to_f16_k<<<(unsigned)((n + 255) / 256), 256, 0, g_q4.stream>>>(src, (__half *)dst_base, n,
                                                                         g_q4.pos_d, stride_elems);
    return q4i_check(cudaGetLastError(), "f32_to_f16_d launch");
}
/* The reference treats the token row as n flat floats at cache + pos*bpt; as a view that is one
 * kv head of width n. */
extern "C" bool q4_hip_kv_append_d(void *kcache, void *vcache, const float *k, const float *v, uint32_t n,
                                   uint32_t bpt, int kind) {
    if (!g_q4.ok || !g_q4.pos_d || !kcache || !vcache || !k || !v || !n || !bpt) return false;
    if (kind < 0 || kind > 2) return false;
    if (kind == Q4K_Q8 && (n % 32u)) return false;   /* whole q8_0 blocks only, as the reference (:8003-8006) */
    const bool vec_ok = (n % 32u) == 0 && (((uintptr_t)k | (uintptr_t)v) & 15u) == 0 &&
                        (kind == Q4K_Q8 || ((((uintptr_t)kcache | (uintptr_t)vcache | bpt) & 15u) == 0));
    if (!vec_ok) {
        if (kind == Q4K_Q8) return q4i_fail(Q4E_ARG, "kv_append_d: q8_0 rows need 16-byte aligned fp32 sources");
        dim3 grid((n + 255u) / 256u, 2);
        if (kind == Q4K_F16)
            q4_append_flat_k<true><<<grid, 256, 0, g_q4.stream>>>((uint8_t *)kcache, (uint8_t *)vcache, k, v, n, bpt, g_q4.pos_d);
        else
            q4_append_flat_k<false><<<grid, 256, 0, g_q4.stream>>>((uint8_t *)kcache, (uint8_t *)vcache, k, v, n, bpt, g_q4.pos_d);
        return q4i_check(cudaGetLastError(), "kv_append_d launch");
    }
    AppendParams p;
    memset(&p, 0, sizeof(p));
    p.one.k = (const uint8_t *)kcache;
    p.one.v = (const uint8_t *)vcache;
    p.one.tok_stride = bpt;
    p.one.max_kv = 0xffffffffu;
    p.n_rows = 1;
    p.n_kvh = 1;
    p.hd = n;
    p.k = k;
    p.v = v;
    p.pos = g_q4.pos_d;
    p.err = g_q4.err_d;
    return launch_append(p, ref_layout(kind));
}

static bool legacy_decode(const float *q, const void *kc, const void *vc, const float *gate, float *out,
                          const int32_t *idx, uint32_t width, uint32_t n_head, uint32_t n_kvh, uint32_t hd,
                          uint32_t n_tok, uint32_t kv_base, uint32_t max_kv, float scale, int kind) {
    if (!g_q4.ok || !q || !kc || !vc || !gate || !out) return false;   /* NULL gate is rejected: :7254,7312 */
    if (n_tok == 0 || hd == 0 || hd > 256 || n_head == 0 || n_kvh == 0) return false;
    if (!hd_ok(hd) || kind < 0 || kind > 2) return q4i_fail(Q4E_ARG, "decode: unsupported hd or kind");
    Q4DecodeArgs a;
    memset(&a, 0, sizeof(a));
    a.one = ref_view(kc, vc, n_kvh, hd, max_kv, kind);
    a.layout = ref_layout(kind);
    a.n_units = n_tok;
    a.n_head = n_head;
    a.n_kvh = n_kvh;
    a.hd = hd;
    a.q = q;
    a.gate = gate;
    a.out = out;
    a.idx = idx;
    a.width = width;
    a.idx_unit_stride = width;
    a.kv_base = kv_base;
    uint32_t rows = kv_base + n_tok;
    a.hint_rows = rows < max_kv ? rows : max_kv;
    a.scale = scale;
    return q4i_decode(a);
}
extern "C" bool q4_hip_qsa_decode_n(const float *d_q, const void *d_kcache, const void *d_vcache,
                                    const float *d_gate, float *d_out, uint32_t n_head, uint32_t n_kvh,
                                    uint32_t hd, uint32_t n_tok, uint32_t kv_base, uint32_t max_kv,
                                    float scale, int kv_f16) {
    return legacy_decode(d_q, d_kcache, d_vcache, d_gate, d_out, nullptr, 0, n_head, n_kvh, hd, n_tok,
                         kv_base, max_kv, scale, kv_f16);
}
extern "C" bool q4_hip_qsa_decode(const float *d_q, const void *d_kcache, const void *d_vcache,
                                  const float *d_gate, float *d_out, uint32_t n_head, uint32_t n_kvh,
                                  uint32_t hd, uint32_t n_kv, uint32_t max_kv, float scale, int kv_f16) {
    if (n_kv == 0) return false;
    return q4_hip_qsa_decode_n(d_q, d_kcache, d_vcache, d_gate, d_out, n_head, n_kvh, hd, 1, n_kv - 1,
                               max_kv, scale, kv_f16);
}
extern "C" bool q4_hip_qsa_decode_idx(const float *d_q, const void *d_kcache, const void *d_vcache,
                                      const float *d_gate, float *d_out, const int32_t *idx, uint32_t width,
                                      uint32_t n_head, uint32_t n_kvh, uint32_t hd, uint32_t n_tok,
                                      uint32_t max_kv, float scale, int kv_f16) {
    if (!idx || width == 0) return false;
    return legacy_decode(d_q, d_kcache, d_vcache, d_gate, d_out, idx, width, n_head, n_kvh, hd, n_tok, 0,
                         max_kv, scale, kv_f16);
}

/* ======================================================================= KV store ========== */

extern "C" uint64_t q4_gpu_kv_bytes(uint32_t n_layers, uint32_t n_kvh, uint32_t hd, uint32_t max_kv, int kind) {
    /* The bytes q4_gpu_kv_create allocates for the planes.  q8_0: one record per (kv head, position) of
     * 2*hd codes + 2*hd/32 fp16 scales, padded to a multiple of 16 bytes: at hd 128 and 256 that is
     * exactly the reference's K+V total (q4_qsa_kv_bytes, src/q4_place.c:92-105: 2 x (hd/32) x 34 per
     * row); at hd 32 / 64 the padding adds 12 / 8 bytes per record (80 vs 68, 144 vs 136). */
    if (kind == Q4K_Q8) return (uint64_t)n_layers * max_kv * n_kvh * q8_record_bytes(hd);
    return (uint64_t)n_layers * max_kv * 2ull * n_kvh * hd * (kind == Q4K_F16 ? 2u : 4u);
}

extern "C" q4_gpu_kv *q4_gpu_kv_create(uint32_t n_layers, uint32_t n_kvh, uint32_t hd, uint32_t max_kv, int kind) {
    if (!g_q4.ok) { q4i_fail(Q4E_INIT, "kv_create: library not initialised"); return nullptr; }
    if (!n_layers || !n_kvh || !hd_ok(hd) || !max_kv || kind < 0 || kind > 2) {
        q4i_fail(Q4E_ARG, "kv_create: bad shape");
        return nullptr;
    }
    q4_gpu_kv *kv = (q4_gpu_kv *)calloc(1, sizeof(q4_gpu_kv));
    if (!kv) return nullptr;
    kv->n_layers = n_layers; kv->n_kvh = n_kvh; kv->hd = hd; kv->max_kv = max_kv; kv->kind = kind;
    /* q8_0: one record per (kv head, position) = K codes | V codes | K scales | V scales, so a gathered
     * position is one contiguous 272-byte read (hd 128) instead of three scattered ones.  fp16 / fp32:
     * a K plane and a V plane of [kv head][position][hd] rows. */
    const uint32_t rb = kind == Q4K_Q8 ? q8_record_bytes(hd) : row_bytes(hd, kind);
    kv->rec_bytes = rb;
    kv->plane_bytes = (uint64_t)n_layers * n_kvh * max_kv * rb;
    kv->s_bytes = 0;
    bool ok = cudaMalloc(&kv->k, kv->plane_bytes) == cudaSuccess;
    if (ok && kind == Q4K_Q8) {
        kv->v = kv->k + hd;
        kv->s = kv->k + 2 * hd;
    } else if (ok) {
        ok = cudaMalloc(&kv->v, kv->plane_bytes) == cudaSuccess;
    }
    if (ok) ok = cudaMalloc(&kv->d_view, sizeof(Q4Cache)) == cudaSuccess;
    if (!ok) {
        (void)cudaGetLastError();
        q4i_fail(Q4E_CUDA, "kv_create: device allocation failed");
        q4_gpu_kv_destroy(kv);
        return nullptr;
    }
    Q4Cache &c = kv->view;
    c.k = kv->k; c.v = kv->v; c.s = kv->s;
    c.tok_stride = rb;
    c.kvh_stride = (uint64_t)max_kv * rb;
    c.layer_stride = (uint64_t)n_kvh * max_kv * rb;
    c.s_tok_stride = rb;                      /* the scales ride in the same record */
    c.s_kvh_stride = c.kvh_stride;
    c.s_layer_stride = c.layer_stride;
    c.max_kv = max_kv;
    if (cudaMemcpy(kv->d_view, &c, sizeof(c), cudaMemcpyHostToDevice) != cudaSuccess) {
        q4i_fail(Q4E_CUDA, "kv_create: view upload failed");
        q4_gpu_kv_destroy(kv);
        return nullptr;
    }
    return kv;
}
extern "C" void q4_gpu_kv_destroy(q4_gpu_kv *kv) {
    if (!kv) return;
    if (kv->k) cudaFree(kv->k);
    if (kv->v && kv->kind != Q4K_Q8) cudaFree(kv->v);   /* q8_0: v and s point into the k allocation */
    if (kv->d_view) cudaFree(kv->d_view);
    free(kv);
}

extern "C" bool q4_gpu_kv_append(q4_gpu_kv *kv, uint32_t layer, const float *k, const float *v, uint32_t pos0,
                                 uint32_t n_tok) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "kv_append: library not initialised");
    Q4_REQUIRE(kv && k && v && n_tok && layer < kv->n_layers, "kv_append: bad argument");
    Q4_REQUIRE((uint64_t)pos0 + n_tok <= kv->max_kv, "kv_append: rows beyond max_kv");
    AppendParams p;
    memset(&p, 0, sizeof(p));
    p.one = kv->view; p.layer = layer; p.n_rows = n_tok; p.n_kvh = kv->n_kvh; p.hd = kv->hd;
    p.k = k; p.v = v; p.pos0 = pos0; p.err = g_q4.err_d;
    return launch_append(p, store_layout(kv->kind));
}
extern "C" bool q4_gpu_kv_append_d(q4_gpu_kv *kv, uint32_t layer, const float *k, const float *v) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "kv_append_d: library not initialised");
    Q4_REQUIRE(kv && k && v && layer < kv->n_layers, "kv_append_d: bad argument");
    AppendParams p;
    memset(&p, 0, sizeof(p));
    p.one = kv->view; p.layer = layer; p.n_rows = 1; p.n_kvh = kv->n_kvh; p.hd = kv->hd;
    p.k = k; p.v = v; p.pos = g_q4.pos_d; p.err = g_q4.err_d;
    return launch_append(p, store_layout(kv->kind));
}

template <bool TO_REF>
static bool relayout(const q4_gpu_kv *kv, uint32_t layer, int which, uint32_t tok0, uint32_t n_tok, void *ref) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "kv relayout: library not initialised");
    Q4_REQUIRE(kv && ref && n_tok && layer < kv->n_layers && (which == 0 || which == 1), "kv relayout: bad argument");
    Q4_REQUIRE((uint64_t)tok0 + n_tok <= kv->max_kv, "kv relayout: rows beyond max_kv");
    const uint64_t threads = (uint64_t)n_tok * kv->n_kvh * (kv->hd / 32u) * 8u;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    switch (kv->kind) {
    case Q4K_Q8:
        q4_relayout_k<LAY_Q8P, TO_REF><<<grid, 256, 0, g_q4.stream>>>(kv->view, layer, which, kv->n_kvh, kv->hd, tok0, n_tok, (uint8_t *)ref);
        break;
    case Q4K_F16:
        q4_relayout_k<LAY_F16, TO_REF><<<grid, 256, 0, g_q4.stream>>>(kv->view, layer, which, kv->n_kvh, kv->hd, tok0, n_tok, (uint8_t *)ref);
        break;
    default:
        q4_relayout_k<LAY_F32, TO_REF><<<grid, 256, 0, g_q4.stream>>>(kv->view, layer, which, kv->n_kvh, kv->hd, tok0, n_tok, (uint8_t *)ref);
        break;
    }
    return q4i_check(cudaGetLastError(), "kv relayout launch");
}
extern "C" bool q4_gpu_kv_export(const q4_gpu_kv *kv, uint32_t layer, int which, uint32_t tok0, uint32_t n_tok, void *dst) {
    return relayout<true>(kv, layer, which, tok0, n_tok, dst);
}
extern "C" bool q4_gpu_kv_import(q4_gpu_kv *kv, uint32_t layer, int which, uint32_t tok0, uint32_t n_tok, const void *src) {
    return relayout<false>(kv, layer, which, tok0, n_tok, const_cast<void *>(src));
}

/* Prefix snapshot = records [0, n_kv) of every (layer, kv head): one strided bulk copy for q8_0 (two
 * for the fp16 / fp32 kinds' K and V planes); pitch = max_kv rows, width = n_kv rows. */
extern "C" uint64_t q4_gpu_kv_snapshot_bytes(const q4_gpu_kv *kv, uint32_t n_kv) {
    if (!kv) return 0;
    const uint64_t rows = (uint64_t)kv->n_layers * kv->n_kvh * n_kv;
    return rows * (kv->kind == Q4K_Q8 ? (uint64_t)kv->rec_bytes : 2ull * row_bytes(kv->hd, kv->kind));
}
/* Device-to-device prefix copy: `height` rows of `width16` 16-byte words, source and destination
 * pitches in bytes.  A block moves 32 KB of one row, eight independent 16-byte loads per thread in
 * flight before the first store, streaming cache hints both ways (nothing is re-read).  Measured at
 * 431 MB: 2-D copy engine path 3.5 TB/s (read + write), this kernel below. */
constexpr uint32_t SNAP_TILE_WORDS = 2048;
static __global__ void __launch_bounds__(256) q4_snap_copy_k(uint8_t *dst, size_t dpitch, const uint8_t *src, size_t spitch,
                                                      size_t width16, uint32_t tiles_per_row) {
    const uint32_t row = blockIdx.x / tiles_per_row, tile = blockIdx.x % tiles_per_row;
    const uint4 *s = reinterpret_cast<const uint4 *>(src + (size_t)row * spitch);
    uint4 *d = reinterpret_cast<uint4 *>(dst + (size_t)row * dpitch);
    const size_t base = (size_t)tile * SNAP_TILE_WORDS + threadIdx.x;
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; i++)
        if (base + i * 256 < width16) v[i] = __ldcs(s + base + i * 256);
#pragma unroll
    for (int i = 0; i < 8; i++)
        if (base + i * 256 < width16) __stcs(d + base + i * 256, v[i]);
}

static bool snapshot(const q4_gpu_kv *kv, uint32_t n_kv, void *buf, int host, bool save) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "kv snapshot: library not initialised");
    Q4_REQUIRE(kv && buf && n_kv && n_kv <= kv->max_kv, "kv snapshot: bad argument");
    const size_t height = (size_t)kv->n_layers * kv->n_kvh;
    const uint32_t rb = kv->rec_bytes;
    uint8_t *b = (uint8_t *)buf;
    const cudaMemcpyKind kind = !host ? cudaMemcpyDeviceToDevice : save ? cudaMemcpyDeviceToHost : cudaMemcpyHostToDevice;
    struct { uint8_t *plane; uint32_t row; } pl[2] = {{kv->k, rb}, {kv->v, rb}};
    for (int i = 0; i < (kv->kind == Q4K_Q8 ? 1 : 2); i++) {
        const size_t width = (size_t)n_kv * pl[i].row, pitch = (size_t)kv->max_kv * pl[i].row;
        if (!host && width % 16 == 0 && pitch % 16 == 0 && ((uintptr_t)b & 15u) == 0) {
            const size_t width16 = width / 16;
            const uint32_t tiles = (uint32_t)((width16 + SNAP_TILE_WORDS - 1) / SNAP_TILE_WORDS);
            const uint32_t grid = tiles * (uint32_t)height;
            if (save) q4_snap_copy_k<<<grid, 256, 0, g_q4.stream>>>(b, width, pl[i].plane, pitch, width16, tiles);
            else q4_snap_copy_k<<<grid, 256, 0, g_q4.stream>>>(pl[i].plane, pitch, b, width, width16, tiles);
            if (!q4i_check(cudaGetLastError(), "kv snapshot copy kernel")) return false;
        } else {
            cudaError_t e = save ? cudaMemcpy2DAsync(b, width, pl[i].plane, pitch, width, height, kind, g_q4.stream)
                                 : cudaMemcpy2DAsync(pl[i].plane, pitch, b, width, width, height, kind, g_q4.stream);
            if (!q4i_check(e, "kv snapshot copy")) return false;
        }
        b += width * height;
    }
    return true;
}
extern "C" bool q4_gpu_kv_save(const q4_gpu_kv *kv, uint32_t n_kv, void *buf, int host) {
    return snapshot(kv, n_kv, buf, host, true);
}
extern "C" bool q4_gpu_kv_restore(q4_gpu_kv *kv, uint32_t n_kv, const void *buf, int host) {
    return snapshot(kv, n_kv, const_cast<void *>(buf), host, false);
}

static bool store_decode(const q4_gpu_kv *kv, uint32_t layer, const void *q, int q_bf16, const float *gate,
                         float *out, float *part, uint32_t n_head, const int32_t *idx, uint32_t width,
                         uint32_t idx_kvh_stride, uint32_t n_kv, float scale) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "kv_decode: library not initialised");
    Q4_REQUIRE(kv && q && (out || part) && layer < kv->n_layers && n_head, "kv_decode: bad argument");
    Q4_REQUIRE(n_kv <= kv->max_kv, "kv_decode: n_kv beyond max_kv");
    Q4DecodeArgs a;
    memset(&a, 0, sizeof(a));
    a.one = kv->view;
    a.layout = store_layout(kv->kind);
    a.layer = layer;
    a.n_units = 1;
    a.n_head = n_head;
    a.n_kvh = kv->n_kvh;
    a.hd = kv->hd;
    a.q = q;
    a.q_bf16 = q_bf16;
    a.gate = gate;
    a.out = out;
    a.part_out = part;
    a.idx = idx;
    a.width = width;
    a.idx_kvh_stride = idx_kvh_stride;
    if (n_kv) {
        a.kv_base = n_kv - 1;
        a.hint_rows = n_kv;
    } else {
        a.pos = g_q4.pos_d;          /* rows = device position word + 1 */
        a.hint_rows = kv->max_kv;
    }
    a.idx_bound_nkv = 1;
    a.scale = scale;
    return q4i_decode(a);
}
extern "C" bool q4_gpu_kv_decode(const q4_gpu_kv *kv, uint32_t layer, const void *q, int q_bf16, const float *gate,
                                 float *out, uint32_t n_head, const int32_t *idx, uint32_t width,
                                 uint32_t idx_kvh_stride, uint32_t n_kv, float scale) {
    return store_decode(kv, layer, q, q_bf16, gate, out, nullptr, n_head, idx, width, idx_kvh_stride, n_kv, scale);
}
extern "C" bool q4_gpu_kv_decode_partial(const q4_gpu_kv *kv, uint32_t layer, const void *q, int q_bf16, float *part,
                                         uint32_t n_head, const int32_t *idx, uint32_t width,
                                         uint32_t idx_kvh_stride, uint32_t n_kv, float scale) {
    return store_decode(kv, layer, q, q_bf16, nullptr, nullptr, part, n_head, idx, width, idx_kvh_stride, n_kv, scale);
}
/* Sparse prefill on the store: the n_tok > 1 form of q4_hip_qsa_decode_idx (gqa_prefill_k<KIND, true>,
 * src/q4_rocm.cu:7319,7342-7357).  Query t attends the rows its own list names; the work is a gather,
 * not a contraction, so it runs as one launch of the decode kernel with a unit per (token, kv head). */
extern "C" bool q4_gpu_kv_decode_idx_n(const q4_gpu_kv *kv, uint32_t layer, const void *q, int q_bf16,
                                       const float *gate, float *out, uint32_t n_head, const int32_t *idx,
                                       uint32_t width, uint32_t idx_kvh_stride, uint32_t idx_tok_stride,
                                       uint32_t n_tok, float scale) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "kv_decode_idx_n: library not initialised");
    Q4_REQUIRE(kv && q && out && idx && width && n_tok && layer < kv->n_layers && n_head,
               "kv_decode_idx_n: bad argument");
    Q4_REQUIRE(idx_tok_stride >= width, "kv_decode_idx_n: lists of consecutive tokens overlap");
    Q4DecodeArgs a;
    memset(&a, 0, sizeof(a));
    a.one = kv->view;
    a.layout = store_layout(kv->kind);
    a.layer = layer;
    a.n_units = n_tok;
    a.n_head = n_head;
    a.n_kvh = kv->n_kvh;
    a.hd = kv->hd;
    a.q = q;
    a.q_bf16 = q_bf16;
    a.gate = gate;
    a.out = out;
    a.idx = idx;
    a.width = width;
    a.idx_kvh_stride = idx_kvh_stride;
    a.idx_unit_stride = idx_tok_stride;
    /* the lists alone bound the rows: entries >= max_kv are skipped and raise the range status bit */
    a.hint_rows = width;
    a.scale = scale;
    return q4i_decode(a);
}

/* ======================================================================= batch ============= */

struct q4_gpu_batch {
    uint32_t max_sessions, n;
    uint32_t n_active;            /* sessions of the latest q4_gpu_batch_set_pos: what every batch launch covers */
    q4_gpu_kv **kv;
    Q4Cache *d_views;             /* device array of the bound stores' views (one load, no pointer chase) */
    int32_t *pos_d, *pos_h;       /* pos_h: pinned ring of 8 uploads, each slot guarded by an event */
    cudaEvent_t pos_ev[8];
    uint32_t ring, max_pos;
};

extern "C" q4_gpu_batch *q4_gpu_batch_create(uint32_t max_sessions) {
    if (!g_q4.ok || !max_sessions) { q4i_fail(Q4E_ARG, "batch_create: bad argument"); return nullptr; }
    q4_gpu_batch *b = (q4_gpu_batch *)calloc(1, sizeof(q4_gpu_batch));
    if (!b) return nullptr;
    b->max_sessions = max_sessions;
    b->kv = (q4_gpu_kv **)calloc(max_sessions, sizeof(q4_gpu_kv *));
    bool ok = b->kv && cudaMalloc(&b->d_views, sizeof(Q4Cache) * max_sessions) == cudaSuccess &&
              cudaMalloc(&b->pos_d, sizeof(int32_t) * max_sessions) == cudaSuccess &&
              cudaMallocHost(&b->pos_h, sizeof(int32_t) * max_sessions * 8) == cudaSuccess;
    if (ok) ok = cudaMemset(b->pos_d, 0, sizeof(int32_t) * max_sessions) == cudaSuccess;
    for (int i = 0; ok && i < 8; i++)
        ok = cudaEventCreateWithFlags(&b->pos_ev[i], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
        (void)cudaGetLastError();
        q4i_fail(Q4E_CUDA, "batch_create: allocation failed");
        q4_gpu_batch_destroy(b);
        return nullptr;
    }
    if (cudaMemset(b->d_views, 0, sizeof(Q4Cache) * max_sessions) != cudaSuccess) (void)cudaGetLastError();
    return b;
}
extern "C" void q4_gpu_batch_destroy(q4_gpu_batch *b) {
    if (!b) return;
    if (b->d_views) cudaFree(b->d_views);
    if (b->pos_d) cudaFree(b->pos_d);
    if (b->pos_h) cudaFreeHost(b->pos_h);
    for (int i = 0; i < 8; i++)
        if (b->pos_ev[i]) cudaEventDestroy(b->pos_ev[i]);
    free(b->kv);
    free(b);
}
extern "C" bool q4_gpu_batch_bind(q4_gpu_batch *b, uint32_t slot, q4_gpu_kv *kv) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "batch_bind: library not initialised");
    Q4_REQUIRE(b && kv && slot < b->max_sessions && !g_q4.capturing, "batch_bind: bad argument");
    if (b->n) {
        const q4_gpu_kv *f = nullptr;
        for (uint32_t i = 0; i < b->n && !f; i++) f = b->kv[i];
        if (f) Q4_REQUIRE(f->n_layers == kv->n_layers && f->n_kvh == kv->n_kvh && f->hd == kv->hd && f->kind == kv->kind,
                          "batch_bind: stores of one batch must share shape and kind");
    }
    b->kv[slot] = kv;
    if (slot + 1 > b->n) b->n = slot + 1;
    /* device-to-device from the store's own device copy of its view: no host buffer to keep alive */
    if (!q4i_check(cudaMemcpyAsync(b->d_views + slot, kv->d_view, sizeof(Q4Cache), cudaMemcpyDeviceToDevice, g_q4.stream),
                   "batch_bind upload"))
        return false;
    return q4i_check(cudaStreamSynchronize(g_q4.stream), "batch_bind sync");
}
extern "C" bool q4_gpu_batch_set_pos(q4_gpu_batch *b, const int32_t *pos, uint32_t n_sessions) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "batch_set_pos: library not initialised");
    Q4_REQUIRE(b && pos && n_sessions && n_sessions <= b->n && !g_q4.capturing, "batch_set_pos: bad argument");
    /* a host running more than 8 steps ahead waits here for the upload that last used this slot */
    const uint32_t slot = b->ring++ & 7u;
    if (!q4i_check(cudaEventSynchronize(b->pos_ev[slot]), "batch_set_pos slot")) return false;
    int32_t *h = b->pos_h + (size_t)slot * b->max_sessions;
    uint32_t mx = 0;
    for (uint32_t i = 0; i < n_sessions; i++) {
        h[i] = pos[i];
        if (pos[i] > (int32_t)mx) mx = (uint32_t)pos[i];
    }
    b->max_pos = mx;
    b->n_active = n_sessions;
    return q4i_check(cudaMemcpyAsync(b->pos_d, h, sizeof(int32_t) * n_sessions, cudaMemcpyHostToDevice, g_q4.stream),
                     "batch_set_pos upload") &&
           q4i_check(cudaEventRecord(b->pos_ev[slot], g_q4.stream), "batch_set_pos event");
}
/* Positions move on the device: pos[s] += delta for the sessions of the last set_pos.  Stream-ordered and
 * capturable, so a decode step that is one CUDA graph (advance, then the layers) needs no host upload
 * between two replays (the upload of q4_gpu_batch_set_pos costs 3-4 us per step as a copy node). */
__global__ static void q4_batch_advance_k(int32_t *pos, uint32_t n, int32_t delta) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) pos[i] += delta;
}
extern "C" bool q4_gpu_batch_advance(q4_gpu_batch *b, int32_t delta) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "batch_advance: library not initialised");
    Q4_REQUIRE(b && b->n_active, "batch_advance: no positions published (q4_gpu_batch_set_pos)");
    q4_batch_advance_k<<<(b->n_active + 127u) / 128u, 128, 0, g_q4.stream>>>(b->pos_d, b->n_active, delta);
    if (!g_q4.capturing) b->max_pos = (uint32_t)((int64_t)b->max_pos + delta < 0 ? 0 : (int64_t)b->max_pos + delta);
    return q4i_check(cudaGetLastError(), "batch_advance launch");
}
extern "C" bool q4_gpu_batch_append(q4_gpu_batch *b, uint32_t layer, const float *k, const float *v) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "batch_append: library not initialised");
    Q4_REQUIRE(b && b->n && k && v && b->kv[0] && layer < b->kv[0]->n_layers, "batch_append: bad argument");
    Q4_REQUIRE(b->n_active, "batch_append: no positions published (q4_gpu_batch_set_pos)");
    AppendParams p;
    memset(&p, 0, sizeof(p));
    p.many = b->d_views; p.layer = layer; p.n_rows = b->n_active; p.n_kvh = b->kv[0]->n_kvh; p.hd = b->kv[0]->hd;
    p.k = k; p.v = v; p.pos = b->pos_d; p.err = g_q4.err_d;
    return launch_append(p, store_layout(b->kv[0]->kind));
}
extern "C" bool q4_gpu_batch_decode(q4_gpu_batch *b, uint32_t layer, const void *q, int q_bf16, const float *gate,
                                    float *out, const int32_t *idx, uint32_t width, uint32_t idx_kvh_stride,
                                    uint32_t idx_sess_stride, uint32_t n_head, float scale) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "batch_decode: library not initialised");
    Q4_REQUIRE(b && b->n && q && out && b->kv[0] && layer < b->kv[0]->n_layers && n_head, "batch_decode: bad argument");
    Q4_REQUIRE(b->n_active, "batch_decode: no positions published (q4_gpu_batch_set_pos)");
    Q4DecodeArgs a;
    memset(&a, 0, sizeof(a));
    a.many = b->d_views;
    a.layout = store_layout(b->kv[0]->kind);
    a.layer = layer;
    a.n_units = b->n_active;
    a.n_head = n_head;
    a.n_kvh = b->kv[0]->n_kvh;
    a.hd = b->kv[0]->hd;
    a.q = q; a.q_bf16 = q_bf16; a.gate = gate; a.out = out;
    a.idx = idx; a.width = width; a.idx_kvh_stride = idx_kvh_stride; a.idx_unit_stride = idx_sess_stride;
    a.pos = b->pos_d;
    a.hint_rows = b->max_pos + 1;
    a.idx_bound_nkv = 1;
    a.scale = scale;
    return q4i_decode(a);
}

/* Append + attend in one call.  On the native q8_0 store this is ONE launch per layer: the attention
 * kernel quantises and stores the newest rows itself; other kinds run the append kernel first. */
extern "C" bool q4_gpu_batch_append_decode(q4_gpu_batch *b, uint32_t layer, const float *k, const float *v, const void *q,
                                           int q_bf16, const float *gate, float *out, const int32_t *idx, uint32_t width,
                                           uint32_t idx_kvh_stride, uint32_t idx_sess_stride, uint32_t n_head, float scale) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "batch_append_decode: library not initialised");
    Q4_REQUIRE(b && b->n && k && v && q && out && b->kv[0] && layer < b->kv[0]->n_layers && n_head,
               "batch_append_decode: bad argument");
    Q4_REQUIRE(b->n_active, "batch_append_decode: no positions published (q4_gpu_batch_set_pos)");
    const bool fused = b->kv[0]->kind == Q4K_Q8 && b->kv[0]->hd == 128;
    if (!fused && !q4_gpu_batch_append(b, layer, k, v)) return false;
    Q4DecodeArgs a;
    memset(&a, 0, sizeof(a));
    a.many = b->d_views;
    a.layout = store_layout(b->kv[0]->kind);
    a.layer = layer;
    a.n_units = b->n_active;
    a.n_head = n_head;
    a.n_kvh = b->kv[0]->n_kvh;
    a.hd = b->kv[0]->hd;
    a.q = q; a.q_bf16 = q_bf16; a.gate = gate; a.out = out;
    a.idx = idx; a.width = width; a.idx_kvh_stride = idx_kvh_stride; a.idx_unit_stride = idx_sess_stride;
    a.pos = b->pos_d;
    a.hint_rows = b->max_pos + 1;
    a.idx_bound_nkv = 1;
    a.scale = scale;
    if (fused) { a.new_k = k; a.new_v = v; }
    return q4i_decode(a);
}
/* Single session, position from the device position word (graph-captured decode). */
extern "C" bool q4_gpu_kv_append_decode_d(q4_gpu_kv *kv, uint32_t layer, const float *k, const float *v, const void *q,
                                          int q_bf16, const float *gate, float *out, uint32_t n_head, const int32_t *idx,
                                          uint32_t width, uint32_t idx_kvh_stride, float scale) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "kv_append_decode_d: library not initialised");
    Q4_REQUIRE(kv && k && v && q && out && layer < kv->n_layers && n_head, "kv_append_decode_d: bad argument");
    const bool fused = kv->kind == Q4K_Q8 && kv->hd == 128;
    if (!fused && !q4_gpu_kv_append_d(kv, layer, k, v)) return false;
    Q4DecodeArgs a;
    memset(&a, 0, sizeof(a));
    a.one = kv->view;
    a.layout = store_layout(kv->kind);
    a.layer = layer;
    a.n_units = 1;
    a.n_head = n_head;
    a.n_kvh = kv->n_kvh;
    a.hd = kv->hd;
    a.q = q; a.q_bf16 = q_bf16; a.gate = gate; a.out = out;
    a.idx = idx; a.width = width; a.idx_kvh_stride = idx_kvh_stride;
    a.pos = g_q4.pos_d;
    a.hint_rows = kv->max_kv;
    a.idx_bound_nkv = 1;
    a.scale = scale;
    if (fused) { a.new_k = k; a.new_v = v; }
    return q4i_decode(a);
}
