/*
 * Dense causal prefill attention over the native q8_0 store on the 5th-generation tensor cores
 * (tcgen05.mma, accumulators in tensor memory).  Query t of the chunk attends rows
 * [0, min(kv_base + t + 1, max_kv)) -- the semantics of gqa_prefill_k (src/q4_rocm.cu:7019-7206) as
 * launched by q4_hip_qsa_decode_n with n_tok > 1 (:7263,7286-7298); the reference computes it with
 * scalar FMAs on an fp16 tile and re-dequantises every K/V tile for every query token.
 *
 * One block = one kv head x a group of query tokens whose (token, head) pairs fill the 128 rows
 * of the MMA (16 tokens x 8 heads at the benchmark shape), so every dequantised K/V tile is shared
 * by the whole GQA group and by 16 tokens.  Per 64-position tile:
 *
 *   all 4 warps : int8 codes + fp16 block scales (prefetched into registers one tile ahead)
 *                 -> fp16 (exact integer via the magic-number trick, times the scale, as the reference's
 *                 fp16 tile) -> shared memory in the K-major 128-byte-swizzled operand layout; V is
 *                 transposed on the way so that both products read K-major operands
 *   one thread  : S[128 x 64]  = Q . K^T      8 x tcgen05.mma (k = 16), fp32 in tensor memory
 *   all 4 warps : thread r owns row r: tcgen05.ld its 64 scores, causal mask, running max with lazy
 *                 rescale (the stored max only moves when it would grow by more than 2^8, so the
 *                 O accumulator in tensor memory is rarely touched), P = exp2(..) as fp16 -> shared
 *   one thread  : O[128 x 128] += P . V        4 x tcgen05.mma
 *
 * Two blocks fit on an SM (82 KB of shared memory, 256 of the 512 tensor-memory columns each), so
 * one block's softmax overlaps the other's MMAs.  Every mbarrier wait is bounded: on expiry the
 * block records Q4E_CUDA in the status word, stops waiting and still frees its tensor memory.
 */
#include <cuda_bf16.h>
#include <math_constants.h>
#include <string.h>

#include "q4_internal.h"

namespace {

constexpr int PF_ROWS = 128, PF_BN = 64, PF_HD = 128;
constexpr uint32_t PF_Q_BYTES = 2 * PF_ROWS * 128, PF_K_BYTES = 2 * PF_BN * 128, PF_V_BYTES = PF_HD * 128,
                   PF_P_BYTES = PF_ROWS * 128;
constexpr uint32_t PF_SMEM = PF_Q_BYTES + PF_K_BYTES + PF_V_BYTES + PF_P_BYTES + 1024 /* alignment */ + 64;
constexpr uint32_t PF_TMEM_COLS = 256, PF_S_COL = 0, PF_O_COL = 64;
constexpr uint32_t PF_SPIN_LIMIT = 1u << 24;
constexpr float PF_RESCALE_TAU = 8.f;

struct PrefillParams {
    Q4Cache C;
    uint32_t layer, n_head, n_kvh, gqa, tpc /* tokens per block */;
    const __nv_bfloat16 *q;
    const float *gate;
    __nv_bfloat16 *out;
    uint32_t n_tok, kv_base;
    float scale_log2e;
    uint32_t *err;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t h2u(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u2h(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
__device__ __forceinline__ uint32_t magic_sub(uint32_t v) { return h2u(__hsub2(u2h(v), u2h(0x64806480u))); }

/* K-major operand tile, 128-byte rows, 16-byte chunks XOR-swizzled by (row & 7) inside 8-row groups */
__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t chunk) { return row * 128u + ((chunk ^ (row & 7u)) << 4); }

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    /* start >> 4 | LBO (unused with swizzle) = 1 | SBO = 1024 B >> 4 | version 1 | SWIZZLE_128B (2) */
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
/* bounded wait: false when the phase did not complete within the spin limit */
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < PF_SPIN_LIMIT; i++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t *r = reinterpret_cast<uint32_t *>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    const uint32_t *r = reinterpret_cast<const uint32_t *>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]),
          "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__global__ void __launch_bounds__(128, 2) q4_prefill_k(const PrefillParams P) {
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t kh = blockIdx.y, t0 = blockIdx.x * P.tpc;
    const Q4Cache &C = P.C;

    /* 1024-byte aligned operand tiles (the swizzle pattern is anchored to the address) */
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t sQ = base, sK = sQ + PF_Q_BYTES, sV = sK + PF_K_BYTES, sP = sV + PF_V_BYTES;
    const uint32_t bar_s = sP + PF_P_BYTES, bar_o = bar_s + 8, s_tmem = bar_o + 8;

    /* row r = (token t0 + r / gqa, head kh*gqa + r % gqa); rows past tpc*gqa or past n_tok are padding */
    const uint32_t tl = tid / P.gqa, hh = tid % P.gqa, tok = t0 + tl;
    const bool row_live = tl < P.tpc && tok < P.n_tok;
    uint32_t row_nkv = 0;                      /* this row attends positions [0, row_nkv) */
    if (row_live) row_nkv = min(P.kv_base + tok + 1u, C.max_kv);
    const uint32_t t_last = min(t0 + P.tpc, P.n_tok) - 1u;
    const uint32_t cta_nkv = min(P.kv_base + t_last + 1u, C.max_kv);
    const uint32_t cta_min_nkv = min(P.kv_base + t0 + 1u, C.max_kv);
    const uint32_t n_tiles = (cta_nkv + PF_BN - 1u) / PF_BN;

    if (tid == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_tmem),
                     "r"(PF_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    /* ---- Q rows: bf16 -> fp16 (exact for normal values), K-major swizzled, 2 k-blocks of 64 dims */
    {
        const __nv_bfloat16 *qrow = P.q + ((size_t)tok * P.n_head + (size_t)kh * P.gqa + hh) * PF_HD;
#pragma unroll
        for (uint32_t c = 0; c < 16; c++) {
            uint4 w = make_uint4(0u, 0u, 0u, 0u);
            if (row_live) w = *reinterpret_cast<const uint4 *>(qrow + c * 8);
            const uint32_t in[4] = {w.x, w.y, w.z, w.w};
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; i++)
                o[i] = h2u(__floats2half2_rn(__uint_as_float(in[i] << 16), __uint_as_float(in[i] & 0xffff0000u)));
            const uint32_t a = sQ + (c >> 3) * (PF_ROWS * 128) + sw128(tid, c & 7);
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
        }
    }

    const uint8_t *kq = C.k + (uint64_t)P.layer * C.layer_stride + (uint64_t)kh * C.kvh_stride;
    const uint8_t *vq = C.v + (uint64_t)P.layer * C.layer_stride + (uint64_t)kh * C.kvh_stride;
    const uint8_t *sc = C.s + (uint64_t)P.layer * C.s_layer_stride + (uint64_t)kh * C.s_kvh_stride;

    /* K units: (row lane + 32u, block warp), u = 0,1.  V unit: (position pair 2*lane, block warp). */
    uint4 kraw[2][2], vraw[2][2];
    __half kscale[2], vscale[2];
    auto prefetch = [&](uint32_t tile) {
        const uint32_t p0 = tile * PF_BN;
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const uint32_t p = p0 + lane + 32u * u;
            const uint32_t pc = min(p, cta_nkv - 1u);
            const uint4 *src = reinterpret_cast<const uint4 *>(kq + (uint64_t)pc * C.tok_stride + warp * 32u);
            kraw[u][0] = __ldg(src);
            kraw[u][1] = __ldg(src + 1);
            kscale[u] = p < cta_nkv ? __ldg(reinterpret_cast<const __half *>(sc + (uint64_t)pc * C.s_tok_stride) + warp)
                                    : __ushort_as_half(0);
        }
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const uint32_t p = p0 + 2u * lane + u;
            const uint32_t pc = min(p, cta_nkv - 1u);
            const uint4 *src = reinterpret_cast<const uint4 *>(vq + (uint64_t)pc * C.tok_stride + warp * 32u);
            vraw[u][0] = __ldg(src);
            vraw[u][1] = __ldg(src + 1);
            /* a scale of 0 for rows past the end keeps stale bytes from ever reaching the MMA as NaN */
            vscale[u] = p < cta_nkv ? __ldg(reinterpret_cast<const __half *>(sc + (uint64_t)pc * C.s_tok_stride) + 4 + warp)
                                    : __ushort_as_half(0);
        }
    };
    auto dequant_to_smem = [&]() {
        /* K: 32 dims of two rows -> 4 chunks each in k-block warp/2 */
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const uint32_t row = lane + 32u * u;
            const __half2 s2 = __half2half2(kscale[u]);
            const uint32_t w[8] = {kraw[u][0].x, kraw[u][0].y, kraw[u][0].z, kraw[u][0].w,
                                   kraw[u][1].x, kraw[u][1].y, kraw[u][1].z, kraw[u][1].w};
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const uint32_t x = w[2 * c + i] ^ 0x80808080u;
                    o[2 * i] = h2u(__hmul2(u2h(magic_sub(__byte_perm(x, 0x64646464u, 0x4140))), s2));
                    o[2 * i + 1] = h2u(__hmul2(u2h(magic_sub(__byte_perm(x, 0x64646464u, 0x4342))), s2));
                }
                const uint32_t a = sK + (warp >> 1) * (PF_BN * 128) + sw128(row, (warp & 1) * 4 + c);
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
            }
        }
        /* V^T: dims 32*warp + j as rows, positions (2*lane, 2*lane+1) as one 4-byte element pair */
        {
            const __half2 s2 = __halves2half2(vscale[0], vscale[1]);
            const uint32_t a0[8] = {vraw[0][0].x, vraw[0][0].y, vraw[0][0].z, vraw[0][0].w,
                                    vraw[0][1].x, vraw[0][1].y, vraw[0][1].z, vraw[0][1].w};
            const uint32_t a1[8] = {vraw[1][0].x, vraw[1][0].y, vraw[1][0].z, vraw[1][0].w,
                                    vraw[1][1].x, vraw[1][1].y, vraw[1][1].z, vraw[1][1].w};
#pragma unroll
            for (int wd = 0; wd < 8; wd++) {
#pragma unroll
                for (int bi = 0; bi < 4; bi++) {
                    const uint32_t u = __byte_perm(a0[wd], a1[wd], ((4 + bi) << 8) | bi);
                    const uint32_t v = h2u(__hmul2(u2h(magic_sub((u & 0x00FF00FFu) ^ 0x64806480u)), s2));
                    const uint32_t d = warp * 32u + wd * 4 + bi;
                    const uint32_t a = sV + d * 128u + (((lane >> 2) ^ (d & 7u)) << 4) + (lane & 3u) * 4u;
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
                }
            }
        }
    };

    prefetch(0);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(s_tmem));
    const uint32_t t_lane = tmem + ((warp * 32u) << 16);   /* this warp's 32 lanes of tensor memory */

    constexpr uint32_t IDESC_QK = (1u << 4) | ((uint32_t)(PF_BN >> 3) << 17) | ((uint32_t)(PF_ROWS >> 4) << 24);
    constexpr uint32_t IDESC_PV = (1u << 4) | ((uint32_t)(PF_HD >> 3) << 17) | ((uint32_t)(PF_ROWS >> 4) << 24);

    float m_ref = -CUDART_INF_F, l_run = 0.f;
    bool ok = true;
    for (uint32_t tile = 0; tile < n_tiles && ok; tile++) {
        const uint32_t par = tile & 1u;
        /* the previous P.V must have drained before V^T and P are overwritten */
        if (tile > 0) ok = mbar_wait(bar_o, par ^ 1u);
        tc_fence_after();
        dequant_to_smem();
        if (tile + 1 < n_tiles) prefetch(tile + 1);
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (uint32_t kk = 0; kk < 8; kk++) {
                const uint64_t ad = umma_desc(sQ + (kk >> 2) * (PF_ROWS * 128) + (kk & 3) * 32);
                const uint64_t bd = umma_desc(sK + (kk >> 2) * (PF_BN * 128) + (kk & 3) * 32);
                umma_f16(tmem + PF_S_COL, ad, bd, IDESC_QK, kk > 0);
            }
            umma_commit(bar_s);
        }
        ok = ok && mbar_wait(bar_s, par);
        tc_fence_after();

        /* ---- softmax of this thread's row */
        float s[64];
        tmem_ld32(t_lane + PF_S_COL, *reinterpret_cast<float(*)[32]>(&s[0]));
        tmem_ld32(t_lane + PF_S_COL + 32, *reinterpret_cast<float(*)[32]>(&s[32]));
        tmem_wait_ld();
        const uint32_t p0 = tile * PF_BN;
        float mx = -CUDART_INF_F;
        if (p0 + PF_BN <= cta_min_nkv && row_live) {
#pragma unroll
            for (int i = 0; i < 64; i++) mx = fmaxf(mx, s[i]);
        } else {
#pragma unroll
            for (int i = 0; i < 64; i++) {
                if (p0 + i >= row_nkv) s[i] = -CUDART_INF_F;
                mx = fmaxf(mx, s[i]);
            }
        }
        mx *= P.scale_log2e;                      /* scale > 0: max commutes with the scaling */
        float alpha = 1.f;
        const bool grow = mx > m_ref + PF_RESCALE_TAU;   /* also true on the first live tile (m_ref = -inf) */
        if (grow) {
            alpha = ex2f(m_ref - mx);             /* 0 on the first tile */
            m_ref = mx;
            l_run *= alpha;
        }
        if (tile > 0 && __any_sync(0xffffffffu, grow)) {
            /* O row *= alpha.  The previous P.V has completed (waited for above). */
#pragma unroll
            for (int c = 0; c < 4; c++) {
                float o[32];
                tmem_ld32(t_lane + PF_O_COL + 32 * c, o);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i++) o[i] *= alpha;
                tmem_st32(t_lane + PF_O_COL + 32 * c, o);
            }
            tmem_wait_st();
        }
        const float mneg = m_ref == -CUDART_INF_F ? 0.f : -m_ref;
        float lsum = 0.f;
#pragma unroll
        for (int c = 0; c < 8; c++) {
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float e0 = ex2f(fmaf(s[8 * c + 2 * i], P.scale_log2e, mneg));
                const float e1 = ex2f(fmaf(s[8 * c + 2 * i + 1], P.scale_log2e, mneg));
                const __half2 h = __floats2half2_rn(e0, e1);
                lsum += __low2float(h) + __high2float(h);   /* the denominator sums what the MMA sees */
                o[i] = h2u(h);
            }
            const uint32_t a = sP + sw128(tid, c);
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
        }
        l_run += lsum;
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (uint32_t kk = 0; kk < 4; kk++) {
                const uint64_t ad = umma_desc(sP + kk * 32);
                const uint64_t bd = umma_desc(sV + kk * 32);
                umma_f16(tmem + PF_O_COL, ad, bd, IDESC_PV, (tile > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(bar_o);
        }
    }
    if (ok && n_tiles > 0) ok = mbar_wait(bar_o, (n_tiles - 1u) & 1u);
    tc_fence_after();
    if (!ok && lane == 0) atomicOr(P.err, (uint32_t)Q4E_CUDA);

    /* ---- epilogue: O / l * sigmoid(gate) -> bf16 */
    if (ok) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        const size_t off = ((size_t)tok * P.n_head + (size_t)kh * P.gqa + hh) * PF_HD;
#pragma unroll
        for (int c = 0; c < 4; c++) {
            float o[32];
            tmem_ld32(t_lane + PF_O_COL + 32 * c, o);
            tmem_wait_ld();
            if (row_live) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint32_t w[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        float x0 = o[i + 2 * j] * inv, x1 = o[i + 2 * j + 1] * inv;
                        if (P.gate) {
                            const float2 gt = *reinterpret_cast<const float2 *>(P.gate + off + 32 * c + i + 2 * j);
                            x0 *= 1.f / (1.f + __expf(-gt.x));
                            x1 *= 1.f / (1.f + __expf(-gt.y));
                        }
                        __nv_bfloat162 b = __floats2bfloat162_rn(x0, x1);
                        w[j] = *reinterpret_cast<uint32_t *>(&b);
                    }
                    *reinterpret_cast<uint4 *>(P.out + off + 32 * c + i) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(PF_TMEM_COLS) : "memory");
}

}  // namespace

extern "C" bool q4_gpu_kv_prefill(const q4_gpu_kv *kv, uint32_t layer, const void *q_bf16, const float *gate,
                                  void *out_bf16, uint32_t n_head, uint32_t n_tok, uint32_t kv_base, float scale) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "kv_prefill: library not initialised");
    Q4_REQUIRE(kv && q_bf16 && out_bf16 && n_head && n_tok && layer < kv->n_layers, "kv_prefill: bad argument");
    Q4_REQUIRE(kv->kind == Q4K_Q8 && kv->hd == PF_HD, "kv_prefill: tensor-core path needs a q8_0 store with hd 128");
    Q4_REQUIRE(n_head % kv->n_kvh == 0 && n_head / kv->n_kvh <= 16, "kv_prefill: n_head/n_kvh must be 1..16");
    Q4_REQUIRE(scale > 0.f, "kv_prefill: scale must be positive");
    Q4_REQUIRE((uint64_t)kv_base + 1 <= kv->max_kv, "kv_prefill: kv_base beyond max_kv");
    static bool attr = false;
    if (!attr) {
        if (!q4i_check(cudaFuncSetAttribute(q4_prefill_k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM),
                       "prefill smem attribute"))
            return false;
        attr = true;
    }
    PrefillParams p;
    memset(&p, 0, sizeof(p));
    p.C = kv->view;
    p.layer = layer;
    p.n_head = n_head;
    p.n_kvh = kv->n_kvh;
    p.gqa = n_head / kv->n_kvh;
    p.tpc = PF_ROWS / p.gqa;
    p.q = (const __nv_bfloat16 *)q_bf16;
    p.gate = gate;
    p.out = (__nv_bfloat16 *)out_bf16;
    p.n_tok = n_tok;
    p.kv_base = kv_base;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.err = g_q4.err_d;
    dim3 grid((n_tok + p.tpc - 1) / p.tpc, kv->n_kvh);
    q4_prefill_k<<<grid, 128, PF_SMEM, g_q4.stream>>>(p);
    return q4i_check(cudaGetLastError(), "prefill launch");
}
