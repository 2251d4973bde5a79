/*
 * Dense causal prefill attention over the native q8_0 store on the 5th-generation tensor cores
 * (tcgen05.mma, accumulators in tensor memory, operands brought in by TMA).  Query t of the chunk
 * attends rows [0, min(kv_base + t + 1, max_kv)) -- the semantics of gqa_prefill_k
 * (src/q4_rocm.cu:7019-7206) as launched by q4_hip_qsa_decode_n with n_tok > 1 (:7263,7286-7298);
 * the reference computes it with scalar FMAs on an fp16 tile and re-dequantises every K/V tile for
 * every query token.
 *
 * Two launches per call:
 *
 *  1. q4_pf_stage_k dequantises the rows the chunk can see, once, into two fp16 staging tensors in
 *     device memory: K as [kv head][row][128] and V transposed as [kv head][dim][row] (value =
 *     fp16(code * scale), the reference's fp16 tile).  25 MB at the benchmark shape, against
 *     1.4 TFLOP of attention that reads each of its tiles 512 times.
 *  2. q4_prefill_k: one block = one kv head x a group of query tokens whose (token, head) pairs
 *     fill the 128 rows of the MMA (16 tokens x 8 heads at the benchmark shape).  Per 64-position
 *     tile, K and V^T arrive by TMA (128-byte swizzle, two stages each) straight into the K-major
 *     operand layout, so no thread touches them:
 *
 *       producer warp (one thread): TMA loads, two tiles of K and of V^T in flight
 *       issuer warp (one thread): O[128 x 128] += P . V[j], 4 x tcgen05.mma (k = 16) with P as the A
 *                     operand in tensor memory, as soon as the softmax warps have published P, then
 *                     S[j+2] = Q . K[j+2]^T, 8 x tcgen05.mma, into the score buffer that held S[j]
 *                     and P[j] (two score buffers in tensor memory, so the next tile's scores are
 *                     always ready; products issued by one thread run in order, so P[j] is read
 *                     before S[j+2] lands on it)
 *       4 softmax warps: thread r owns row r: tcgen05.ld its 64 scores of tile j, causal mask,
 *                     running max with lazy rescale (the stored max only moves when it would grow
 *                     by more than 2^8, so the O accumulator in tensor memory is rarely touched),
 *                     P = exp2(..) as fp16 -> tcgen05.st into the first 32 columns of the score
 *                     buffer just read, mbarrier arrive.  Nothing here waits for the previous P . V
 *                     unless O has to be rescaled.
 *
 *     The roles meet only at mbarriers (scores ready, P ready, P.V drained, tiles landed): there
 *     is no block-wide barrier inside the tile loop.  Two blocks fit on an SM (97 KB of shared
 *     memory, 256 of the 512 tensor-memory columns each).
 *
 * Every mbarrier wait is bounded: on expiry the thread raises a block-wide abort flag that every
 * other wait polls, the block records Q4E_CUDA in the status word, and still frees its tensor memory.
 */
#include <cuda.h>
#include <cuda_bf16.h>
#include <math_constants.h>
#include <string.h>

#include "q4_internal.h"

namespace {

constexpr int PF_ROWS = 128, PF_BN = 64, PF_HD = 128;
constexpr uint32_t PF_Q_BYTES = 2 * PF_ROWS * 128, PF_K_BYTES = 2 * PF_BN * 128, PF_V_BYTES = PF_HD * 128;
constexpr uint32_t PF_STAGES = 2;
constexpr uint32_t PF_THREADS = PF_ROWS + 64;   /* 4 softmax warps, the tensor-core issuer, the TMA producer */
/* Q | P | K stages | V stages | barriers in the alignment slack */
constexpr uint32_t PF_TILE_BYTES = PF_Q_BYTES + PF_STAGES * (PF_K_BYTES + PF_V_BYTES);
constexpr uint32_t PF_SMEM = PF_TILE_BYTES + 1024;
constexpr uint32_t PF_TMEM_COLS = 256, PF_S_COL = 0, PF_O_COL = 128;   /* S0 at 0, S1 at 64, O at 128 */
constexpr uint32_t PF_SPIN_LIMIT = 1u << 24;
constexpr float PF_RESCALE_TAU = 8.f;

struct PrefillParams {
    uint32_t n_head, n_kvh, gqa, tpc /* tokens per block */;
    const __nv_bfloat16 *q;
    const float *gate;
    __nv_bfloat16 *out;
    uint32_t n_tok, kv_base, max_kv;
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
/* same product with the A operand in tensor memory (lane = row, one 32-bit column = two consecutive k) */
__device__ __forceinline__ void umma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
/* one probe of a phase; the callers bound the number of probes */
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0u;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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

/* ---- TMA: 3-D tiled loads that complete on an mbarrier */
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t x, int32_t y,
                                            int32_t z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}

/* ---- staging: rows [0, n) of (layer, kv head) -> fp16 K [kh][row][128] and V^T [kh][dim][n_pad].
 * Block = 64 positions of one kv head, 256 threads: thread t takes the 32-value block t & 3 of row
 * t >> 2, for K and for V; V goes through shared memory to come out position-contiguous. */
constexpr int PF_VT_PITCH = PF_BN + 2;   /* halves per dim row of the transposition tile (odd word count) */
__device__ __forceinline__ void dequant32(const uint8_t *codes, __half scale, uint32_t (&o)[16]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4 *>(codes)), b = __ldg(reinterpret_cast<const uint4 *>(codes) + 1);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    const __half2 s2 = __half2half2(scale);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        /* int8 -> the fp16 numbers 1152 + code by a byte permute, minus 1152 (exact), times the scale */
        const uint32_t x = w[i] ^ 0x80808080u;
        o[2 * i] = h2u(__hmul2(u2h(magic_sub(__byte_perm(x, 0x64646464u, 0x4140))), s2));
        o[2 * i + 1] = h2u(__hmul2(u2h(magic_sub(__byte_perm(x, 0x64646464u, 0x4342))), s2));
    }
}
__global__ void __launch_bounds__(256) q4_pf_stage_k(const Q4Cache C, uint32_t layer, uint32_t n, uint32_t n_pad,
                                                     __half *kf, __half *vt) {
    __shared__ __half tile[PF_HD * PF_VT_PITCH];
    const uint32_t kh = blockIdx.y, p0 = blockIdx.x * PF_BN, tid = threadIdx.x;
    const uint32_t r = tid >> 2, qb = tid & 3u, p = p0 + r;
    const uint8_t *kq = C.k + (uint64_t)layer * C.layer_stride + (uint64_t)kh * C.kvh_stride;
    const uint8_t *vq = C.v + (uint64_t)layer * C.layer_stride + (uint64_t)kh * C.kvh_stride;
    const uint8_t *sc = C.s + (uint64_t)layer * C.s_layer_stride + (uint64_t)kh * C.s_kvh_stride;
    uint32_t o[16];
    if (p < n) {
        const __half *srow = reinterpret_cast<const __half *>(sc + (uint64_t)p * C.s_tok_stride);
        dequant32(kq + (uint64_t)p * C.tok_stride + qb * 32u, __ldg(srow + qb), o);
        uint4 *dst = reinterpret_cast<uint4 *>(kf + ((size_t)kh * n + p) * PF_HD + qb * 32u);
#pragma unroll
        for (int i = 0; i < 4; i++) dst[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        dequant32(vq + (uint64_t)p * C.tok_stride + qb * 32u, __ldg(srow + 4 + qb), o);
    } else {
#pragma unroll
        for (int i = 0; i < 16; i++) o[i] = 0u;
    }
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const __half2 h = u2h(o[i]);
        tile[(qb * 32u + 2 * i) * PF_VT_PITCH + r] = __low2half(h);
        tile[(qb * 32u + 2 * i + 1) * PF_VT_PITCH + r] = __high2half(h);
    }
    __syncthreads();
    /* dim d = tid >> 1, positions 32 * (tid & 1) .. + 31: 64 contiguous bytes of V^T */
    const uint32_t d = tid >> 1, h0 = (tid & 1u) * 32u;
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 16; i++)
        w[i] = *reinterpret_cast<const uint32_t *>(&tile[d * PF_VT_PITCH + h0 + 2 * i]);
    uint4 *dst = reinterpret_cast<uint4 *>(vt + ((size_t)kh * PF_HD + d) * n_pad + p0 + h0);
#pragma unroll
    for (int i = 0; i < 4; i++) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
}


__global__ void __launch_bounds__(PF_THREADS, 2) q4_prefill_k(const PrefillParams P, const __grid_constant__ CUtensorMap map_k,
                                                              const __grid_constant__ CUtensorMap map_v) {
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    /* later token groups see more rows: launch them first so the tail of the grid is made of short blocks */
    const uint32_t kh = blockIdx.y, t0 = (gridDim.x - 1u - blockIdx.x) * P.tpc;

    /* 1024-byte aligned operand tiles (the swizzle pattern is anchored to the address) */
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t sQ = base, sK = sQ + PF_Q_BYTES, sV = sK + PF_STAGES * PF_K_BYTES;
    /* barriers in the alignment slack in front of the tiles when there is room, else behind them */
    const uint32_t bars = (base - smem_u32(smem_dyn) >= 96u) ? smem_u32(smem_dyn) : base + PF_TILE_BYTES;
    /* bar_p: one per score buffer.  A softmax warp may publish P of tile j + 1 before a slower warp has published
     * tile j (nothing but the score buffers holds it back), so consecutive tiles must not count on one barrier. */
    const uint32_t full_k = bars, full_v = bars + 16, bar_s = bars + 32, bar_o = bars + 48, bar_p = bars + 72,
                   s_tmem = bars + 64, s_abort = bars + 68;

    /* softmax thread r < 128 owns row r = (token t0 + r / gqa, head kh*gqa + r % gqa); rows past tpc*gqa or
     * past n_tok are padding.  Warp 4 issues the MMAs, warp 5 the TMA loads (one thread each). */
    const bool softmax_thread = tid < PF_ROWS;
    const uint32_t tl = tid / P.gqa, hh = tid % P.gqa, tok = t0 + tl;
    const bool row_live = softmax_thread && tl < P.tpc && tok < P.n_tok;
    uint32_t row_nkv = 0;                      /* this row attends positions [0, row_nkv) */
    if (row_live) row_nkv = min(P.kv_base + tok + 1u, P.max_kv);
    const uint32_t t_last = min(t0 + P.tpc, P.n_tok) - 1u;
    const uint32_t cta_nkv = min(P.kv_base + t_last + 1u, P.max_kv);
    const uint32_t cta_min_nkv = min(P.kv_base + t0 + 1u, P.max_kv);
    const uint32_t n_tiles = (cta_nkv + PF_BN - 1u) / PF_BN;

    if (warp == 4) {
        if (lane == 0) {
#pragma unroll
            for (uint32_t s = 0; s < PF_STAGES; s++) {
                mbar_init(full_k + 8 * s, 1);
                mbar_init(full_v + 8 * s, 1);
                mbar_init(bar_s + 8 * s, 1);
            }
            mbar_init(bar_o, 1);
            mbar_init(bar_p, PF_ROWS);
            mbar_init(bar_p + 8, PF_ROWS);
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(s_abort), "r"(0u) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_tmem),
                     "r"(PF_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else if (warp < 4) {
        /* ---- Q rows: bf16 -> fp16 (exact for normal values), K-major swizzled, 2 k-blocks of 64 dims */
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
        fence_async_smem();
    }
    tc_fence_before();
    __syncthreads();          /* barriers initialised, Q in place, tensor memory allocated */
    tc_fence_after();
    uint32_t tmem;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(s_tmem));

    constexpr uint32_t IDESC_QK = (1u << 4) | ((uint32_t)(PF_BN >> 3) << 17) | ((uint32_t)(PF_ROWS >> 4) << 24);
    constexpr uint32_t IDESC_PV = (1u << 4) | ((uint32_t)(PF_HD >> 3) << 17) | ((uint32_t)(PF_ROWS >> 4) << 24);
    /* bounded wait that also gives up when any thread of the block has given up */
    auto wait = [&](uint32_t bar, uint32_t parity) -> bool {
        for (uint32_t i = 0; i < PF_SPIN_LIMIT; i++) {
            if (mbar_test(bar, parity)) return true;
            if ((i & 1023u) == 1023u) {
                uint32_t a;
                asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(a) : "r"(s_abort) : "memory");
                if (a) return false;
            }
        }
        asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(s_abort), "r"(1u) : "memory");
        return false;
    };
    bool ok = true;

    if (warp == 5) {
        /* ================= producer: one thread keeps two tiles of K and of V^T in flight ================= */
        if (lane == 0 && n_tiles > 0) {
            auto load_k = [&](uint32_t tile) {     /* two 64-dim boxes of 64 rows */
                const uint32_t st = tile % PF_STAGES, bar = full_k + 8 * st, dst = sK + st * PF_K_BYTES;
                mbar_expect_tx(bar, PF_K_BYTES);
                tma_load_3d(dst, &map_k, bar, 0, (int32_t)(tile * PF_BN), (int32_t)kh);
                tma_load_3d(dst + PF_BN * 128, &map_k, bar, 64, (int32_t)(tile * PF_BN), (int32_t)kh);
            };
            auto load_v = [&](uint32_t tile) {     /* one box: 64 positions x 128 dims of V^T */
                const uint32_t st = tile % PF_STAGES, bar = full_v + 8 * st;
                mbar_expect_tx(bar, PF_V_BYTES);
                tma_load_3d(sV + st * PF_V_BYTES, &map_v, bar, (int32_t)(tile * PF_BN), 0, (int32_t)kh);
            };
            uint32_t k_issued = 1, v_issued = 1;
            load_k(0);
            load_v(0);
            if (n_tiles > 1) {
                load_k(1);
                load_v(1);
                k_issued = v_issued = 2;
            }
            for (uint32_t tile = 0; tile < n_tiles && ok; tile++) {
                const uint32_t st = tile % PF_STAGES, use = (tile / PF_STAGES) & 1u;
                /* Q.K of this tile complete: its K stage takes the tile two ahead */
                if (tile + 2 < n_tiles) {
                    ok = wait(bar_s + 8 * st, use);
                    if (ok) { load_k(tile + 2); k_issued = tile + 3; }
                }
                /* P.V of the previous tile complete: its V stage takes the tile after this one */
                if (ok && tile > 0 && tile + 1 < n_tiles) {
                    ok = wait(bar_o, (tile - 1u) & 1u);
                    if (ok) { load_v(tile + 1); v_issued = tile + 2; }
                }
            }
            /* Gave up somewhere: copies still in flight must land before the block's shared memory is
             * released (bounded again; these probes ignore the abort flag; phases that completed long ago
             * answer at once). */
            if (!ok) {
                for (uint32_t t = k_issued > 2 ? k_issued - 2 : 0; t < k_issued; t++)
                    for (uint32_t i = 0; i < PF_SPIN_LIMIT && !mbar_test(full_k + 8 * (t % PF_STAGES), (t / PF_STAGES) & 1u); i++) {}
                for (uint32_t t = v_issued > 2 ? v_issued - 2 : 0; t < v_issued; t++)
                    for (uint32_t i = 0; i < PF_SPIN_LIMIT && !mbar_test(full_v + 8 * (t % PF_STAGES), (t / PF_STAGES) & 1u); i++) {}
            }
        }
    } else if (warp == 4) {
        /* ================= tensor-core issuer: one thread ================= */
        if (lane == 0 && n_tiles > 0) {
            auto issue_qk = [&](uint32_t tile) {
                const uint32_t st = tile % PF_STAGES;
#pragma unroll
                for (uint32_t kk = 0; kk < 8; kk++) {
                    const uint64_t ad = umma_desc(sQ + (kk >> 2) * (PF_ROWS * 128) + (kk & 3) * 32);
                    const uint64_t bd = umma_desc(sK + st * PF_K_BYTES + (kk >> 2) * (PF_BN * 128) + (kk & 3) * 32);
                    umma_f16(tmem + PF_S_COL + st * PF_BN, ad, bd, IDESC_QK, kk > 0);
                }
                umma_commit(bar_s + 8 * st);
            };
            /* both score buffers are filled ahead of the softmax */
            ok = wait(full_k, 0);
            tc_fence_after();
            if (ok) issue_qk(0);
            if (ok && n_tiles > 1) {
                ok = wait(full_k + 8, 0);
                tc_fence_after();
                if (ok) issue_qk(1);
            }
            for (uint32_t tile = 0; tile < n_tiles && ok; tile++) {
                const uint32_t st = tile % PF_STAGES, use = (tile / PF_STAGES) & 1u;
                /* operands first (they land while the softmax runs), then the softmax's hand-over, so that
                 * nothing but the issue itself stands between "P is ready" and the two products */
                ok = wait(full_v + 8 * st, use);
                if (ok && tile + 2 < n_tiles) ok = wait(full_k + 8 * st, ((tile + 2) / PF_STAGES) & 1u);
                /* softmax of this tile done: P is in shared memory, O is rescaled, S[st] has been read */
                ok = ok && wait(bar_p + 8 * st, use);
                tc_fence_after();
                if (ok) {
#pragma unroll
                    for (uint32_t kk = 0; kk < 4; kk++) {
                        const uint64_t bd = umma_desc(sV + st * PF_V_BYTES + kk * 32);
                        umma_f16_ta(tmem + PF_O_COL, tmem + PF_S_COL + st * PF_BN + kk * 8, bd, IDESC_PV,
                                    (tile > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(bar_o);
                    if (tile + 2 < n_tiles) issue_qk(tile + 2);
                }
            }
        }
    } else {
        /* ================= softmax (warps 0-3): thread r owns row r ================= */
        const uint32_t t_lane = tmem + ((warp * 32u) << 16);   /* this warp's 32 lanes of tensor memory */
        float m_ref = -CUDART_INF_F, l_run = 0.f;
        for (uint32_t tile = 0; tile < n_tiles && ok; tile++) {
            const uint32_t st = tile % PF_STAGES, use = (tile / PF_STAGES) & 1u;
            ok = __all_sync(0xffffffffu, wait(bar_s + 8 * st, use));   /* a warp leaves the loop as one */
            tc_fence_after();
            float s[64];
            tmem_ld32(t_lane + PF_S_COL + st * PF_BN, *reinterpret_cast<float(*)[32]>(&s[0]));
            tmem_ld32(t_lane + PF_S_COL + st * PF_BN + 32, *reinterpret_cast<float(*)[32]>(&s[32]));
            tmem_wait_ld();
            const uint32_t p0 = tile * PF_BN;
            float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F, mx2 = -CUDART_INF_F, mx3 = -CUDART_INF_F;
            if (!(p0 + PF_BN <= cta_min_nkv && row_live)) {
#pragma unroll
                for (int i = 0; i < 64; i++)
                    if (p0 + i >= row_nkv) s[i] = -CUDART_INF_F;
            }
#pragma unroll
            for (int i = 0; i < 64; i += 4) {
                mx0 = fmaxf(mx0, s[i]); mx1 = fmaxf(mx1, s[i + 1]);
                mx2 = fmaxf(mx2, s[i + 2]); mx3 = fmaxf(mx3, s[i + 3]);
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * P.scale_log2e;   /* scale > 0 */
            float alpha = 1.f;
            const bool grow = mx > m_ref + PF_RESCALE_TAU;   /* also true on the first live tile (m_ref = -inf) */
            if (grow) {
                alpha = ex2f(m_ref - mx);             /* 0 on the first tile */
                m_ref = mx;
                l_run *= alpha;
            }
            const float mneg = m_ref == -CUDART_INF_F ? 0.f : -m_ref;
            float ls0 = 0.f, ls1 = 0.f;
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 32; i++) {
                const float e0 = ex2f(fmaf(s[2 * i], P.scale_log2e, mneg));
                const float e1 = ex2f(fmaf(s[2 * i + 1], P.scale_log2e, mneg));
                ls0 += e0;
                ls1 += e1;
                pk[i] = h2u(__floats2half2_rn(e0, e1));
            }
            l_run += ls0 + ls1;
            /* O is rescaled only when the stored maximum moved; the previous P.V must have drained first.  P itself
             * waits for nothing: it goes into the first 32 columns of the score buffer this thread has just read
             * (two fp16 per column), which the tensor core reads as the A operand of P.V before the scores of the
             * tile two ahead are written there (products issued by one thread run in order). */
            if (tile > 0 && __any_sync(0xffffffffu, grow)) {
                ok = __all_sync(0xffffffffu, ok && wait(bar_o, (tile - 1u) & 1u));
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    float o[32];
                    tmem_ld32(t_lane + PF_O_COL + 32 * c, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] *= alpha;
                    tmem_st32(t_lane + PF_O_COL + 32 * c, o);
                }
            }
            tmem_st32(t_lane + PF_S_COL + st * PF_BN, *reinterpret_cast<const float(*)[32]>(&pk[0]));
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar_p + 8 * st);
        }
        /* The last P.V.  A parity wait can tell the current phase from the one before it, no further: this thread
         * has not followed the phases of bar_o tile by tile, and when it gets here the product of tile n - 3 is
         * complete (the scores of tile n - 1 were committed behind it) but perhaps not yet that of tile n - 2. */
        if (ok && n_tiles > 1) ok = wait(bar_o, (n_tiles - 2u) & 1u);
        if (ok && n_tiles > 0) ok = wait(bar_o, (n_tiles - 1u) & 1u);
        tc_fence_after();

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
    }
    if (!ok && lane == 0) atomicOr(P.err, (uint32_t)Q4E_CUDA);
    tc_fence_before();
    __syncthreads();
    if (warp == 4)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(PF_TMEM_COLS) : "memory");
}

/* ---- host side: staging tensors, tensor maps, launches */
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult st;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &st) == cudaSuccess &&
            st == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        else
            (void)cudaGetLastError();
    }
    return fn;
}

/* fp16 staging of the rows a chunk can see; grows on demand, never inside a graph capture */
__half *g_stage = nullptr;
size_t g_stage_halves = 0;
bool stage_reserve(size_t halves) {
    if (halves <= g_stage_halves) return true;
    if (g_q4.capturing) return q4i_fail(Q4E_SCRATCH, "kv_prefill: staging buffer too small inside a capture");
    if (!q4i_check(cudaStreamSynchronize(g_q4.stream), "prefill staging sync")) return false;
    if (g_stage) cudaFree(g_stage);
    g_stage = nullptr;
    g_stage_halves = 0;
    const size_t want = halves + halves / 4;
    if (!q4i_check(cudaMalloc(&g_stage, want * sizeof(__half)), "prefill staging alloc")) return false;
    g_stage_halves = want;
    return true;
}

}  // namespace


void q4i_prefill_release() {
    if (g_stage) cudaFree(g_stage);
    g_stage = nullptr;
    g_stage_halves = 0;
}

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
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return q4i_fail(Q4E_CUDA, "kv_prefill: cuTensorMapEncodeTiled is not available from this driver");

    /* rows the chunk can see, staged as fp16: K [kvh][n][128], V^T [kvh][128][n_pad] */
    const uint64_t n64 = (uint64_t)kv_base + n_tok;
    const uint32_t n = (uint32_t)(n64 < kv->max_kv ? n64 : kv->max_kv);
    const uint32_t n_pad = (n + PF_BN - 1u) / PF_BN * PF_BN;
    const size_t k_halves = (size_t)kv->n_kvh * n * PF_HD, v_halves = (size_t)kv->n_kvh * PF_HD * n_pad;
    const size_t k_room = (k_halves + 63) & ~(size_t)63;    /* keeps V^T 128-byte aligned */
    if (!stage_reserve(k_room + v_halves)) return false;
    __half *kf = g_stage, *vt = g_stage + k_room;
    q4_pf_stage_k<<<dim3(n_pad / PF_BN, kv->n_kvh), 256, 0, g_q4.stream>>>(kv->view, layer, n, n_pad, kf, vt);
    if (!q4i_check(cudaGetLastError(), "prefill staging launch")) return false;

    CUtensorMap map_k, map_v;
    {
        const cuuint64_t dims[3] = {PF_HD, n, kv->n_kvh};
        const cuuint64_t strides[2] = {PF_HD * sizeof(__half), (cuuint64_t)n * PF_HD * sizeof(__half)};
        const cuuint32_t box[3] = {64, PF_BN, 1}, estr[3] = {1, 1, 1};
        if (enc(&map_k, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, kf, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return q4i_fail(Q4E_CUDA, "kv_prefill: tensor map (K) rejected");
    }
    {
        const cuuint64_t dims[3] = {n, PF_HD, kv->n_kvh};
        const cuuint64_t strides[2] = {(cuuint64_t)n_pad * sizeof(__half), (cuuint64_t)PF_HD * n_pad * sizeof(__half)};
        const cuuint32_t box[3] = {PF_BN, PF_HD, 1}, estr[3] = {1, 1, 1};
        if (enc(&map_v, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, vt, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return q4i_fail(Q4E_CUDA, "kv_prefill: tensor map (V) rejected");
    }

    PrefillParams p;
    memset(&p, 0, sizeof(p));
    p.n_head = n_head;
    p.n_kvh = kv->n_kvh;
    p.gqa = n_head / kv->n_kvh;
    p.tpc = PF_ROWS / p.gqa;
    p.q = (const __nv_bfloat16 *)q_bf16;
    p.gate = gate;
    p.out = (__nv_bfloat16 *)out_bf16;
    p.n_tok = n_tok;
    p.kv_base = kv_base;
    p.max_kv = kv->max_kv;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.err = g_q4.err_d;
    dim3 grid((n_tok + p.tpc - 1) / p.tpc, kv->n_kvh);
    q4_prefill_k<<<grid, PF_THREADS, PF_SMEM, g_q4.stream>>>(p, map_k, map_v);
    return q4i_check(cudaGetLastError(), "prefill launch");
}
