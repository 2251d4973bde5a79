/*
 * Decode attention for one query token per unit over a q8_0 / fp16 / fp32 KV cache:
 * split-KV flash decoding with the GQA group sharing every K/V row it reads.
 *
 * Replaces gqa_dec_split_k + gqa_dec_comb_k (and the gqa_decode_fast fallback) of the reference,
 * src/q4_rocm.cu:6549-7012, with the semantics of its launchers (:7249-7364): positions < 0 are
 * padding and are skipped, a unit with no live position outputs 0, the output is the
 * softmax-weighted V times sigmoid(gate).
 *
 * Shape of the kernel.  The path is bound by HBM, and with 8 query heads sharing each K/V byte the
 * scalar FMA pipe cannot keep up with B200's memory system (8 FMA per int8 byte at ~23 B/clk/SM
 * is more than the 128 FMA/clk an SM has), so the two contractions run on the tensor cores with
 * warp-level MMA.  Every byte of the cache is read from global memory once.  For the native q8_0
 * store at hd 128 each warp owns a 4-stage ring of 16-position tiles in shared memory (the tile's
 * records as they lie in the store, 272 bytes apart).  A tile of 16 consecutive positions is one
 * contiguous span of the store: it comes in with fully coalesced 16-byte cp.async copies, or, in a
 * dense scan, with one 4352-byte bulk copy (cp.async.bulk, completion on the stage's mbarrier); any
 * other tile is gathered row by row with 16-byte cp.async copies.  Per tile the warp unloads the
 * stage into MMA fragments (ldmatrix for the K rows, transposing ldmatrix for the V rows), refills
 * the stage at once with the tile four ahead, and then computes from registers, so four tiles per
 * warp are in flight all the time; there is no block barrier in the main loop, warps stream
 * independently.  The other layouts load fragments straight into registers with sector-aligned
 * 4/8/16-byte loads.
 *
 *   one warp-step = 16 positions:
 *     S^T[16 pos x 8 heads]  = K[16 x hd] . Q^T        (m16n8k16, K rows are the A operand)
 *     online softmax on S^T  (per head: max over positions by warp shuffles)
 *     P^T -> fp16, 8x8 transposed in-warp (movmatrix) into the B operand
 *     O^T[hd x 8 heads]     += V^T[hd x 16 pos] . P^T   (V bytes are the A operand)
 *
 *   q8_0: int8 codes are converted to exact fp16 integers in registers (byte permute; the K side
 *   folds the offset into the MMA's initial accumulator, the V side subtracts it); K block scales
 *   multiply the four per-block partial dot products in fp32, V block scales are folded into P^T
 *   per 32-wide block of hd.  Nothing is rounded except Q (to fp16 once; exact for bf16 queries)
 *   and the softmax weights (fp16, and the denominator sums the same rounded weights).
 *
 * grid = (splits, kv heads, units).  Every block reduces its warps' partials in shared memory.  Up to
 * 16 splits form one thread-block cluster and merge through distributed shared memory (no scratch, no
 * atomics: every block pushes the heads of its record to the blocks that own them, and the pushes
 * complete an mbarrier there).  More splits write (acc, m, l) records to scratch; when the whole grid
 * is resident the unit's blocks meet at a counter and share out (head, 32-dim) slices of the merge,
 * otherwise -- and in the sequence-sharded exchange, whose last block must hold the rank's record --
 * the last block to arrive per group of 16 merges, two levels at most.  Either way the layer is one
 * launch.
 */
#include <cuda_bf16.h>
#include <math_constants.h>
#include <stdlib.h>
#include <string.h>

#include "q4_internal.h"

namespace {

constexpr int DEC_WARPS = 4;
constexpr int DEC_THREADS = DEC_WARPS * 32;
constexpr uint32_t DEC_MAX_SPLIT = 256;
constexpr uint32_t DEC_GROUP = 16;   /* records merged per level of the two-level merge */
constexpr uint32_t MERGE_SCRATCH_FLOATS = 2 * DEC_GROUP * 16 + 32;   /* weights, sums, per-head max and total */
constexpr uint32_t DEC_CLUSTER_MAX = 16;   /* most splits of a unit that merge through one cluster (8 is the portable size) */

struct DecParams {
    Q4Cache one;
    const Q4Cache *many;
    uint32_t layer, n_head, n_kvh, gqa;
    const void *q;
    int q_bf16;
    const float *gate;
    float *out, *part_out;
    const int32_t *idx;
    uint32_t width, idx_kvh_stride, idx_unit_stride;
    const int32_t *pos;
    uint32_t kv_base;
    uint32_t idx_bound_nkv;   /* 1: list entries must be below the rows written so far (newest + 1), else below max_kv */
    float scale_log2e;
    uint32_t S;
    uint32_t cluster; /* blocks per cluster (0 = none): the S splits of a unit form one cluster and merge through DSMEM */
    float *scratch;
    uint32_t *counters;
    uint32_t *err;
    const Q4XchgDev *xchg;   /* sequence-sharded decode: exchange window (null otherwise) */
    uint32_t xchg_phase;
    const float *new_k, *new_v;   /* fused append of the newest row (native q8_0 store), or null */
    uint32_t pdl;                 /* launched with programmatic stream serialization */
    uint32_t gridmerge;           /* long scans: every split's record goes to scratch, the unit's blocks meet at a counter,
                                   * and (head, 32-dim) slices of the merge are shared out among them */
    uint32_t push_bytes;          /* > 0: the launch carries this much extra shared memory and merges by pushing */
    uint32_t push_async;          /* pushes complete an mbarrier of the receiving block (its last 16 bytes) instead of
                                   * meeting at a cluster barrier */
    uint32_t bulk_runs;           /* tiles of 16 consecutive positions come in by one bulk copy each (else by cp.async) */
};

/* ---- small device helpers ---------------------------------------------------------------- */
__device__ __forceinline__ uint32_t ldg32(const void *p) {
    uint32_t v;
    asm("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg16(const void *p) {
    uint16_t v;
    asm("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg64(const void *p) {
    uint2 v;
    asm("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ldg128(const void *p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(p));
    return v;
}
/* 16-byte asynchronous copy, or 16 zero bytes for a padding position.  The copy uses the plain form
 * without a source-size operand so that neighbouring lanes coalesce into whole sectors. */
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void *gsrc, bool live) {
    if (live)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
    else
        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(smem_dst), "r"(0u) : "memory");
}
/* The K and the V chunk of one record (V codes follow the K codes at +HD, in the store and in a ring stage);
 * nothing is copied for a padding position. */
template <int HD>
__device__ __forceinline__ void cp_async16_kv(uint32_t smem_dst, const void *gsrc, int32_t pos) {
    asm volatile(
        "{\n\t.reg .pred q;\n\tsetp.ge.s32 q, %2, 0;\n\t"
        "@q cp.async.cg.shared.global [%0], [%1], 16;\n\t"
        "@q cp.async.cg.shared.global [%0+%3], [%1+%3], 16;\n\t}"
        ::"r"(smem_dst), "l"(gsrc), "r"(pos), "n"(HD) : "memory");
}
/* 512 consecutive bytes per warp instruction: lane l copies bytes [OFF + 16 l, OFF + 16 l + 16) */
template <int OFF>
__device__ __forceinline__ void cp_async16_at(uint32_t smem_dst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0+%2], [%1+%2], 16;" ::"r"(smem_dst), "l"(gsrc), "n"(OFF) : "memory");
}
/* one record, global -> shared, through the bulk-copy engine; completion is counted in bytes on the mbarrier */
__device__ __forceinline__ void bulk_copy_g2s(uint32_t smem_dst, const void *gsrc, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void ring_bar_init(uint32_t bar) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void ring_bar_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ring_bar_test(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0u;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
/* four 8x8 matrices of 16-bit elements (eight 16-byte rows each; lanes 8i..8i+7 give the row addresses of
 * matrix i); thread (g, t) receives elements 2t, 2t+1 of row g of every matrix -- of the transposed
 * matrix with .trans, i.e. element g of rows 2t and 2t+1 */
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr) : "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
/* same product with the initial accumulator in registers of its own: rows g and g+8 start from (c0, c1) */
__device__ __forceinline__ void mma16816_from(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1, float c0, float c1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%10,%11};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ uint32_t movmatrix_t(uint32_t x) {
    uint32_t y;
    asm("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t h2u(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u2h(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) { return h2u(__floats2half2_rn(lo, hi)); }

/* 0x6480 is fp16 1152 = 1024 + 128: (code ^ 0x80) in the low mantissa bits of 1024.0 is the fp16
 * number 1152 + code, so one subtract gives the int8 code as an exact fp16. */
__device__ __forceinline__ uint32_t magic_sub(uint32_t v) {
    return h2u(__hsub2(u2h(v), u2h(0x64806480u)));
}
/* 4 int8 in one word -> fp16x2 of bytes (0,1) and of bytes (2,3). */
__device__ __forceinline__ void cvt_i8x4(uint32_t w, uint32_t &lo, uint32_t &hi) {
    uint32_t x = w ^ 0x80808080u;
    lo = magic_sub(__byte_perm(x, 0x64646464u, 0x4140));
    hi = magic_sub(__byte_perm(x, 0x64646464u, 0x4342));
}
/* byte BI of word a and of word b -> fp16x2 {a.BI, b.BI}. */
template <int BI>
__device__ __forceinline__ uint32_t cvt_i8_pair(uint32_t a, uint32_t b) {
    uint32_t u = __byte_perm(a, b, ((4 + BI) << 8) | BI);
    return magic_sub((u & 0x00FF00FFu) ^ 0x64806480u);
}
__device__ __forceinline__ float warp_max_over_g(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
}
__device__ __forceinline__ float warp_sum_over_g(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    return v + __shfl_xor_sync(0xffffffffu, v, 16);
}

/* Which head dimension the accumulator pair (c0,c1) / (c2,c3) of output tile mt holds for lane
 * group g.  The register-direct q8 paths interleave so that each tile stays inside one 32-wide scale
 * block; the staged path (fragments through ldmatrix) and the fp16 / fp32 rows use plain 16-dim tiles. */
template <int LAY, bool STAGED>
__device__ __forceinline__ int out_dim(int mt, int g, int hi) {
    if ((LAY == LAY_Q8P || LAY == LAY_Q8R) && !STAGED) return 32 * (mt >> 1) + 4 * g + 2 * (mt & 1) + hi;
    return 16 * mt + 2 * g + hi;
}
/* Which 4 head dimensions lane t feeds to k-step ks of the QK product (same map for Q and K). */
template <int LAY>
__device__ __forceinline__ int qk_dim(int ks, int t) {
    if (LAY == LAY_Q8P || LAY == LAY_Q8R) return 32 * (ks >> 1) + 8 * t + 4 * (ks & 1);
    return 16 * ks + 4 * t;
}

/* ---- merge of (acc, m, l) records ------------------------------------------------------------- */
struct MergeOut {
    float *out, *part_out;
    const float *gate;
    size_t row0;       /* index of the group's first head in [unit][head] order */
    uint32_t gqa;
};

/* arrive on a counter; true for the last of `expected` arrivals (which also re-arms it) */
__device__ __noinline__ bool arrive_last(uint32_t *ctr, uint32_t expected) {
    __shared__ uint32_t s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t prev = atomicAdd(ctr, 1u);
        s_last = (prev == expected - 1u);
        if (s_last) *ctr = 0u;   /* ready for the next launch / graph replay */
    }
    __syncthreads();
    const bool last = s_last != 0u;
    if (last) __threadfence();
    return last;
}

/* what a merge does with 4 dims of one head: a record for the next level, the public record
 * {m (natural-log units), l, acc[HD]}, or the final out = acc / l * sigmoid(gate) */
template <int HD>
__device__ __forceinline__ void merge_store(float *dst_rec, const MergeOut &mo, uint32_t h, uint32_t d, float M, float L,
                                            float4 A) {
    constexpr int REC = HD + 4;
    if (dst_rec) {
        float *o = dst_rec + (size_t)h * REC;
        *reinterpret_cast<float4 *>(o + d) = A;
        if (d == 0) { o[HD] = M; o[HD + 1] = L; }
    } else if (mo.part_out) {
        float *pr = mo.part_out + (mo.row0 + h) * (HD + 2);
        if (d == 0) {
            pr[0] = L > 0.f ? M * 0.6931471805599453f : 0.f;
            pr[1] = L;
        }
        pr[2 + d] = A.x; pr[3 + d] = A.y; pr[4 + d] = A.z; pr[5 + d] = A.w;
    } else {
        const float inv = L > 0.f ? 1.f / L : 0.f;
        float4 o = make_float4(A.x * inv, A.y * inv, A.z * inv, A.w * inv);
        const size_t off = (mo.row0 + h) * HD + d;
        if (mo.gate) {
            const float4 gt = *reinterpret_cast<const float4 *>(mo.gate + off);
            o.x *= 1.f / (1.f + __expf(-gt.x)); o.y *= 1.f / (1.f + __expf(-gt.y));
            o.z *= 1.f / (1.f + __expf(-gt.z)); o.w *= 1.f / (1.f + __expf(-gt.w));
        }
        *reinterpret_cast<float4 *>(mo.out + off) = o;
    }
}

/* Merge `count` (<= DEC_GROUP) records spaced HEADS*REC floats apart (log2-domain max).  Weights are
 * computed once per (record, head); then every thread owns 4 output dims of some heads and streams
 * the accumulators with 8 independent 16-byte loads in flight.  dst_rec != null stores a merged
 * record for the next level, otherwise the result is finalised: out = acc / l * sigmoid(gate), or the
 * public record {m (natural-log units), l, acc[HD]}.  Deliberately not inlined: the kernel calls it
 * from one place for every merge level, and a small kernel image matters for launches that run each
 * instruction once. */
template <int HD, int HEADS>
__device__ __noinline__ void merge_records(const float *recs, uint32_t count, bool global, float *dst_rec,
                                           const MergeOut mo, float *scratch /* MERGE_SCRATCH_FLOATS of shared memory */) {
    constexpr int REC = HD + 4;
    float *s_w = scratch, *s_l = scratch + DEC_GROUP * 16, *s_M = scratch + 2 * DEC_GROUP * 16, *s_L = s_M + 16;
    const uint32_t gqa = mo.gqa;
    if (!global && count == DEC_WARPS && dst_rec) {
        /* The block's own four warp records, in shared memory: every thread recomputes the four weights
         * of its head (no shared weights, no barriers in between) and writes its 4 dims of the block
         * record.  This runs once in every block of every launch. */
        for (uint32_t i = threadIdx.x; i < gqa * (HD / 4); i += DEC_THREADS) {
            const uint32_t h = i / (HD / 4), d = (i % (HD / 4)) * 4;
            float2 ml[DEC_WARPS];
            float4 x[DEC_WARPS];
#pragma unroll
            for (int k = 0; k < DEC_WARPS; k++) {
                const float *r = recs + ((size_t)k * HEADS + h) * REC;
                ml[k] = *reinterpret_cast<const float2 *>(r + HD);
                x[k] = *reinterpret_cast<const float4 *>(r + d);
            }
            float M = -CUDART_INF_F;
#pragma unroll
            for (int k = 0; k < DEC_WARPS; k++) M = fmaxf(M, ml[k].x);
            const float Mu = M == -CUDART_INF_F ? 0.f : M;
            float L = 0.f;
            float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int k = 0; k < DEC_WARPS; k++) {
                const float w = ex2(ml[k].x - Mu);
                L = fmaf(w, ml[k].y, L);
                A.x = fmaf(w, x[k].x, A.x); A.y = fmaf(w, x[k].y, A.y);
                A.z = fmaf(w, x[k].z, A.z); A.w = fmaf(w, x[k].w, A.w);
            }
            float *o = dst_rec + (size_t)h * REC;
            *reinterpret_cast<float4 *>(o + d) = A;
            if (d == 0) { o[HD] = M; o[HD + 1] = L; }
        }
        __syncthreads();
        return;
    }
    if (global) {
        /* Records of other blocks, in global memory (L2): one batch of independent loads per output item
         * -- all (m, l) pairs and all accumulator slices -- and the weights recomputed per thread, so a
         * merge level costs one memory round trip per item and no barrier.  Only the last block to arrive
         * at a level runs this. */
        for (uint32_t i = threadIdx.x; i < gqa * (HD / 4); i += DEC_THREADS) {
            const uint32_t h = i / (HD / 4), d = (i % (HD / 4)) * 4;
            float2 ml[DEC_GROUP];
            float4 x[DEC_GROUP];
#pragma unroll
            for (uint32_t k = 0; k < DEC_GROUP; k++) {
                const float *r = recs + ((size_t)min(k, count - 1u) * HEADS + h) * REC;
                ml[k] = __ldcg(reinterpret_cast<const float2 *>(r + HD));
                x[k] = __ldcg(reinterpret_cast<const float4 *>(r + d));
            }
            float M = -CUDART_INF_F;
#pragma unroll
            for (uint32_t k = 0; k < DEC_GROUP; k++)
                if (k < count) M = fmaxf(M, ml[k].x);
            const float Mu = M == -CUDART_INF_F ? 0.f : M;
            float L = 0.f;
            float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (uint32_t k = 0; k < DEC_GROUP; k++) {
                const float w = k < count ? ex2(ml[k].x - Mu) : 0.f;
                L = fmaf(w, ml[k].y, L);
                A.x = fmaf(w, x[k].x, A.x); A.y = fmaf(w, x[k].y, A.y);
                A.z = fmaf(w, x[k].z, A.z); A.w = fmaf(w, x[k].w, A.w);
            }
            merge_store<HD>(dst_rec, mo, h, d, M, L, A);
        }
        __syncthreads();
        return;
    }
    for (uint32_t i = threadIdx.x; i < count * HEADS; i += DEC_THREADS) {
        const float2 *r = reinterpret_cast<const float2 *>(recs + (size_t)i * REC + HD);
        const float2 ml = global ? __ldcg(r) : *r;   /* one round trip for every m and l */
        s_w[i] = ml.x;
        s_l[i] = ml.y;
    }
    __syncthreads();
    if (threadIdx.x < gqa) {
        const uint32_t h = threadIdx.x;
        float M = -CUDART_INF_F;
        for (uint32_t s = 0; s < count; s++) M = fmaxf(M, s_w[s * HEADS + h]);
        const float Mu = M == -CUDART_INF_F ? 0.f : M;
        float L = 0.f;
        for (uint32_t s = 0; s < count; s++) {
            const float w = ex2(s_w[s * HEADS + h] - Mu);
            s_w[s * HEADS + h] = w;
            L = fmaf(w, s_l[s * HEADS + h], L);
        }
        s_M[h] = M;
        s_L[h] = L;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < gqa * (HD / 4); i += DEC_THREADS) {
        const uint32_t h = i / (HD / 4), d = (i % (HD / 4)) * 4;
        float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t s0 = 0; s0 < count; s0 += 8) {
            float4 x[8];
#pragma unroll
            for (uint32_t k = 0; k < 8; k++) {
                const uint32_t sidx = min(s0 + k, count - 1u);
                const float4 *r = reinterpret_cast<const float4 *>(recs + ((size_t)sidx * HEADS + h) * REC + d);
                x[k] = global ? __ldcg(r) : *r;
            }
#pragma unroll
            for (uint32_t k = 0; k < 8; k++) {
                const float w = s0 + k < count ? s_w[(s0 + k) * HEADS + h] : 0.f;
                A.x = fmaf(w, x[k].x, A.x); A.y = fmaf(w, x[k].y, A.y);
                A.z = fmaf(w, x[k].z, A.z); A.w = fmaf(w, x[k].w, A.w);
            }
        }
        merge_store<HD>(dst_rec, mo, h, d, s_M[h], s_L[h], A);
    }
    __syncthreads();   /* s_w is reused by the next level */
}

/* ---- merge inside a thread-block cluster (distributed shared memory) -------------------------- */
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ float ld_cluster(uint32_t a) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
    return v;
}
/* When the splits of a unit are the blocks of one cluster (at most 16), every block leaves its record
 * in its own shared memory and block r merges heads r, r+S, .. by reading all S records through
 * distributed shared memory: no scratch, no atomics, no global round trips.  Called between two
 * cluster barriers (records complete before, nobody exits while peers still read after).  (Clusters of 8
 * as a first level under a merge in global memory were measured for units with hundreds of splits:
 * slower than two levels in global memory, 53.8 vs 51.5 us at 262144 rows.) */
template <int HD, int HEADS>
__device__ __noinline__ void cluster_merge(uint32_t rec_saddr, uint32_t S, uint32_t rank, const MergeOut mo) {
    constexpr int REC = HD + 4;
    for (uint32_t h = rank; h < mo.gqa; h += S) {
        float m[DEC_CLUSTER_MAX], l[DEC_CLUSTER_MAX];
        float M = -CUDART_INF_F;
#pragma unroll
        for (uint32_t s = 0; s < DEC_CLUSTER_MAX; s++) {
            m[s] = -CUDART_INF_F;
            l[s] = 0.f;
            if (s < S) {
                const uint32_t b = map_to_rank(rec_saddr + (h * REC + HD) * 4, s);
                m[s] = ld_cluster(b);
                l[s] = ld_cluster(b + 4);
            }
            M = fmaxf(M, m[s]);
        }
        const float Mu = M == -CUDART_INF_F ? 0.f : M;
        float L = 0.f;
#pragma unroll
        for (uint32_t s = 0; s < DEC_CLUSTER_MAX; s++) {
            m[s] = ex2(m[s] - Mu);
            L = fmaf(m[s], l[s], L);
        }
        for (uint32_t d = threadIdx.x; d < (uint32_t)HD; d += DEC_THREADS) {
            float a[DEC_CLUSTER_MAX];
#pragma unroll
            for (uint32_t s = 0; s < DEC_CLUSTER_MAX; s++)
                a[s] = s < S ? ld_cluster(map_to_rank(rec_saddr + (h * REC + d) * 4, s)) : 0.f;
            float A = 0.f;
#pragma unroll
            for (uint32_t s = 0; s < DEC_CLUSTER_MAX; s++) A = fmaf(m[s], a[s], A);
            if (mo.part_out) {
                float *pr = mo.part_out + (mo.row0 + h) * (HD + 2);
                if (d == 0) {
                    pr[0] = L > 0.f ? M * 0.6931471805599453f : 0.f;
                    pr[1] = L;
                }
                pr[2 + d] = A;
            } else {
                float o = L > 0.f ? A / L : 0.f;
                const size_t off = (mo.row0 + h) * HD + d;
                if (mo.gate) o *= 1.f / (1.f + __expf(-mo.gate[off]));
                mo.out[off] = o;
            }
        }
    }
}

constexpr uint32_t PUSH_SPIN_LIMIT = 1u << 22;   /* probes of the receive barrier before the block gives up */
/* Push form of the cluster merge, for launches that carry extra shared memory for it (a few units in
 * flight, clusters of more than 8 blocks): every block stores head h of its record into the receive
 * area of block h % S (slot (h / S) * S + own rank) through distributed shared memory, one cluster
 * barrier makes the stores visible, and every block merges the heads it owns from its OWN shared
 * memory.  Nobody reads a peer's memory after the barrier, so the second barrier of the pull form (and
 * the ~1 us it adds to a 9 us kernel) is not needed; the receive area lies behind the ring, so a fast
 * peer may push while this block is still in its position loop. */
template <int HD, int HEADS>
__device__ __noinline__ void cluster_push_merge(const float *own, const float *recv, uint32_t S, uint32_t rank,
                                                const MergeOut mo, uint32_t bar, uint32_t *err) {
    constexpr int REC = HD + 4;
    const uint32_t recv_saddr = (uint32_t)__cvta_generic_to_shared(recv);
    if (bar) {
        /* Every 16-byte store reports its bytes to the receiving block's barrier; a block that owns heads waits
         * for exactly the bytes of its heads' S records, a block that owns none is done once it has pushed.
         * Nobody waits for the slowest block of the cluster unless it needs that block's record. */
        const uint32_t n_own = rank < mo.gqa ? (mo.gqa - rank + S - 1u) / S : 0u;
        if (threadIdx.x == 0 && n_own) ring_bar_expect(bar, n_own * S * REC * 4u);
        for (uint32_t i = threadIdx.x; i < mo.gqa * (REC / 4); i += DEC_THREADS) {
            const uint32_t h = i / (REC / 4), c = i % (REC / 4);
            const float4 v = *reinterpret_cast<const float4 *>(own + (size_t)h * REC + 4 * c);
            const uint32_t dst = map_to_rank(recv_saddr + ((((h / S) * S + rank) * REC) + 4 * c) * 4, h % S);
            const uint32_t rbar = map_to_rank(bar, h % S);
            asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1,%2,%3,%4}, [%5];"
                         ::"r"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"(rbar) : "memory");
        }
        if (!n_own) return;
        uint32_t probes = 0;
        while (!ring_bar_test(bar, 0u) && ++probes < PUSH_SPIN_LIMIT) {}
        if (probes >= PUSH_SPIN_LIMIT) {      /* a peer's record never arrived: reported, the output is not valid */
            atomicOr(err, (uint32_t)Q4E_CUDA);
            return;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < mo.gqa * (REC / 4); i += DEC_THREADS) {
            const uint32_t h = i / (REC / 4), c = i % (REC / 4);
            const float4 v = *reinterpret_cast<const float4 *>(own + (size_t)h * REC + 4 * c);
            const uint32_t dst = map_to_rank(recv_saddr + ((((h / S) * S + rank) * REC) + 4 * c) * 4, h % S);
            asm volatile("st.shared::cluster.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
        }
        cluster_sync_all();
    }
    for (uint32_t h = rank, j = 0; h < mo.gqa; h += S, j++) {
        const float *base = recv + (size_t)j * S * REC;
        float m[DEC_CLUSTER_MAX], l[DEC_CLUSTER_MAX];
        float M = -CUDART_INF_F;
#pragma unroll
        for (uint32_t s = 0; s < DEC_CLUSTER_MAX; s++) {
            m[s] = -CUDART_INF_F;
            l[s] = 0.f;
            if (s < S) {
                const float2 ml = *reinterpret_cast<const float2 *>(base + (size_t)s * REC + HD);
                m[s] = ml.x;
                l[s] = ml.y;
            }
            M = fmaxf(M, m[s]);
        }
        const float Mu = M == -CUDART_INF_F ? 0.f : M;
        float L = 0.f;
#pragma unroll
        for (uint32_t s = 0; s < DEC_CLUSTER_MAX; s++) {
            m[s] = ex2(m[s] - Mu);
            L = fmaf(m[s], l[s], L);
        }
        for (uint32_t d = threadIdx.x; d < (uint32_t)HD; d += DEC_THREADS) {
            float A = 0.f;
#pragma unroll
            for (uint32_t s = 0; s < DEC_CLUSTER_MAX; s++)
                if (s < S) A = fmaf(m[s], base[(size_t)s * REC + d], A);
            if (mo.part_out) {
                float *pr = mo.part_out + (mo.row0 + h) * (HD + 2);
                if (d == 0) {
                    pr[0] = L > 0.f ? M * 0.6931471805599453f : 0.f;
                    pr[1] = L;
                }
                pr[2 + d] = A;
            } else {
                float o = L > 0.f ? A / L : 0.f;
                const size_t off = (mo.row0 + h) * HD + d;
                if (mo.gate) o *= 1.f / (1.f + __expf(-mo.gate[off]));
                mo.out[off] = o;
            }
        }
    }
}

/* ---- merge of a long scan's records by all of the unit's blocks ---------------------------------
 * A unit with hundreds of splits (a dense scan over 262144 rows: 222 blocks per kv head) used to merge in two
 * levels, each a fence + atomic + the last block of a group reading 16 records: two serial round trips through L2
 * behind the slowest block.  Here every block writes its record, the unit's S blocks meet at a counter (they are
 * all resident: the launcher checks that the grid fits in one wave), and the first gqa * HD / 32 of them each
 * merge one (head, 32 dims) slice of all S records: the weights once per record, then 16 record lanes x 8 threads
 * of 4 dims stream the accumulators.  The wait is bounded; the last block to leave re-arms the two counters. */
constexpr uint32_t GRID_SPIN_LIMIT = 1u << 22;
template <int HD, int HEADS>
__device__ __noinline__ void grid_merge(const float *recs, uint32_t S, uint32_t split, uint32_t *ctr, const MergeOut mo,
                                        float *scr /* >= 256 + 16 * 32 + 8 floats of shared memory */, uint32_t *err) {
    constexpr int REC = HD + 4, CH = HD / 32;
    __shared__ uint32_t s_ok;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        atomicAdd(&ctr[0], 1u);
        uint32_t spins = 0, seen;
        do {
            asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(seen) : "l"(ctr) : "memory");
        } while (seen < S && ++spins < GRID_SPIN_LIMIT);
        s_ok = seen >= S ? 1u : 0u;
    }
    __syncthreads();
    const bool ok = s_ok != 0u;
    float *s_w = scr, *s_part = scr + 256, *s_red = scr + 256 + 16 * 32;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (ok)
        for (uint32_t task = split; task < mo.gqa * CH; task += S) {
            const uint32_t h = task / CH, d0 = (task % CH) * 32;
            /* weights of the S records of head h (m in log2 units; an empty record has l = 0) */
            float mloc = -CUDART_INF_F;
            for (uint32_t r = threadIdx.x; r < S; r += DEC_THREADS) {
                const float2 ml = __ldcg(reinterpret_cast<const float2 *>(recs + ((size_t)r * HEADS + h) * REC + HD));
                if (ml.y > 0.f) mloc = fmaxf(mloc, ml.x);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
            if (lane == 0) s_red[warp] = mloc;
            __syncthreads();
            const float M = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
            const float Mu = M == -CUDART_INF_F ? 0.f : M;
            float lloc = 0.f;
            for (uint32_t r = threadIdx.x; r < S; r += DEC_THREADS) {
                const float2 ml = __ldcg(reinterpret_cast<const float2 *>(recs + ((size_t)r * HEADS + h) * REC + HD));
                const float w = ml.y > 0.f ? ex2(ml.x - Mu) : 0.f;
                s_w[r] = w;
                lloc = fmaf(w, ml.y, lloc);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) lloc += __shfl_xor_sync(0xffffffffu, lloc, o);
            __syncthreads();                       /* s_red read by everyone, s_w written */
            if (lane == 0) s_red[4 + warp] = lloc;
            __syncthreads();
            const float L = (s_red[4] + s_red[5]) + (s_red[6] + s_red[7]);
            /* 16 record lanes x 8 threads of 4 dims */
            const uint32_t q = threadIdx.x >> 3, dq = (threadIdx.x & 7u) * 4u;
            float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t r = q; r < S; r += 16) {
                const float w = s_w[r];
                const float4 x = __ldcg(reinterpret_cast<const float4 *>(recs + ((size_t)r * HEADS + h) * REC + d0 + dq));
                A.x = fmaf(w, x.x, A.x); A.y = fmaf(w, x.y, A.y); A.z = fmaf(w, x.z, A.z); A.w = fmaf(w, x.w, A.w);
            }
            *reinterpret_cast<float4 *>(s_part + q * 32 + dq) = A;
            __syncthreads();
            if (threadIdx.x < 8) {
                float4 T = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int k = 0; k < 16; k++) {
                    const float4 x = *reinterpret_cast<const float4 *>(s_part + k * 32 + dq);
                    T.x += x.x; T.y += x.y; T.z += x.z; T.w += x.w;
                }
                merge_store<HD>(nullptr, mo, h, d0 + dq, M, L, T);
            }
            __syncthreads();
        }
    if (threadIdx.x == 0) {
        if (!ok) atomicOr(err, (uint32_t)Q4E_CUDA);
        __threadfence();
        if (atomicAdd(&ctr[1], 1u) == S - 1u) {   /* everyone has passed the meeting point: ready for the next launch */
            ctr[1] = 0u;
            __threadfence();
            ctr[0] = 0u;
        }
    }
}

/* ---- exchange of the units' records between ranks (sequence-sharded decode) --------------------
 * The block that finishes a unit's last merge holds the rank's record in shared memory.  It stores
 * the record into slot (parity, unit, rank) of every rank's window, its own included, as 8-byte
 * packets {fp32 value, epoch}: peer stores over NVLink, no fence and no separate flag, because a
 * packet is written atomically and carries its own validity (the call's epoch).  It then reads all
 * `world` records from its own window, polling each packet until the epoch matches, and merges
 * them into the output.  Slots are double-buffered by the parity of the epoch: a rank can be at most
 * one call ahead of a peer, because it cannot finish call e+1 before the peer has published e+1,
 * which the peer does only after it has finished reading call e.  Every wait is bounded; when one
 * runs out, status bit Q4E_PEER is set and the output is the rank's own part. */
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void *p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys_v4(void *p, uint4 v) {
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
/* packets of slot (parity, unit, writer) in window w */
__device__ __forceinline__ uint2 *xchg_slot(const Q4XchgDev *xd, Q4XchgWin *w, uint32_t par, uint32_t unit,
                                            uint32_t writer) {
    uint2 *base = reinterpret_cast<uint2 *>(reinterpret_cast<char *>(w) + XCHG_REC_OFFSET);
    return base + ((size_t)(par * xd->units + unit) * xd->world + writer) * xd->slot_floats;
}
template <int HD, int HEADS>
__device__ __noinline__ void xchg_wait_merge(const Q4XchgDev *xd, uint32_t unit, uint32_t epoch, const MergeOut mo,
                                             uint32_t *err) {
    constexpr int REC = HD + 4;
    __shared__ uint32_t s_missing;
    const uint32_t rank = xd->rank, world = xd->world, par = epoch & 1u;
    Q4XchgWin *w = xd->win[rank];
    if (threadIdx.x == 0) s_missing = 0u;
    __syncthreads();
    const unsigned long long t0 = global_ns(), limit = xd->timeout_ns;
    /* pass 0 merges all ranks' records; pass 1 runs only after a wait ran out and merges this rank's alone */
    for (int pass = 0; pass < 2; pass++) {
        const bool alone = pass == 1;
        const uint32_t n_src = alone ? 1u : world;
        for (uint32_t i = threadIdx.x; i < mo.gqa * (HD / 4); i += DEC_THREADS) {
            const uint32_t h = i / (HD / 4), d = (i % (HD / 4)) * 4;
            float M = -CUDART_INF_F, L = 0.f;
            float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t s0 = 0; s0 < n_src; s0 += 4) {
                uint4 pm[4], pa[4], pb[4];   /* {m, e, l, e}, {x0, e, x1, e}, {x2, e, x3, e} */
                uint32_t polls = 0;
                for (;;) {
                    bool ok = true;
#pragma unroll
                    for (uint32_t k = 0; k < 4; k++) {
                        const uint32_t src = alone ? rank : min(s0 + k, world - 1u);
                        const uint2 *pk = xchg_slot(xd, w, par, unit, src) + (size_t)h * REC;
                        pm[k] = ld_relaxed_sys_v4(pk + HD);
                        pa[k] = ld_relaxed_sys_v4(pk + d);
                        pb[k] = ld_relaxed_sys_v4(pk + d + 2);
                    }
#pragma unroll
                    for (uint32_t k = 0; k < 4; k++)
                        ok = ok && pm[k].y == epoch && pm[k].w == epoch && pa[k].y == epoch && pa[k].w == epoch &&
                             pb[k].y == epoch && pb[k].w == epoch;
                    if (ok) break;
                    if (++polls > 32u) __nanosleep(100);
                    /* time limit, plus a poll limit in case the timer does not advance */
                    if ((polls & 63u) == 0u && (global_ns() - t0 > limit || polls > (1u << 24))) {
                        atomicOr(&s_missing, 1u);
                        break;
                    }
                }
                if (!alone && s_missing) break;   /* this or another thread gave up: pass 1 redoes the item */
                float Mn = M;
#pragma unroll
                for (uint32_t k = 0; k < 4; k++)
                    if (s0 + k < n_src) Mn = fmaxf(Mn, __uint_as_float(pm[k].x));
                const float Mu = Mn == -CUDART_INF_F ? 0.f : Mn;
                const float c = ex2(M - Mu);   /* 0 for the first chunk (M = -inf) */
                L *= c; A.x *= c; A.y *= c; A.z *= c; A.w *= c;
#pragma unroll
                for (uint32_t k = 0; k < 4; k++) {
                    const float wgt = s0 + k < n_src ? ex2(__uint_as_float(pm[k].x) - Mu) : 0.f;
                    L = fmaf(wgt, __uint_as_float(pm[k].z), L);
                    A.x = fmaf(wgt, __uint_as_float(pa[k].x), A.x); A.y = fmaf(wgt, __uint_as_float(pa[k].z), A.y);
                    A.z = fmaf(wgt, __uint_as_float(pb[k].x), A.z); A.w = fmaf(wgt, __uint_as_float(pb[k].z), A.w);
                }
                M = Mn;
            }
            const float inv = L > 0.f ? 1.f / L : 0.f;
            float4 o = make_float4(A.x * inv, A.y * inv, A.z * inv, A.w * inv);
            const size_t off = (mo.row0 + h) * HD + d;
            if (mo.gate) {
                const float4 gt = *reinterpret_cast<const float4 *>(mo.gate + off);
                o.x *= 1.f / (1.f + __expf(-gt.x)); o.y *= 1.f / (1.f + __expf(-gt.y));
                o.z *= 1.f / (1.f + __expf(-gt.z)); o.w *= 1.f / (1.f + __expf(-gt.w));
            }
            *reinterpret_cast<float4 *>(mo.out + off) = o;
        }
        __syncthreads();
        if (!s_missing || alone) break;
        if (threadIdx.x == 0) atomicOr(err, (uint32_t)Q4E_PEER);
    }
}
/* rec: the rank's merged record for the unit, [gqa][REC] floats in shared memory, complete (the merge
 * that wrote it ends with a block barrier) */
template <int HD, int HEADS>
__device__ __noinline__ void xchg_finish(const Q4XchgDev *xd, uint32_t phase, uint32_t unit, const float *rec,
                                         const MergeOut mo, uint32_t *err) {
    constexpr int REC = HD + 4;
    const uint32_t rank = xd->rank, world = xd->world;
    Q4XchgWin *w = xd->win[rank];
    const uint32_t epoch = __ldcg(&w->epoch[unit]) + 1u, par = epoch & 1u;
    const uint32_t n2 = mo.gqa * REC / 2;
    for (uint32_t q = 0; q < world; q++) {
        const uint32_t p = (rank + 1u + q) % world;   /* peers first, own window last */
        uint4 *dst = reinterpret_cast<uint4 *>(xchg_slot(xd, xd->win[p], par, unit, rank));
        for (uint32_t i = threadIdx.x; i < n2; i += DEC_THREADS) {
            const float2 v = *reinterpret_cast<const float2 *>(rec + 2 * i);
            st_relaxed_sys_v4(dst + i, make_uint4(__float_as_uint(v.x), epoch, __float_as_uint(v.y), epoch));
        }
    }
    __syncthreads();   /* every thread has read the old epoch before it changes */
    if (threadIdx.x == 0) w->epoch[unit] = epoch;
    if (phase == XCHG_PUSH) return;
    xchg_wait_merge<HD, HEADS>(xd, unit, epoch, mo, err);
}
/* the wait-and-merge half as its own launch (one block per unit), after a push-only decode */
template <int HD, int HEADS>
__global__ void __launch_bounds__(DEC_THREADS) q4_xchg_merge_k(const Q4XchgDev *xd, uint32_t gqa, const float *gate,
                                                               float *out, uint32_t *err) {
    const uint32_t unit = blockIdx.x;
    MergeOut mo;
    mo.out = out; mo.part_out = nullptr; mo.gate = gate;
    mo.row0 = (size_t)unit * gqa;
    mo.gqa = gqa;
    xchg_wait_merge<HD, HEADS>(xd, unit, __ldcg(&xd->win[xd->rank]->epoch[unit]), mo, err);
}


/* ---- the kernel ---------------------------------------------------------------------------- */
constexpr int RING_STAGES = 4;
/* A stage holds the 16 records of a tile as they lie in the store: row r at r * 272 = K codes | V codes | K and V
 * block scales.  Rows 272 bytes apart put the eight 16-byte row pieces of one 8x8 ldmatrix block into eight
 * different bank groups ((17 r + c) mod 8), so no swizzle is needed, and a tile whose 16 positions are
 * consecutive is one contiguous 4352-byte span of the store, which one bulk copy (cp.async.bulk, completion
 * counted in bytes on the stage's mbarrier) brings in; other tiles are gathered with 16-byte cp.async copies. */
constexpr int RING_ROW = 272;
constexpr int RING_V_OFF = 128;                             /* V codes of a row relative to its K codes */
constexpr int RING_MASK_OFF = 16 * RING_ROW;                /* bits 0-15: live positions, bit 16: brought in by a bulk copy */
constexpr uint32_t RING_RUN_BIT = 1u << 16;
constexpr int RING_STAGE_BYTES = 16 * RING_ROW + 32;        /* rows, mask word */
constexpr int RING_BAR_BYTES = DEC_WARPS * RING_STAGES * 8; /* one mbarrier per stage, behind the rings of all warps */
constexpr uint32_t RING_SPIN_LIMIT = 1u << 22;             /* probes of a stage's mbarrier before the block gives up */

template <int LAY, int HD, int NHT>
struct DecCfg {
    static constexpr bool STAGED = (LAY == LAY_Q8P && HD == 128);
    static constexpr int HEADS = 8 * NHT;
    static constexpr int REC = HD + 4;          /* acc[HD], m, l, 2 pad: 16-byte aligned records */
    static constexpr size_t EPI_BYTES = (size_t)DEC_WARPS * HEADS * REC * sizeof(float);
    static constexpr size_t RING_BYTES = STAGED ? (size_t)DEC_WARPS * RING_STAGES * RING_STAGE_BYTES + RING_BAR_BYTES : 0;
    static constexpr size_t REC_BYTES = (size_t)HEADS * REC * sizeof(float);   /* the block's merged record */
    static constexpr size_t TAIL_BYTES = EPI_BYTES + REC_BYTES + MERGE_SCRATCH_FLOATS * sizeof(float);   /* after the loop */
    static constexpr size_t SMEM = TAIL_BYTES > RING_BYTES ? TAIL_BYTES : RING_BYTES;
    static constexpr int MIN_BLOCKS = STAGED ? (NHT == 1 ? 3 : 2) : (HD * NHT <= 128 ? 3 : 1);
};

template <int LAY, int HD, int NHT>
__global__ void __launch_bounds__(DEC_THREADS, (DecCfg<LAY, HD, NHT>::MIN_BLOCKS))
q4_decode_k(const DecParams P) {
    using Cfg = DecCfg<LAY, HD, NHT>;
    constexpr int NB = HD / 32;   /* q8_0 blocks per row */
    constexpr int KS = HD / 16;   /* k-steps of the QK product */
    constexpr int MT = HD / 16;   /* 16-dim output tiles of the PV product */
    constexpr int HEADS = Cfg::HEADS;
    constexpr int REC = Cfg::REC;
    constexpr bool Q8 = (LAY == LAY_Q8P || LAY == LAY_Q8R);
    constexpr int NBQ = Q8 ? NB : 1;

    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const uint32_t split = blockIdx.x, kh = blockIdx.y, u = blockIdx.z;
    const uint32_t S = P.S;

    const Q4Cache C = P.many ? P.many[u] : P.one;
    /* The blocks of a cluster write into one another's shared memory at the end (push merge).  A block's
     * shared memory may be accessed remotely only once that block runs, so every block announces itself here
     * and waits for its peers' announcements just before its first remote access: by then they have all
     * arrived long ago and the wait costs nothing. */
    if (P.cluster) {
        if (P.push_async) {
            /* the barrier that the peers' pushes complete: initialised before this block announces itself */
            if (threadIdx.x == 0) {
                ring_bar_init((uint32_t)__cvta_generic_to_shared(smem_raw + DecCfg<LAY, HD, NHT>::SMEM + P.push_bytes - 16u));
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            }
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        } else {
            asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
        }
    }
    /* Programmatic dependent launch: the blocks of this launch may already be resident while the previous
     * kernel of the stream drains.  Only the cache view above (written when the store was created or bound)
     * is read before this point; positions, lists, queries and rows are read after it. */
    if (P.pdl) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        /* the next launch of the stream may bring its blocks in as slots free up (it still waits, at its
         * own griddepcontrol.wait, for this grid to finish before it reads anything this grid writes) */
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    const uint32_t newest = P.pos ? (uint32_t)P.pos[P.many ? u : 0] : P.kv_base + u;
    uint32_t n_kv = newest + 1u;
    if (n_kv > C.max_kv) n_kv = C.max_kv;
    const int32_t *list = P.idx ? P.idx + (size_t)u * P.idx_unit_stride + (size_t)kh * P.idx_kvh_stride
                                : nullptr;
    const uint32_t n_pos = list ? P.width : n_kv;
    const uint32_t steps = (n_pos + 15u) >> 4;
    const uint32_t per = (steps + S - 1u) / S;
    const uint32_t s_begin = split * per;
    const uint32_t s_end = min(s_begin + per, steps);

    const uint8_t *kbase = C.k + (uint64_t)P.layer * C.layer_stride + (uint64_t)kh * C.kvh_stride;
    const uint8_t *vbase = C.v + (uint64_t)P.layer * C.layer_stride + (uint64_t)kh * C.kvh_stride;
    const uint8_t *sbase = nullptr;
    if (LAY == LAY_Q8P)
        sbase = C.s + (uint64_t)P.layer * C.s_layer_stride + (uint64_t)kh * C.s_kvh_stride;
    const uint32_t tok_stride = C.tok_stride, s_tok_stride = C.s_tok_stride;
    const uint32_t max_kv = C.max_kv;
    /* list entries at or beyond this are skipped and raise the range status: the rows written so far for a
     * store (rows behind them hold nothing), the capacity for a caller-owned cache of the reference ABI */
    const uint32_t bound = P.idx_bound_nkv ? n_kv : max_kv;

    /* ---- fused append, first half: the load of the unit's new K/V row is issued here, next to the
     * loads of the list entries below, so that the two round trips overlap; the row is quantised and
     * stored just before the first cache row is read.  8 lanes per 32-value block, the first hd/4
     * threads take the K row and the next hd/4 the V row. */
    float4 ap_x = make_float4(0.f, 0.f, 0.f, 0.f);
    bool ap_which = false, ap_live = false;
    uint32_t ap_b = 0, ap_sub = 0;
    if constexpr (Cfg::STAGED) {   /* rows are read with cp.async (coherent at L2), never through the read-only path */
        if (P.new_k) {
            constexpr uint32_t QL = HD / 4;
            const uint32_t tid = threadIdx.x;
            ap_which = tid >= QL;
            ap_live = tid < 2 * QL && newest < max_kv;
            const uint32_t w = ap_which ? tid - QL : tid;
            ap_b = w >> 3;
            ap_sub = w & 7u;
            if (ap_live)
                ap_x = *reinterpret_cast<const float4 *>((ap_which ? P.new_v : P.new_k) +
                                                         ((size_t)u * P.n_kvh + kh) * HD + ap_b * 32 + ap_sub * 4);
        }
    }

    /* position j of the list / range, or -1 (padding, out of range) */
    auto position = [&](uint32_t j) -> int32_t {
        if (j >= n_pos) return -1;
        if (!list) return (int32_t)j;
        int32_t p = list[j];
        if (p >= (int32_t)bound) {
            atomicOr(P.err, (uint32_t)Q4E_RANGE);
            p = -1;
        }
        return p;
    };

    /* ---- Q fragments (B operand of the QK product): head nt*8+g, dims qk_dim(ks, t)..+3 */
    uint32_t qf[NHT][KS][2];
#pragma unroll
    for (int nt = 0; nt < NHT; nt++) {
        const uint32_t hg = nt * 8 + g;
        const bool live = hg < P.gqa;
        const size_t qoff = ((size_t)u * P.n_head + (size_t)kh * P.gqa + hg) * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            float x0 = 0.f, x1 = 0.f, x2 = 0.f, x3 = 0.f;
            if (live) {
                const int d = qk_dim<LAY>(ks, t);
                if (P.q_bf16) {
                    const uint2 w = *reinterpret_cast<const uint2 *>(
                        reinterpret_cast<const __nv_bfloat16 *>(P.q) + qoff + d);
                    x0 = __uint_as_float(w.x << 16);
                    x1 = __uint_as_float(w.x & 0xffff0000u);
                    x2 = __uint_as_float(w.y << 16);
                    x3 = __uint_as_float(w.y & 0xffff0000u);
                } else {
                    const float4 w =
                        *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(P.q) + qoff + d);
                    x0 = w.x; x1 = w.y; x2 = w.z; x3 = w.w;
                }
            }
            qf[nt][ks][0] = pack_h2(x0, x1);
            qf[nt][ks][1] = pack_h2(x2, x3);
        }
    }

    float m_run[NHT][2], l_run[NHT][2], acc[NHT][MT][4];
#pragma unroll
    for (int nt = 0; nt < NHT; nt++) {
        m_run[nt][0] = m_run[nt][1] = -CUDART_INF_F;
        l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
            acc[nt][mt][0] = acc[nt][mt][1] = acc[nt][mt][2] = acc[nt][mt][3] = 0.f;
    }

    /* One warp-step: 16 positions.  K rows are slots g, g+8 (pk); V rows are slots 2t, 2t+1, 2t+8,
     * 2t+9 (pv).  q8 layouts pass their codes and scales in registers; fp16 / fp32 rows are loaded
     * here from krow / vrow. */
    auto compute = [&](const int32_t (&pk)[2], const int32_t (&pv)[4], const uint2 (&kw)[2][NBQ],
                       const uint32_t (&vw)[4][NBQ], const float (&ksc)[2][NBQ], const __half (&vsc)[4][NBQ],
                       const uint8_t *const (&krow)[2], const uint8_t *const (&vrow)[4]) {
        /* ---- S^T = K . Q^T (log2 domain: scale * log2(e) folded in) */
        float sc[NHT][4];
#pragma unroll
        for (int nt = 0; nt < NHT; nt++) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
        if constexpr (Q8) {
#pragma unroll
            for (int b = 0; b < NB; b++) {
                float cb[NHT][4];
#pragma unroll
                for (int nt = 0; nt < NHT; nt++) cb[nt][0] = cb[nt][1] = cb[nt][2] = cb[nt][3] = 0.f;
#pragma unroll
                for (int jj = 0; jj < 2; jj++) {
                    uint32_t a0, a1, a2, a3;
                    cvt_i8x4(jj ? kw[0][b].y : kw[0][b].x, a0, a2);
                    cvt_i8x4(jj ? kw[1][b].y : kw[1][b].x, a1, a3);
#pragma unroll
                    for (int nt = 0; nt < NHT; nt++)
                        mma16816(cb[nt], a0, a1, a2, a3, qf[nt][2 * b + jj][0], qf[nt][2 * b + jj][1]);
                }
#pragma unroll
                for (int nt = 0; nt < NHT; nt++) {
                    sc[nt][0] = fmaf(ksc[0][b], cb[nt][0], sc[nt][0]);
                    sc[nt][1] = fmaf(ksc[0][b], cb[nt][1], sc[nt][1]);
                    sc[nt][2] = fmaf(ksc[1][b], cb[nt][2], sc[nt][2]);
                    sc[nt][3] = fmaf(ksc[1][b], cb[nt][3], sc[nt][3]);
                }
            }
        } else {
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                uint32_t a[4];
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    uint32_t lo = 0u, hi = 0u;
                    if (pk[r] >= 0) {
                        if constexpr (LAY == LAY_F16) {
                            const uint2 w = ldg64(krow[r] + (16 * ks + 4 * t) * 2);
                            lo = w.x; hi = w.y;
                        } else {
                            const uint4 w = ldg128(krow[r] + (16 * ks + 4 * t) * 4);
                            lo = pack_h2(__uint_as_float(w.x), __uint_as_float(w.y));
                            hi = pack_h2(__uint_as_float(w.z), __uint_as_float(w.w));
                        }
                    }
                    a[r] = lo; a[2 + r] = hi;
                }
#pragma unroll
                for (int nt = 0; nt < NHT; nt++)
                    mma16816(sc[nt], a[0], a[1], a[2], a[3], qf[nt][ks][0], qf[nt][ks][1]);
            }
#pragma unroll
            for (int nt = 0; nt < NHT; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) sc[nt][e] *= P.scale_log2e;
        }

        /* ---- online softmax; lanes (g, t) hold positions g / g+8 for heads 2t, 2t+1 */
        uint32_t pb0[NHT], pb1[NHT];
#pragma unroll
        for (int nt = 0; nt < NHT; nt++) {
            if (pk[0] < 0) sc[nt][0] = sc[nt][1] = -CUDART_INF_F;
            if (pk[1] < 0) sc[nt][2] = sc[nt][3] = -CUDART_INF_F;
            const float mx0 = warp_max_over_g(fmaxf(sc[nt][0], sc[nt][2]));
            const float mx1 = warp_max_over_g(fmaxf(sc[nt][1], sc[nt][3]));
            const float mn0 = fmaxf(m_run[nt][0], mx0), mn1 = fmaxf(m_run[nt][1], mx1);
            const float mu0 = mn0 == -CUDART_INF_F ? 0.f : mn0;
            const float mu1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
            const float al0 = ex2(m_run[nt][0] - mu0), al1 = ex2(m_run[nt][1] - mu1);
            m_run[nt][0] = mn0;
            m_run[nt][1] = mn1;
            const __half2 h0 = __floats2half2_rn(ex2(sc[nt][0] - mu0), ex2(sc[nt][1] - mu1));
            const __half2 h1 = __floats2half2_rn(ex2(sc[nt][2] - mu0), ex2(sc[nt][3] - mu1));
            l_run[nt][0] = fmaf(l_run[nt][0], al0, __low2float(h0) + __low2float(h1));
            l_run[nt][1] = fmaf(l_run[nt][1], al1, __high2float(h0) + __high2float(h1));
            if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    acc[nt][mt][0] *= al0; acc[nt][mt][1] *= al1;
                    acc[nt][mt][2] *= al0; acc[nt][mt][3] *= al1;
                }
            }
            pb0[nt] = movmatrix_t(h2u(h0));   /* {P[pos 2t][head g], P[pos 2t+1][head g]} */
            pb1[nt] = movmatrix_t(h2u(h1));   /* positions 2t+8, 2t+9 */
        }

        /* ---- O^T += V^T . P^T */
        if constexpr (Q8) {
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const __half2 s01 = __halves2half2(vsc[0][b], vsc[1][b]);
                const __half2 s23 = __halves2half2(vsc[2][b], vsc[3][b]);
                uint32_t bb0[NHT], bb1[NHT];
#pragma unroll
                for (int nt = 0; nt < NHT; nt++) {
                    bb0[nt] = h2u(__hmul2(u2h(pb0[nt]), s01));
                    bb1[nt] = h2u(__hmul2(u2h(pb1[nt]), s23));
                }
                {
                    const uint32_t a0 = cvt_i8_pair<0>(vw[0][b], vw[1][b]);
                    const uint32_t a1 = cvt_i8_pair<1>(vw[0][b], vw[1][b]);
                    const uint32_t a2 = cvt_i8_pair<0>(vw[2][b], vw[3][b]);
                    const uint32_t a3 = cvt_i8_pair<1>(vw[2][b], vw[3][b]);
#pragma unroll
                    for (int nt = 0; nt < NHT; nt++) mma16816(acc[nt][2 * b], a0, a1, a2, a3, bb0[nt], bb1[nt]);
                }
                {
                    const uint32_t a0 = cvt_i8_pair<2>(vw[0][b], vw[1][b]);
                    const uint32_t a1 = cvt_i8_pair<3>(vw[0][b], vw[1][b]);
                    const uint32_t a2 = cvt_i8_pair<2>(vw[2][b], vw[3][b]);
                    const uint32_t a3 = cvt_i8_pair<3>(vw[2][b], vw[3][b]);
#pragma unroll
                    for (int nt = 0; nt < NHT; nt++)
                        mma16816(acc[nt][2 * b + 1], a0, a1, a2, a3, bb0[nt], bb1[nt]);
                }
            }
        } else {
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                /* rows g / g+8 of the tile are dims 16mt+2g / 16mt+2g+1 */
                uint32_t lo[4], hi[4];
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    lo[r] = hi[r] = 0u;
                    if (pv[r] >= 0) {
                        if constexpr (LAY == LAY_F16) {
                            const uint32_t w = ldg32(vrow[r] + (16 * mt + 2 * g) * 2);
                            lo[r] = w & 0xffffu; hi[r] = w >> 16;
                        } else {
                            const uint2 w = ldg64(vrow[r] + (16 * mt + 2 * g) * 4);
                            const uint32_t h = pack_h2(__uint_as_float(w.x), __uint_as_float(w.y));
                            lo[r] = h & 0xffffu; hi[r] = h >> 16;
                        }
                    }
                }
                const uint32_t a0 = lo[0] | (lo[1] << 16), a1 = hi[0] | (hi[1] << 16);
                const uint32_t a2 = lo[2] | (lo[3] << 16), a3 = hi[2] | (hi[3] << 16);
#pragma unroll
                for (int nt = 0; nt < NHT; nt++) mma16816(acc[nt][mt], a0, a1, a2, a3, pb0[nt], pb1[nt]);
            }
        }
    };

    if constexpr (Cfg::STAGED) {
        /* ---- native q8_0 store, hd 128: every warp owns a ring of RING_STAGES 16-position stages that it
         * fills with 16-byte cp.async copies gathered by position.  Per tile the warp waits for the oldest
         * stage, moves the whole tile into registers as MMA fragments (ldmatrix for the K rows, transposing
         * ldmatrix for the V rows, the scale rows and the mask of live positions), refills the stage at once
         * with the tile RING_STAGES ahead, and only then does the arithmetic: all stages but the one being
         * unloaded are in flight all the time.  There is no block barrier in the loop.
         * Stage = the tile's 16 records, 272 bytes apart, as they lie in the store | mask word.  A tile of 16
         * consecutive positions (every tile of a dense scan, the recent window of a selection list) is one
         * contiguous span of the store and is copied 512 consecutive bytes per instruction; other tiles are
         * gathered row by row.  Padding positions copy nothing: their scale row is zeroed (so they add nothing to
         * P.V whatever the stale code bytes are) and their scores are masked. */
        const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem_raw) +
                              (uint32_t)warp * RING_STAGES * RING_STAGE_BYTES;
        const uint32_t n_my = s_begin + warp < s_end ? (s_end - s_begin - warp + DEC_WARPS - 1u) / DEC_WARPS : 0u;
        const uint32_t r16 = lane & 15, c8 = lane & 7;
        /* ldmatrix row address of this lane for block b: matrix lane / 8 = rows 8 * (that & 1) .., chunk 2b + lane / 16 */
        uint32_t moff[NB];
#pragma unroll
        for (int b = 0; b < NB; b++)
            moff[b] = (uint32_t)((lane & 7) + ((lane >> 3) & 1) * 8) * RING_ROW + (uint32_t)(2 * b + (lane >> 4)) * 16;
        /* one mbarrier per stage for the bulk copies, behind the rings of all warps (the epilogue never reaches
         * them); par: the phase each stage's barrier completes next */
        const uint32_t bars = (uint32_t)__cvta_generic_to_shared(smem_raw) + DEC_WARPS * RING_STAGES * RING_STAGE_BYTES +
                              (uint32_t)warp * RING_STAGES * 8;
        uint32_t par = 0;
        bool ring_dead = false;   /* a bulk copy never arrived within the probe limit: the block reports it and stops computing */
        if (P.bulk_runs) {
            if (lane < RING_STAGES) ring_bar_init(bars + lane * 8);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
        }

        /* The list entry is only loaded here; its range check waits until issue() needs the value, several
         * tiles later, so the load latency stays off the critical path. */
        auto my_pos = [&](uint32_t it) -> int32_t {
            const uint32_t j = ((s_begin + warp + it * DEC_WARPS) << 4) + r16;
            if (it >= n_my || j >= n_pos) return -1;
            return list ? list[j] : (int32_t)j;
        };
        auto issue = [&](uint32_t it, int32_t p) {
            if (it < n_my) {
                if (p >= (int32_t)bound) {
                    atomicOr(P.err, (uint32_t)Q4E_RANGE);
                    p = -1;
                }
                const uint32_t st = ring + (it % RING_STAGES) * RING_STAGE_BYTES;
                const uint32_t livemask = __ballot_sync(0xffffffffu, p >= 0) & 0xffffu;
                /* 16 consecutive positions: the tile is one contiguous span of the store */
                const int32_t p0 = __shfl_sync(0xffffffffu, p, 0);
                const bool run = __all_sync(0xffffffffu, p0 >= 0 && p == p0 + (int32_t)r16);
                if (run && P.bulk_runs) {
                    if (lane == 0) {
                        const uint32_t bar = bars + (it % RING_STAGES) * 8;
                        /* the stage was last read (and perhaps written) through the generic proxy */
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        ring_bar_expect(bar, 16 * RING_ROW);
                        bulk_copy_g2s(st, kbase + (uint64_t)(uint32_t)p0 * tok_stride, 16 * RING_ROW, bar);
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(st + RING_MASK_OFF), "r"(livemask | RING_RUN_BIT) : "memory");
                    }
                } else {
                    if (run) {
                        const uint8_t *src = kbase + (uint64_t)(uint32_t)p0 * tok_stride + lane * 16;
                        const uint32_t dst = st + lane * 16;
                        cp_async16_at<0>(dst, src);    cp_async16_at<512>(dst, src);  cp_async16_at<1024>(dst, src);
                        cp_async16_at<1536>(dst, src); cp_async16_at<2048>(dst, src); cp_async16_at<2560>(dst, src);
                        cp_async16_at<3072>(dst, src); cp_async16_at<3584>(dst, src);
                        if (lane < 16) cp_async16_at<4096>(dst, src);
                    } else {
#pragma unroll
                        for (uint32_t j = 0; j < 4; j++) {
                            const uint32_t row = 4 * j + (lane >> 3);
                            const int32_t pr = __shfl_sync(0xffffffffu, p, row);
                            cp_async16_kv<HD>(st + row * RING_ROW + c8 * 16, kbase + (uint64_t)(uint32_t)max(pr, 0) * tok_stride + c8 * 16, pr);
                        }
                        if (lane < 16)
                            cp_async16(st + r16 * RING_ROW + 2 * HD, kbase + (uint64_t)(uint32_t)max(p, 0) * tok_stride + 2 * HD, p >= 0);
                    }
                    if (lane == 0) asm volatile("st.shared.u32 [%0], %1;" ::"r"(st + RING_MASK_OFF), "r"(livemask) : "memory");
                }
            }
            cp_async_commit();   /* one group per tile, empty or not, keeps the wait count uniform */
        };
        /* ---- queries: the raw values are requested now, next to the list entries, and converted after the ring
         * has been filled (lane (g, t) takes dims 16ks + 4t .. + 3 of head nt*8 + g) */
        uint32_t qraw[NHT][KS][4];
#pragma unroll
        for (int nt = 0; nt < NHT; nt++) {
            const uint32_t hg = nt * 8 + g;
            const bool live = hg < P.gqa;
            const size_t qoff = ((size_t)u * P.n_head + (size_t)kh * P.gqa + hg) * HD;
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                qraw[nt][ks][0] = qraw[nt][ks][1] = qraw[nt][ks][2] = qraw[nt][ks][3] = 0u;
                if (live) {
                    const int d = 16 * ks + 4 * t;
                    if (P.q_bf16) {
                        const uint2 w = *reinterpret_cast<const uint2 *>(reinterpret_cast<const __nv_bfloat16 *>(P.q) + qoff + d);
                        qraw[nt][ks][0] = w.x; qraw[nt][ks][1] = w.y;
                    } else {
                        const uint4 w = *reinterpret_cast<const uint4 *>(reinterpret_cast<const float *>(P.q) + qoff + d);
                        qraw[nt][ks][0] = w.x; qraw[nt][ks][1] = w.y; qraw[nt][ks][2] = w.z; qraw[nt][ks][3] = w.w;
                    }
                }
            }
        }
        int32_t pa = my_pos(0), pb = my_pos(1), pc = my_pos(2), pd = my_pos(3);
        int32_t pn0 = my_pos(4), pn1 = my_pos(5), pn2 = my_pos(6);
        /* ---- fused append, second half.  Every split of the unit quantises and stores the unit's newest row
         * (identical bytes from every split, so no block depends on another having written); a block's own
         * store is ordered before its later reads by the barrier.  A warp whose first tiles do not name the
         * newest row fills its ring before that, so the append runs under the first copies. */
        bool hold = false;
        if (P.new_k) {
            const int32_t nw = (int32_t)newest;
            hold = __any_sync(0xffffffffu, pa == nw || pb == nw || pc == nw || pd == nw);
        }
        if (!hold) { issue(0, pa); issue(1, pb); issue(2, pc); issue(3, pd); }
        if (P.new_k) {
            float d, id;
            q4d_block_scale(ap_x, d, id);
            if (ap_live) {
                uint8_t *row = const_cast<uint8_t *>(kbase) + (uint64_t)newest * tok_stride;
                *reinterpret_cast<uint32_t *>(row + (ap_which ? HD : 0) + ap_b * 32 + ap_sub * 4) = q4d_quant4(ap_x, id);
                if (ap_sub == 0) reinterpret_cast<__half *>(row + 2 * HD)[(ap_which ? NB : 0) + ap_b] = __float2half_rn(d);
            }
            if (newest >= max_kv && threadIdx.x == 0) atomicOr(P.err, (uint32_t)Q4E_RANGE);
            if (P.bulk_runs) asm volatile("fence.proxy.async;" ::: "memory");   /* the row may be read back by the bulk-copy engine */
            __syncthreads();
        }
        if (hold) { issue(0, pa); issue(1, pb); issue(2, pc); issue(3, pd); }

        /* Q fragments as fp16 (exact for bf16 queries; scale * log2(e) multiplies the scores in fp32 later):
         * lane (g, t) holds dims 16ks + 4t .. + 3 of head nt*8 + g, the columns the K fragments below carry in
         * k-slots 2t, 2t+1, 2t+8, 2t+9.  And,
         * per 32-wide block, -1152 * sum(q): K codes enter the MMA as the fp16 numbers 1152 + code (one byte
         * permute per pair, no subtract), so each block's partial product starts from that correction. */
        uint32_t qs[NHT][KS][2];
        float qcorr[NHT][NB][2];
#pragma unroll
        for (int nt = 0; nt < NHT; nt++) {
            float bsum[NB];
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                float x0, x1, x2, x3;
                if (P.q_bf16) {
                    x0 = __uint_as_float(qraw[nt][ks][0] << 16);
                    x1 = __uint_as_float(qraw[nt][ks][0] & 0xffff0000u);
                    x2 = __uint_as_float(qraw[nt][ks][1] << 16);
                    x3 = __uint_as_float(qraw[nt][ks][1] & 0xffff0000u);
                } else {
                    x0 = __uint_as_float(qraw[nt][ks][0]); x1 = __uint_as_float(qraw[nt][ks][1]);
                    x2 = __uint_as_float(qraw[nt][ks][2]); x3 = __uint_as_float(qraw[nt][ks][3]);
                }
                const __half2 h0 = __floats2half2_rn(x0, x1);
                const __half2 h1 = __floats2half2_rn(x2, x3);
                qs[nt][ks][0] = h2u(h0);
                qs[nt][ks][1] = h2u(h1);
                const float part = (__low2float(h0) + __high2float(h0)) + (__low2float(h1) + __high2float(h1));
                if (ks & 1) bsum[ks >> 1] += part; else bsum[ks >> 1] = part;
            }
#pragma unroll
            for (int b = 0; b < NB; b++) {
                float v = bsum[b];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);     /* sum over the block for head nt*8+g */
                qcorr[nt][b][0] = -1152.f * __shfl_sync(0xffffffffu, v, (2 * t) * 4);
                qcorr[nt][b][1] = -1152.f * __shfl_sync(0xffffffffu, v, (2 * t + 1) * 4);
            }
        }

        for (uint32_t it = 0; it < n_my; it++) {
            cp_async_wait<RING_STAGES - 1>();    /* all but the newest RING_STAGES - 1 tiles have landed: tile `it` is in, if gathered */
            __syncwarp();
            const uint32_t st = ring + (it % RING_STAGES) * RING_STAGE_BYTES;
            const uint32_t livemask = lds32(st + RING_MASK_OFF);
            if (livemask & RING_RUN_BIT) {
                /* brought in by a bulk copy: bounded wait for its bytes on the stage's mbarrier; if they never come
                 * the block reports it and stops computing */
                const uint32_t sbit = 1u << (it % RING_STAGES), bar = bars + (it % RING_STAGES) * 8;
                uint32_t probes = 0;
                while (!ring_bar_test(bar, (par & sbit) ? 1u : 0u) && ++probes < RING_SPIN_LIMIT) {}
                par ^= sbit;
                if (__any_sync(0xffffffffu, probes >= RING_SPIN_LIMIT)) {
                    ring_dead = true;
                    break;
                }
            }
            /* ---- the tile into registers.  K: matrix i of block b = rows 8 (i & 1).., 16 dims from 32b + 16 (i >> 1):
             * kf[b][i] = position g (+8 for odd i), 4 codes of dims 32b + 16 (i >> 1) + 4t.  V, transposed:
             * vf[b][i] = positions 2t, 2t+1 (+8 for odd i), 2 codes each of dims 32b + 16 (i >> 1) + 2g, + 1. */
            uint32_t kf[NB][4], vf[NB][4];
#pragma unroll
            for (int b = 0; b < NB; b++) ldmatrix_x4(kf[b], st + moff[b]);
#pragma unroll
            for (int b = 0; b < NB; b++) ldmatrix_x4_trans(vf[b], st + RING_V_OFF + moff[b]);
            /* scale row of position r: K block scales, then V block scales */
            auto srow = [&](int r) -> uint32_t { return st + r * RING_ROW + 2 * HD; };
            const uint2 ks0 = lds64(srow(g)), ks1 = lds64(srow(g + 8));
            uint2 vs[4];
#pragma unroll
            for (int r = 0; r < 4; r++) vs[r] = lds64(srow(2 * t + (r & 1) + 8 * (r >> 1)) + 8);
            /* codes to offset binary: (code ^ 0x80) under the exponent byte 0x64 is the fp16 number 1152 + code */
#pragma unroll
            for (int b = 0; b < NB; b++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    kf[b][i] ^= 0x80808080u;
                    vf[b][i] ^= 0x80808080u;
                }
            __syncwarp();                        /* every lane has unloaded the stage */
            issue(it + RING_STAGES, pn0);        /* refill it with the tile RING_STAGES ahead */
            pn0 = pn1; pn1 = pn2;
            pn2 = my_pos(it + RING_STAGES + 3);

            /* ---- S^T = K . Q^T */
            const bool kok0 = (livemask >> g) & 1u, kok1 = (livemask >> (g + 8)) & 1u;
            float ksc[2][NB];
            {
                const float2 a01 = __half22float2(u2h(ks0.x)), a23 = __half22float2(u2h(ks0.y));
                const float2 b01 = __half22float2(u2h(ks1.x)), b23 = __half22float2(u2h(ks1.y));
                ksc[0][0] = a01.x; ksc[0][1] = a01.y; ksc[0][2] = a23.x; ksc[0][3] = a23.y;
                ksc[1][0] = b01.x; ksc[1][1] = b01.y; ksc[1][2] = b23.x; ksc[1][3] = b23.y;
            }
            float sc[NHT][4];
#pragma unroll
            for (int nt = 0; nt < NHT; nt++) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
            for (int b = 0; b < NB; b++) {
                float cb[NHT][4];
                {
                    const uint32_t a0 = __byte_perm(kf[b][0], 0x64646464u, 0x4140), a2 = __byte_perm(kf[b][0], 0x64646464u, 0x4342);
                    const uint32_t a1 = __byte_perm(kf[b][1], 0x64646464u, 0x4140), a3 = __byte_perm(kf[b][1], 0x64646464u, 0x4342);
#pragma unroll
                    for (int nt = 0; nt < NHT; nt++)
                        mma16816_from(cb[nt], a0, a1, a2, a3, qs[nt][2 * b][0], qs[nt][2 * b][1], qcorr[nt][b][0], qcorr[nt][b][1]);
                }
                {
                    const uint32_t a0 = __byte_perm(kf[b][2], 0x64646464u, 0x4140), a2 = __byte_perm(kf[b][2], 0x64646464u, 0x4342);
                    const uint32_t a1 = __byte_perm(kf[b][3], 0x64646464u, 0x4140), a3 = __byte_perm(kf[b][3], 0x64646464u, 0x4342);
#pragma unroll
                    for (int nt = 0; nt < NHT; nt++)
                        mma16816(cb[nt], a0, a1, a2, a3, qs[nt][2 * b + 1][0], qs[nt][2 * b + 1][1]);
                }
#pragma unroll
                for (int nt = 0; nt < NHT; nt++) {
                    sc[nt][0] = fmaf(ksc[0][b], cb[nt][0], sc[nt][0]);
                    sc[nt][1] = fmaf(ksc[0][b], cb[nt][1], sc[nt][1]);
                    sc[nt][2] = fmaf(ksc[1][b], cb[nt][2], sc[nt][2]);
                    sc[nt][3] = fmaf(ksc[1][b], cb[nt][3], sc[nt][3]);
                }
            }

            /* ---- online softmax in the log2 domain; lanes (g, t) hold positions g / g+8 for heads 2t, 2t+1 */
            uint32_t pb0[NHT], pb1[NHT];
#pragma unroll
            for (int nt = 0; nt < NHT; nt++) {
                sc[nt][0] = kok0 ? sc[nt][0] * P.scale_log2e : -CUDART_INF_F;
                sc[nt][1] = kok0 ? sc[nt][1] * P.scale_log2e : -CUDART_INF_F;
                sc[nt][2] = kok1 ? sc[nt][2] * P.scale_log2e : -CUDART_INF_F;
                sc[nt][3] = kok1 ? sc[nt][3] * P.scale_log2e : -CUDART_INF_F;
                const float mx0 = warp_max_over_g(fmaxf(sc[nt][0], sc[nt][2]));
                const float mx1 = warp_max_over_g(fmaxf(sc[nt][1], sc[nt][3]));
                const float mn0 = fmaxf(m_run[nt][0], mx0), mn1 = fmaxf(m_run[nt][1], mx1);
                const float mu0 = mn0 == -CUDART_INF_F ? 0.f : mn0;
                const float mu1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
                const float al0 = ex2(m_run[nt][0] - mu0), al1 = ex2(m_run[nt][1] - mu1);
                m_run[nt][0] = mn0;
                m_run[nt][1] = mn1;
                const __half2 h0 = __floats2half2_rn(ex2(sc[nt][0] - mu0), ex2(sc[nt][1] - mu1));
                const __half2 h1 = __floats2half2_rn(ex2(sc[nt][2] - mu0), ex2(sc[nt][3] - mu1));
                const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
                l_run[nt][0] = fmaf(l_run[nt][0], al0, f0.x + f1.x);
                l_run[nt][1] = fmaf(l_run[nt][1], al1, f0.y + f1.y);
                if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
                        acc[nt][mt][0] *= al0; acc[nt][mt][1] *= al1;
                        acc[nt][mt][2] *= al0; acc[nt][mt][3] *= al1;
                    }
                }
                pb0[nt] = movmatrix_t(h2u(h0));   /* {P[pos 2t][head g], P[pos 2t+1][head g]} */
                pb1[nt] = movmatrix_t(h2u(h1));   /* positions 2t+8, 2t+9 */
            }

            /* ---- O^T += V^T . P^T: tile mt = 16 dims, row g = dim 16mt + 2g, row g+8 = dim 16mt + 2g + 1 */
#pragma unroll
            for (int b = 0; b < NB; b++) {
                /* fp16 scale of block b: halves 0,1 in .x, halves 2,3 in .y */
                const uint32_t sel = (b & 1) ? 0x7632 : 0x5410;
                const uint32_t s01 = __byte_perm(b < 2 ? vs[0].x : vs[0].y, b < 2 ? vs[1].x : vs[1].y, sel);
                const uint32_t s23 = __byte_perm(b < 2 ? vs[2].x : vs[2].y, b < 2 ? vs[3].x : vs[3].y, sel);
                uint32_t bb0[NHT], bb1[NHT];
#pragma unroll
                for (int nt = 0; nt < NHT; nt++) {
                    bb0[nt] = h2u(__hmul2(u2h(pb0[nt]), u2h(s01)));
                    bb1[nt] = h2u(__hmul2(u2h(pb1[nt]), u2h(s23)));
                }
#pragma unroll
                for (int hf = 0; hf < 2; hf++) {
                    const uint32_t v01 = vf[b][2 * hf], v89 = vf[b][2 * hf + 1];
                    const uint32_t a0 = magic_sub(__byte_perm(v01, 0x64646464u, 0x4240));
                    const uint32_t a1 = magic_sub(__byte_perm(v01, 0x64646464u, 0x4341));
                    const uint32_t a2 = magic_sub(__byte_perm(v89, 0x64646464u, 0x4240));
                    const uint32_t a3 = magic_sub(__byte_perm(v89, 0x64646464u, 0x4341));
#pragma unroll
                    for (int nt = 0; nt < NHT; nt++) mma16816(acc[nt][2 * b + hf], a0, a1, a2, a3, bb0[nt], bb1[nt]);
                }
            }
        }
        cp_async_wait<0>();
        if (ring_dead) {
            /* bulk copies that may still be in flight must land (or the probe limit pass again) before the block
             * leaves its shared memory behind; barriers whose phase completed answer at once */
            for (uint32_t s_i = 0; s_i < RING_STAGES; s_i++)
                for (uint32_t probes = 0; probes < (RING_SPIN_LIMIT >> 6) && !ring_bar_test(bars + s_i * 8, (par >> s_i) & 1u); probes++) {}
            if (lane == 0) atomicOr(P.err, (uint32_t)Q4E_CUDA);
        }
        __syncthreads();    /* the epilogue below reuses the ring memory of all warps */
    } else {
        for (uint32_t step = s_begin + warp; step < s_end; step += DEC_WARPS) {
            const uint32_t j0 = step << 4;
            int32_t pk[2], pv[4];
            if (list) {
                const int32_t mine = position(j0 + (lane & 15));
                pk[0] = __shfl_sync(0xffffffffu, mine, g);
                pk[1] = __shfl_sync(0xffffffffu, mine, g + 8);
                pv[0] = __shfl_sync(0xffffffffu, mine, 2 * t);
                pv[1] = __shfl_sync(0xffffffffu, mine, 2 * t + 1);
                pv[2] = __shfl_sync(0xffffffffu, mine, 2 * t + 8);
                pv[3] = __shfl_sync(0xffffffffu, mine, 2 * t + 9);
            } else {
                pk[0] = position(j0 + g); pk[1] = position(j0 + g + 8);
                pv[0] = position(j0 + 2 * t); pv[1] = position(j0 + 2 * t + 1);
                pv[2] = position(j0 + 2 * t + 8); pv[3] = position(j0 + 2 * t + 9);
            }
            const uint8_t *krow[2], *vrow[4];
#pragma unroll
            for (int r = 0; r < 2; r++) krow[r] = kbase + (uint64_t)(pk[r] < 0 ? 0 : pk[r]) * tok_stride;
#pragma unroll
            for (int r = 0; r < 4; r++) vrow[r] = vbase + (uint64_t)(pv[r] < 0 ? 0 : pv[r]) * tok_stride;
            uint2 kw[2][NBQ];
            uint32_t vw[4][NBQ];
            float ksc[2][NBQ];
            __half vsc[4][NBQ];
            if constexpr (LAY == LAY_Q8P) {
#pragma unroll
                for (int r = 0; r < 2; r++)
#pragma unroll
                    for (int b = 0; b < NB; b++)
                        kw[r][b] = pk[r] >= 0 ? ldg64(krow[r] + 32 * b + 8 * t) : make_uint2(0u, 0u);
#pragma unroll
                for (int r = 0; r < 4; r++)
#pragma unroll
                    for (int b = 0; b < NB; b++)
                        vw[r][b] = pv[r] >= 0 ? ldg32(vrow[r] + 32 * b + 4 * g) : 0u;
                /* scale row: NB fp16 for K then NB fp16 for V */
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const uint8_t *sp = sbase + (uint64_t)(pk[r] < 0 ? 0 : pk[r]) * s_tok_stride;
                    __align__(16) __half h[NB];
                    if constexpr (NB == 4) { uint2 w = ldg64(sp); *reinterpret_cast<uint2 *>(h) = w; }
                    else if constexpr (NB == 8) { uint4 w = ldg128(sp); *reinterpret_cast<uint4 *>(h) = w; }
                    else if constexpr (NB == 2) { uint32_t w = ldg32(sp); *reinterpret_cast<uint32_t *>(h) = w; }
                    else { uint16_t w = (uint16_t)ldg16(sp); *reinterpret_cast<uint16_t *>(h) = w; }
#pragma unroll
                    for (int b = 0; b < NB; b++)
                        ksc[r][b] = pk[r] >= 0 ? __half2float(h[b]) * P.scale_log2e : 0.f;
                }
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    const uint8_t *sp = sbase + (uint64_t)(pv[r] < 0 ? 0 : pv[r]) * s_tok_stride + 2 * NB;
                    __align__(16) __half h[NB];
                    if constexpr (NB == 4) { uint2 w = ldg64(sp); *reinterpret_cast<uint2 *>(h) = w; }
                    else if constexpr (NB == 8) { uint4 w = ldg128(sp); *reinterpret_cast<uint4 *>(h) = w; }
                    else if constexpr (NB == 2) { uint32_t w = ldg32(sp); *reinterpret_cast<uint32_t *>(h) = w; }
                    else { uint16_t w = (uint16_t)ldg16(sp); *reinterpret_cast<uint16_t *>(h) = w; }
#pragma unroll
                    for (int b = 0; b < NB; b++) vsc[r][b] = pv[r] >= 0 ? h[b] : __ushort_as_half(0);
                }
            } else if constexpr (LAY == LAY_Q8R) {
                /* reference layout: 34-byte blocks {fp16 scale, 32 x int8}, only 2-byte aligned */
#pragma unroll
                for (int r = 0; r < 2; r++)
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        const uint8_t *bp = krow[r] + 34 * b;
                        if (pk[r] >= 0) {
                            const uint8_t *cp = bp + 2 + 8 * t;
                            kw[r][b].x = ldg16(cp) | (ldg16(cp + 2) << 16);
                            kw[r][b].y = ldg16(cp + 4) | (ldg16(cp + 6) << 16);
                            ksc[r][b] = __half2float(__ushort_as_half((uint16_t)ldg16(bp))) * P.scale_log2e;
                        } else {
                            kw[r][b] = make_uint2(0u, 0u);
                            ksc[r][b] = 0.f;
                        }
                    }
#pragma unroll
                for (int r = 0; r < 4; r++)
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        const uint8_t *bp = vrow[r] + 34 * b;
                        if (pv[r] >= 0) {
                            const uint8_t *cp = bp + 2 + 4 * g;
                            vw[r][b] = ldg16(cp) | (ldg16(cp + 2) << 16);
                            vsc[r][b] = __ushort_as_half((uint16_t)ldg16(bp));
                        } else {
                            vw[r][b] = 0u;
                            vsc[r][b] = __ushort_as_half(0);
                        }
                    }
            }
            compute(pk, pv, kw, vw, ksc, vsc, krow, vrow);
        }
    }

    /* ---- block reduction of the warps' partials ------------------------------------------- */
    float *sm = reinterpret_cast<float *>(smem_raw);   /* [DEC_WARPS][HEADS][REC] : acc[HD], m, l */
#pragma unroll
    for (int nt = 0; nt < NHT; nt++) {
        const float l0 = warp_sum_over_g(l_run[nt][0]), l1 = warp_sum_over_g(l_run[nt][1]);
        float *r0 = sm + ((size_t)warp * HEADS + nt * 8 + 2 * t) * REC;
        float *r1 = r0 + REC;
        if (g == 0) {
            r0[HD] = m_run[nt][0]; r0[HD + 1] = l0;
            r1[HD] = m_run[nt][1]; r1[HD + 1] = l1;
        }
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const int d0 = out_dim<LAY, Cfg::STAGED>(mt, g, 0), d1 = out_dim<LAY, Cfg::STAGED>(mt, g, 1);
            r0[d0] = acc[nt][mt][0]; r1[d0] = acc[nt][mt][1];
            r0[d1] = acc[nt][mt][2]; r1[d1] = acc[nt][mt][3];
        }
    }
    __syncthreads();

    const size_t unit = (size_t)u * P.n_kvh + kh;
    MergeOut mo;
    mo.out = P.out; mo.part_out = P.part_out; mo.gate = P.gate;
    mo.row0 = (size_t)u * P.n_head + (size_t)kh * P.gqa;
    mo.gqa = P.gqa;
    float *mscr = reinterpret_cast<float *>(smem_raw + Cfg::EPI_BYTES + Cfg::REC_BYTES);   /* scratch of the merges */
    /* exchange mode: the unit's last merge leaves this rank's record here instead of finalising */
    float *fin = P.xchg ? reinterpret_cast<float *>(smem_raw + Cfg::EPI_BYTES) : nullptr;
    if (S == 1) {
        merge_records<HD, HEADS>(sm, DEC_WARPS, false, fin, mo, mscr);
        if (fin) xchg_finish<HD, HEADS>(P.xchg, P.xchg_phase, (uint32_t)unit, fin, mo, P.err);
        return;
    }
    if (P.cluster) {
        float *own = reinterpret_cast<float *>(smem_raw + Cfg::EPI_BYTES);
        merge_records<HD, HEADS>(sm, DEC_WARPS, false, own, mo, mscr);
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   /* every peer block has started (arrive at entry) */
        if (P.push_bytes) {
            cluster_push_merge<HD, HEADS>(own, reinterpret_cast<const float *>(smem_raw + Cfg::SMEM), S, cluster_ctarank(), mo,
                                          P.push_async ? (uint32_t)__cvta_generic_to_shared(smem_raw + Cfg::SMEM + P.push_bytes - 16u) : 0u,
                                          P.err);
            return;
        }
        cluster_sync_all();
        cluster_merge<HD, HEADS>((uint32_t)__cvta_generic_to_shared(own), S, cluster_ctarank(), mo);
        cluster_sync_all();
        return;
    }
    /* level 1: record per block; groups of DEC_GROUP blocks are merged by their last arrival,
     * level 2: the group records are merged by the last group to finish. */
    const uint32_t n_groups = (S + DEC_GROUP - 1u) / DEC_GROUP;
    const uint32_t grp = split / DEC_GROUP;
    const uint32_t grp_size = min(DEC_GROUP, S - grp * DEC_GROUP);
    float *rec1 = P.scratch + (unit * (size_t)(S + n_groups)) * HEADS * REC;
    if (P.gridmerge) {
        merge_records<HD, HEADS>(sm, DEC_WARPS, false, rec1 + (size_t)split * HEADS * REC, mo, mscr);
        __syncthreads();   /* the warp records in shared memory are no longer needed: their space is the scratch */
        grid_merge<HD, HEADS>(rec1, S, split, P.counters + unit * (1u + DEC_MAX_SPLIT / DEC_GROUP), mo, sm, P.err);
        return;
    }
    float *rec2 = rec1 + (size_t)S * HEADS * REC;
    uint32_t *ctr = P.counters + unit * (1u + DEC_MAX_SPLIT / DEC_GROUP);
    /* one call site for every level keeps a single copy of the merge code in the kernel */
    const float *src = sm;
    uint32_t count = DEC_WARPS;
    bool global = false;
    float *dst = rec1 + (size_t)split * HEADS * REC;
    uint32_t *arrive = ctr + 1 + grp;
    uint32_t expected = grp_size;
    bool last = false;
    for (int level = 0;; level++) {
        merge_records<HD, HEADS>(src, count, global, dst, mo, mscr);
        if (last) {                                        /* finalised, or this rank's record is complete */
            if (fin) xchg_finish<HD, HEADS>(P.xchg, P.xchg_phase, (uint32_t)unit, fin, mo, P.err);
            return;
        }
        if (!arrive_last(arrive, expected)) return;        /* someone else carries on */
        global = true;
        if (level == 0) {
            src = rec1 + (size_t)grp * DEC_GROUP * HEADS * REC;
            count = grp_size;
            last = n_groups == 1;
            dst = last ? nullptr : rec2 + (size_t)grp * HEADS * REC;
            arrive = ctr;
            expected = n_groups;
        } else {
            src = rec2;
            count = n_groups;
            last = true;
            dst = nullptr;
        }
        if (last) dst = fin;
    }
}

/* Merge of externally produced records (sequence-sharded decode): parts [n_parts][n_head][hd+2]
 * with m in natural-log units, as gqa_dec_comb_k (src/q4_rocm.cu:6968-7012). */
__global__ void q4_lse_merge_k(const float *parts, uint32_t n_parts, uint32_t n_head, uint32_t hd,
                               const float *gate, float *out) {
    const uint32_t h = blockIdx.x, rec = hd + 2;
    float M = -CUDART_INF_F;
    for (uint32_t s = 0; s < n_parts; s++) {
        const float *r = parts + ((size_t)s * n_head + h) * rec;
        if (r[1] > 0.f) M = fmaxf(M, r[0]);
    }
    float L = 0.f;
    for (uint32_t s = 0; s < n_parts; s++) {
        const float *r = parts + ((size_t)s * n_head + h) * rec;
        if (r[1] > 0.f) L = fmaf(__expf(r[0] - M), r[1], L);
    }
    for (uint32_t d = threadIdx.x; d < hd; d += blockDim.x) {
        float A = 0.f;
        for (uint32_t s = 0; s < n_parts; s++) {
            const float *r = parts + ((size_t)s * n_head + h) * rec;
            if (r[1] > 0.f) A = fmaf(__expf(r[0] - M), r[2 + d], A);
        }
        float o = L > 0.f ? A / L : 0.f;
        if (gate) o *= 1.f / (1.f + __expf(-gate[(size_t)h * hd + d]));
        out[(size_t)h * hd + d] = o;
    }
}

template <int LAY, int HD, int NHT>
bool launch(const DecParams &p_in, dim3 grid) {
    constexpr size_t smem_base = DecCfg<LAY, HD, NHT>::SMEM;
    constexpr size_t SMEM_LIMIT = smem_base + 2u * DEC_CLUSTER_MAX * (HD + 4) * sizeof(float) + 16u;   /* ring / epilogue + the largest receive area of the push merge */
    static bool attr_done = false;
    if (!attr_done) {
        if (!q4i_check(cudaFuncSetAttribute(q4_decode_k<LAY, HD, NHT>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT),
                       "decode smem attribute"))
            return false;
        (void)cudaFuncSetAttribute(q4_decode_k<LAY, HD, NHT>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    }
    attr_done = true;
    DecParams p = p_in;
    const uint64_t blocks = (uint64_t)grid.x * grid.y * grid.z;
    /* how many clusters of this shape can be resident at once with `bytes` of dynamic shared memory per block */
    auto resident_clusters = [&](size_t bytes) -> uint64_t {
        static size_t c_bytes[4];
        static uint32_t c_cluster[4];
        static int c_n[4], c_used = 0;
        for (int i = 0; i < c_used; i++)
            if (c_bytes[i] == bytes && c_cluster[i] == p.cluster) return (uint64_t)c_n[i];
        cudaLaunchConfig_t qc;
        memset(&qc, 0, sizeof(qc));
        qc.gridDim = grid;
        qc.blockDim = dim3(DEC_THREADS);
        qc.dynamicSmemBytes = bytes;
        cudaLaunchAttribute qa[1];
        qa[0].id = cudaLaunchAttributeClusterDimension;
        qa[0].val.clusterDim.x = p.cluster;
        qa[0].val.clusterDim.y = 1;
        qa[0].val.clusterDim.z = 1;
        qc.attrs = qa;
        qc.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, q4_decode_k<LAY, HD, NHT>, &qc) != cudaSuccess) {
            (void)cudaGetLastError();
            n = 0;
        }
        const int slot = c_used < 4 ? c_used++ : 3;
        c_bytes[slot] = bytes; c_cluster[slot] = p.cluster; c_n[slot] = n;
        return (uint64_t)n;
    };
    /* The push merge needs extra shared memory; it is used only if that leaves the grid in one wave.
     * (Asking for still more shared memory, so that a shallow grid spreads one or two blocks deep over all
     * SMs instead of three deep over some, was measured: no gain at 1-8 sessions, 3 us slower at 16.) */
    if (p.push_bytes && resident_clusters(smem_base + p.push_bytes) < blocks / p.cluster) p.push_bytes = 0;
    if (!p.push_bytes) p.push_async = 0;
    if (p.gridmerge) {
        /* the blocks of a unit wait for one another: only when the whole grid is resident at once */
        static int occ = -1;
        if (occ < 0 && cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, q4_decode_k<LAY, HD, NHT>, DEC_THREADS, smem_base) != cudaSuccess) {
            (void)cudaGetLastError();
            occ = 0;
        }
        if (blocks > (uint64_t)occ * (uint64_t)g_q4.sm_count) p.gridmerge = 0;
    }
    const size_t smem = smem_base + p.push_bytes;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = dim3(DEC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = g_q4.stream;
    cudaLaunchAttribute at[3];
    unsigned n_at = 0;
    if (p.cluster) {
        at[n_at].id = cudaLaunchAttributeClusterDimension;
        at[n_at].val.clusterDim.x = p.cluster;
        at[n_at].val.clusterDim.y = 1;
        at[n_at].val.clusterDim.z = 1;
        n_at++;
        /* Where the blocks of a cluster land: the load-balancing preference keeps a shallow grid one or two
         * blocks deep on every SM where the default stacks three on some (8 sessions: 8.7 against 9.8 us per
         * launch with clusters of 12); no effect on full grids.  Q4_DEC_CLUSTER_POLICY=0 leaves the choice to the
         * driver, 1 asks for the spread policy. */
        static int pol = -1;
        if (pol < 0) { const char *e = getenv("Q4_DEC_CLUSTER_POLICY"); pol = e ? atoi(e) : 2; }
        if (pol) {
            at[n_at].id = cudaLaunchAttributeClusterSchedulingPolicyPreference;
            at[n_at].val.clusterSchedulingPolicyPreference = pol == 1 ? cudaClusterSchedulingPolicySpread : cudaClusterSchedulingPolicyLoadBalancing;
            n_at++;
        }
    }
    if (p.pdl) {
        at[n_at].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[n_at].val.programmaticStreamSerializationAllowed = 1;
        n_at++;
    }
    cfg.attrs = at;
    cfg.numAttrs = n_at;
    return q4i_check(cudaLaunchKernelEx(&cfg, q4_decode_k<LAY, HD, NHT>, p), "decode launch");
}
template <int LAY, int HD>
bool launch_nht(const DecParams &p, dim3 grid) {
    return p.gqa <= 8 ? launch<LAY, HD, 1>(p, grid) : launch<LAY, HD, 2>(p, grid);
}
template <int LAY>
bool launch_hd(const DecParams &p, dim3 grid, uint32_t hd) {
    switch (hd) {
    case 32: return launch_nht<LAY, 32>(p, grid);
    case 64: return launch_nht<LAY, 64>(p, grid);
    case 128: return launch_nht<LAY, 128>(p, grid);
    case 256: return launch_nht<LAY, 256>(p, grid);
    }
    return q4i_fail(Q4E_ARG, "decode: hd must be 32, 64, 128 or 256");
}

uint32_t split_override() {
    /* same knob as the reference (Q4_DEC_SPLIT_S, src/q4_rocm.cu:6750-6760); 0 = automatic */
    static int s = -1;
    if (s < 0) {
        const char *e = getenv("Q4_DEC_SPLIT_S");
        long v = e ? strtol(e, nullptr, 10) : 0;
        s = (int)(v < 0 ? 0 : v > (long)DEC_MAX_SPLIT ? (long)DEC_MAX_SPLIT : v);
    }
    return (uint32_t)s;
}

}  // namespace

bool q4i_decode(const Q4DecodeArgs &a) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "decode: library not initialised");
    Q4_REQUIRE(a.q && (a.out || a.part_out) && a.n_units && a.n_head && a.n_kvh, "decode: null/zero argument");
    Q4_REQUIRE(a.n_head % a.n_kvh == 0 && a.n_head / a.n_kvh <= 16, "decode: n_head/n_kvh must be 1..16");
    Q4_REQUIRE(!a.idx || a.width, "decode: zero-width index list");
    const uint32_t gqa = a.n_head / a.n_kvh;
    const uint32_t heads = gqa <= 8 ? 8 : 16;

    /* split so that the grid fills every SM a few blocks deep, each block keeping its warps busy */
    const uint32_t rows = a.idx ? a.width : (a.hint_rows ? a.hint_rows : 1u);
    const uint32_t steps = (rows + 15u) / 16u;
    const uint32_t units = a.n_units * a.n_kvh;
    uint32_t S = split_override();
    if (!S) {
        /* one wave of 3 resident blocks per SM */
        const uint32_t target = (uint32_t)g_q4.sm_count * 3u;
        S = target / units;
        /* several units of unequal length (dense batch): finer slices so the block scheduler can balance */
        if (!a.idx && a.n_units > 1) S = S > (steps + 63u) / 64u ? S : (steps + 63u) / 64u;
        /* every warp keeps at least one tile of a list, four of a dense scan (measured at 16384 / 32768 rows:
         * 12.0 / 14.6 us per layer against 13.5 / 15.4 with one tile per warp; no difference from 49152 rows on) */
        const uint32_t per_block = (a.idx || a.xchg) ? DEC_WARPS : 4u * DEC_WARPS;   /* the exchange form merges in two levels: finer splits serve it better (8 ranks x 32768 rows: 24.7 against 26.0 us) */
        const uint32_t cap = (steps + per_block - 1u) / per_block;
        if (S > cap) S = cap;
    }
    if (S > DEC_MAX_SPLIT) S = DEC_MAX_SPLIT;
    if (S > DEC_GROUP && S < 2 * DEC_GROUP) S = DEC_GROUP;   /* one merge level instead of two */
    if (S < 1) S = 1;
    /* Short lists (a few hundred tiles per unit) are bound by the latency of the merge, not by bandwidth:
     * at most 8 splits (16 when only a few units are in flight), launched as one cluster per unit, merge
     * through distributed shared memory. */
    static int use_cluster = -1;
    if (use_cluster < 0) {
        const char *e = getenv("Q4_DEC_CLUSTER");
        use_cluster = e ? atoi(e) : 1;
    }
    uint32_t cluster = 0;   /* blocks per cluster; 0 = plain launch with the merge in global memory */
    if (a.xchg) Q4_REQUIRE(a.n_units == 1 && a.out && !a.part_out && !a.many, "decode: exchange mode is for one token of one session");
    if (use_cluster && !a.scratch_part && !a.xchg && (S <= 8 || steps <= 512)) {
        /* A few units only (single session, small batch): larger clusters shorten each warp's share, as long as
         * the blocks still spread one or two deep over the SMs.  Measured with the load-balancing placement, us
         * per launch at 2 / 4 / 8 / 16 sessions of 2 kv heads: clusters of 16: 7.3 / 7.7 / 10.5 / 18.6, of 13:
         * 7.3 / 7.7 / 8.5 / 18.6, of 12: 7.4 / 7.8 / 8.7 / 12.2, of 8: - / 8.7 / 10.0 / 13.3. */
        const uint32_t sms = (uint32_t)g_q4.sm_count;
        const uint32_t cmax = steps < 8u * DEC_CLUSTER_MAX ? 8u
                              : units * 32u <= sms ? DEC_CLUSTER_MAX
                              : units * 26u <= sms * 3u ? 13u
                              : units * 60u <= sms * 13u ? 12u : 8u;
        if (S > cmax) S = cmax;
        cluster = S > 1 ? S : 0u;
    }

    if (a.scratch_part && a.scratch_clamp) {
        /* fixed-size caller scratch: fewer splits until the records fit */
        while (S > 1 && (size_t)units * (S + (S + DEC_GROUP - 1u) / DEC_GROUP) * heads * (a.hd + 4) > a.scratch_part_floats)
            S--;
    }
    const uint32_t n_groups = (S + DEC_GROUP - 1u) / DEC_GROUP;
    const size_t need_part = (size_t)units * (S + n_groups) * heads * (a.hd + 4);
    const size_t need_ctr = (size_t)units * (1u + DEC_MAX_SPLIT / DEC_GROUP);
    float *scratch = a.scratch_part;
    uint32_t *counters = a.scratch_counters;
    if (scratch) {
        if ((S > 1 && a.scratch_part_floats < need_part) || a.scratch_n_counters < need_ctr)
            return q4i_fail(Q4E_SCRATCH, "decode: caller scratch too small");
    } else {
        if (!q4i_scratch(S > 1 && cluster != S ? need_part : 0, need_ctr)) return false;
        scratch = g_q4.part;
        counters = g_q4.counters;
    }

    DecParams p;
    p.one = a.one;
    p.many = a.many;
    p.layer = a.layer;
    p.n_head = a.n_head;
    p.n_kvh = a.n_kvh;
    p.gqa = gqa;
    p.q = a.q;
    p.q_bf16 = a.q_bf16;
    p.gate = a.gate;
    p.out = a.out;
    p.part_out = a.part_out;
    p.idx = a.idx;
    p.width = a.width;
    p.idx_kvh_stride = a.idx_kvh_stride;
    p.idx_unit_stride = a.idx_unit_stride;
    p.pos = a.pos;
    p.kv_base = a.kv_base;
    p.idx_bound_nkv = a.idx_bound_nkv ? 1u : 0u;
    p.scale_log2e = a.scale * 1.4426950408889634f;
    p.S = S;
    p.cluster = cluster;
    /* the push merge needs extra shared memory; the launcher drops it where that would cost a wave */
    p.push_bytes = cluster > 1 ? ((gqa + cluster - 1u) / cluster) * cluster * (a.hd + 4u) * (uint32_t)sizeof(float) + 16u : 0u;
    {
        /* Q4_DEC_PUSH_ASYNC=0: the pushes meet at a cluster barrier instead of completing the receiver's mbarrier */
        static int pa = -1;
        if (pa < 0) { const char *e = getenv("Q4_DEC_PUSH_ASYNC"); pa = e ? atoi(e) : 1; }
        p.push_async = p.push_bytes && pa ? 1u : 0u;
    }
    p.scratch = scratch;
    p.counters = counters;
    p.err = g_q4.err_d;
    {
        /* Bulk copies for runs of consecutive positions pay off on dense scans (every tile is a run: one copy
         * instruction per tile instead of nine); in a gathered list they are slower than coalesced cp.async
         * (measured: 64-session batch 27.4 vs 26.6 us, single session 8.3 vs 7.9 us).  Q4_DEC_BULK=0 / 1 forces
         * the choice. */
        static int bulk = -2;
        if (bulk == -2) { const char *e = getenv("Q4_DEC_BULK"); bulk = e ? atoi(e) : -1; }
        p.bulk_runs = bulk >= 0 ? (bulk ? 1u : 0u) : (a.idx ? 0u : 1u);
    }
    {
        /* Q4_DEC_GRIDMERGE=0: long scans merge in two levels, each by the last block of a group to arrive */
        static int gm = -1;
        if (gm < 0) { const char *e = getenv("Q4_DEC_GRIDMERGE"); gm = e ? atoi(e) : 1; }
        p.gridmerge = (gm && !cluster && S > DEC_GROUP && !a.xchg) ? 1u : 0u;
    }
    p.xchg = a.xchg;
    p.xchg_phase = (uint32_t)a.xchg_phase;
    p.new_k = a.new_k;
    p.new_v = a.new_v;
    {
        /* Q4_DEC_PDL=0 switches programmatic dependent launch off */
        static int pdl = -1;
        if (pdl < 0) { const char *e = getenv("Q4_DEC_PDL"); pdl = e ? atoi(e) : 1; }
        p.pdl = pdl ? 1u : 0u;
    }
    if (a.new_k || a.new_v)
        Q4_REQUIRE(a.new_k && a.new_v && a.layout == LAY_Q8P && a.hd == 128,
                   "decode: fused append needs both rows and the native q8_0 store at hd 128");
    dim3 grid(S, a.n_kvh, a.n_units);
    switch (a.layout) {
    case LAY_F32: return launch_hd<LAY_F32>(p, grid, a.hd);
    case LAY_F16: return launch_hd<LAY_F16>(p, grid, a.hd);
    case LAY_Q8P: return launch_hd<LAY_Q8P>(p, grid, a.hd);
    case LAY_Q8R: return launch_hd<LAY_Q8R>(p, grid, a.hd);
    }
    return q4i_fail(Q4E_ARG, "decode: bad layout");
}

namespace {
template <int HD>
bool launch_xchg_merge(const q4_gpu_xchg *x, uint32_t gqa, const float *gate, float *out) {
    if (gqa <= 8) q4_xchg_merge_k<HD, 8><<<x->n_kvh, DEC_THREADS, 0, g_q4.stream>>>(x->dev, gqa, gate, out, g_q4.err_d);
    else q4_xchg_merge_k<HD, 16><<<x->n_kvh, DEC_THREADS, 0, g_q4.stream>>>(x->dev, gqa, gate, out, g_q4.err_d);
    return q4i_check(cudaGetLastError(), "exchange merge launch");
}
}  // namespace
bool q4i_xchg_merge(const q4_gpu_xchg *x, const float *gate, float *out) {
    const uint32_t gqa = x->n_head / x->n_kvh;
    switch (x->hd) {
    case 32: return launch_xchg_merge<32>(x, gqa, gate, out);
    case 64: return launch_xchg_merge<64>(x, gqa, gate, out);
    case 128: return launch_xchg_merge<128>(x, gqa, gate, out);
    case 256: return launch_xchg_merge<256>(x, gqa, gate, out);
    }
    return q4i_fail(Q4E_ARG, "exchange merge: hd must be 32, 64, 128 or 256");
}

extern "C" bool q4_gpu_lse_merge(const float *parts, uint32_t n_parts, uint32_t n_head, uint32_t hd,
                                 const float *gate, float *out) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "lse_merge: library not initialised");
    Q4_REQUIRE(parts && out && n_parts && n_head && hd, "lse_merge: null/zero argument");
    q4_lse_merge_k<<<n_head, 128, 0, g_q4.stream>>>(parts, n_parts, n_head, hd, gate, out);
    return q4i_check(cudaGetLastError(), "lse_merge launch");
}

/* ---- decode without any allocation ------------------------------------------------------------
 * Scratch for the split-KV records lives in the library image itself: every GPU that loads the
 * library holds these 4 MB + 272 B until the process exits.  The names below are host-side stand-ins
 * in host code; the device addresses come from cudaGetSymbolAddress, once per device. */
constexpr size_t Q4_STATIC_PART_FLOATS = (size_t)1 << 20;   /* 4 MB of records */
constexpr size_t Q4_STATIC_COUNTERS = 4 * (1 + DEC_MAX_SPLIT / DEC_GROUP);   /* up to 4 kv heads */
static __device__ __align__(256) float q4_static_part[Q4_STATIC_PART_FLOATS];
static __device__ __align__(256) uint32_t q4_static_counters[Q4_STATIC_COUNTERS];

extern "C" bool q4_gpu_kv_decode_noalloc(const q4_gpu_kv *kv, uint32_t layer, const void *q, int q_bf16,
                                         const float *gate, float *out, uint32_t n_head, const int32_t *idx,
                                         uint32_t width, uint32_t idx_kvh_stride, uint32_t n_kv, float scale) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "kv_decode_noalloc: library not initialised");
    Q4_REQUIRE(kv && q && out && layer < kv->n_layers && n_head, "kv_decode_noalloc: bad argument");
    Q4_REQUIRE(n_kv <= kv->max_kv, "kv_decode_noalloc: n_kv beyond max_kv");
    if (kv->n_kvh > 4 || n_head % kv->n_kvh || n_head / kv->n_kvh > 16)
        return q4i_fail(Q4E_SCRATCH, "kv_decode_noalloc: shape beyond the built-in scratch (at most 4 kv heads, "
                                     "16 query heads per kv head)");
    /* set-up, once per device, with that device current: resolve the arrays' device addresses */
    static float *part_dev[64];
    static uint32_t *ctr_dev[64];
    int dev = -1;
    if (!q4i_check(cudaGetDevice(&dev), "kv_decode_noalloc: cudaGetDevice")) return false;
    if (dev < 0 || dev >= 64) return q4i_fail(Q4E_ARG, "kv_decode_noalloc: device index out of range");
    if (!part_dev[dev]) {
        float *p = nullptr;
        uint32_t *c = nullptr;
        if (!q4i_check(cudaGetSymbolAddress((void **)&p, q4_static_part), "kv_decode_noalloc: symbol address (records)"))
            return false;
        if (!q4i_check(cudaGetSymbolAddress((void **)&c, q4_static_counters), "kv_decode_noalloc: symbol address (counters)"))
            return false;
        part_dev[dev] = p;
        ctr_dev[dev] = c;
    }
    /* the arrival counters must start at zero; the records need no clearing (every record that is
     * read has been written by this launch) */
    if (!q4i_check(cudaMemsetAsync(ctr_dev[dev], 0, Q4_STATIC_COUNTERS * sizeof(uint32_t), g_q4.stream),
                   "kv_decode_noalloc: counter clear"))
        return false;
    Q4DecodeArgs a;
    memset(&a, 0, sizeof(a));
    a.one = kv->view;
    a.layout = kv->kind == Q4K_Q8 ? LAY_Q8P : kv->kind == Q4K_F16 ? LAY_F16 : LAY_F32;
    a.layer = layer;
    a.n_units = 1;
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
    if (n_kv) {
        a.kv_base = n_kv - 1;
        a.hint_rows = n_kv;
    } else {
        a.pos = g_q4.pos_d;
        a.hint_rows = kv->max_kv;
    }
    a.idx_bound_nkv = 1;
    a.scale = scale;
    a.scratch_part = part_dev[dev];
    a.scratch_counters = ctr_dev[dev];
    a.scratch_part_floats = Q4_STATIC_PART_FLOATS;
    a.scratch_n_counters = Q4_STATIC_COUNTERS;
    a.scratch_clamp = 1;
    return q4i_decode(a);
}
