/*
 * QSA indexer: the step that produces the 2051-wide selection lists the sparse decode consumes.
 *
 *   pool   qsa_pool_k / qsa_pool_dk (src/q4_rocm.cu:7366-7402, 7880-7933): block b of `ratio` tokens =
 *          mean of their raw fp16 keys, RMSNorm, RoPE at the block's first position, fp32 [block][128]
 *   score  qsa_score_k / qsa_score_dk (:7405-7436, 7469-7502): score[b] = sum_h relu(q_h . pool[b])
 *          over the blocks the token can see -- at ctx 262 144 a 33.5 MB scan per layer, 30x the
 *          bytes of the sparse attention it feeds, so this is the HBM-bound part
 *   top-k  qsa_topk_k / the qsa_tk_* family (:7506-7666, 7722-7846): exact top-512 blocks by (score
 *          descending, index ascending), expanded to positions plus the newest partial block
 *
 * Results are defined by the reference down to the order of the list, so the arithmetic keeps its
 * association: the sum of squares is the same pairwise tree, a dot product is one fused multiply-add
 * per dim in dim order (four heads = four independent chains per thread), and the selection is an
 * exact radix select followed by an index-ordered compaction.  What changes is the mapping: a warp
 * per pooled block with the tree in shuffles, a thread per pooled block for the scan with each warp's
 * 32 rows staged in shared memory by coalesced asynchronous copies, and ONE launch per token for the
 * whole selection instead of the reference's 12: a cluster of 8 blocks with the keys in registers, the
 * histograms summed through distributed shared memory, the digit picked by a warp scan, ballot ranks
 * and scans over warps and blocks for the ordered emit (rows longer than 65 536 blocks: one block that
 * re-reads the row, 16 independent loads at a time).
 */
#include <math_constants.h>
#include <string.h>

#include "q4_internal.h"

namespace {

constexpr uint32_t IX_HD = 128;
constexpr uint32_t IX_TK_THREADS = 1024, IX_MAX_KBLK = 512;

/* ---- pool: one warp per block, lane l holds dims l, l+32, l+64, l+96 */
__global__ void __launch_bounds__(128) q4_ix_pool_k(const __half *raw, float *pool, const float *wn, uint32_t ratio,
                                                    uint32_t b0, uint32_t b1, uint32_t n_rot, float base, float eps,
                                                    const int32_t *pp) {
    const uint32_t lane = threadIdx.x & 31u, w = blockIdx.x * 4u + (threadIdx.x >> 5);
    if (pp) {   /* device position: the block this token completes, if any */
        const uint32_t pos = (uint32_t)*pp;
        b0 = pos / ratio;
        b1 = (pos + 1u) / ratio;
    }
    const uint32_t b = b0 + w;
    if (b >= b1) return;
    const __half *src = raw + (size_t)b * ratio * IX_HD;
    float v[4], r[4];
#pragma unroll
    for (int c = 0; c < 4; c++) {
        float s = 0.f;
        for (uint32_t j = 0; j < ratio; j++) s += __half2float(src[(size_t)j * IX_HD + lane + 32u * c]);
        v[c] = __fdiv_rn(s, (float)ratio);
        r[c] = __fmul_rn(v[c], v[c]);
    }
    /* red[d] += red[d + st] for st = 64, 32 is local to the lane; 16 .. 1 are shuffles */
    float a = __fadd_rn(__fadd_rn(r[0], r[2]), __fadd_rn(r[1], r[3]));
#pragma unroll
    for (int st = 16; st > 0; st >>= 1) a = __fadd_rn(a, __shfl_down_sync(0xffffffffu, a, st));
    const float tot = __shfl_sync(0xffffffffu, a, 0);
    const float inv = rsqrtf(__fadd_rn(__fdiv_rn(tot, (float)IX_HD), eps));
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const uint32_t d = lane + 32u * c;
        v[c] = __fmul_rn(__fmul_rn(v[c], inv), wn ? wn[d] : 1.f);
    }
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const uint32_t d = lane + 32u * c;
        const float other = __shfl_xor_sync(0xffffffffu, v[c], 1);
        if ((d & ~1u) < n_rot) {
            const uint32_t p = d >> 1;
            const float freq = powf(base, -(float)p / (float)(n_rot / 2u));
            const float ang = (float)(b * ratio) * freq;
            const float cs = cosf(ang), sn = sinf(ang);
            /* even dim: x0 * c - x1 * s; odd dim: x0 * s + x1 * c, with (x0, x1) the pair */
            v[c] = (d & 1u) ? __fadd_rn(__fmul_rn(other, sn), __fmul_rn(v[c], cs))
                            : __fsub_rn(__fmul_rn(v[c], cs), __fmul_rn(other, sn));
        }
        pool[(size_t)b * IX_HD + d] = v[c];
    }
}

/* ---- score: one thread per pooled block, 4 heads = 4 fused-multiply-add chains in dim order.
 * Persistent warps: a warp takes every n-th tile of 32 rows (512 B each), brings the next tile into
 * the other of its two shared-memory buffers with one 16-byte asynchronous copy per lane and row --
 * fully coalesced, 16 KB in flight per warp while the previous tile is being scored -- and every lane
 * walks its own row there.  Rows are 132 floats apart: 16-byte reads of eight consecutive rows fall
 * into eight different bank groups, so the walk is conflict free; the query is read as a broadcast. */
/* Programmatic dependent launch: the blocks of a launch may become resident while the previous kernel of
 * the stream drains; nothing the previous kernels write (position word, pool, scores, queries) is read
 * before this point.  A no-op for a launch without the attribute. */
__device__ __forceinline__ void ix_pdl_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
/* Q4_IX_PDL=0 switches it off for the score and selection launches */
bool ix_pdl() {
    static int on = -1;
    if (on < 0) { const char *e = getenv("Q4_IX_PDL"); on = e ? atoi(e) : 1; }
    return on != 0;
}
constexpr uint32_t SC_ROW_FLOATS = IX_HD + 4, SC_WARPS = 2;
constexpr uint32_t SC_TILE_BYTES = 32u * SC_ROW_FLOATS * sizeof(float);
constexpr uint32_t SC_SMEM = SC_WARPS * 2u * SC_TILE_BYTES + IX_HD * sizeof(float4);
__global__ void __launch_bounds__(SC_WARPS * 32) q4_ix_score_k(const float *q, const float *pool, float *score,
                                                               uint32_t n_blocks, uint32_t stride, uint32_t n_head,
                                                               uint32_t pos0, uint32_t ratio, const int32_t *pp,
                                                               const float *const *pools, const int32_t *pos_arr) {
    extern __shared__ __align__(16) uint8_t sc_smem[];
    float4 *qs = reinterpret_cast<float4 *>(sc_smem);   /* [dim] = the 4 heads' values (0 for heads that do not exist) */
    const uint32_t t = blockIdx.y, lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    ix_pdl_sync();
    /* batched form: row t is session t, with its own pool and its own position */
    const uint32_t pos = pos_arr ? (uint32_t)pos_arr[t] : (pp ? (uint32_t)*pp : pos0) + t;
    if (pos_arr) pool = pools[t];
    const uint32_t n_vis = ratio ? (pos + 1u) / ratio : 0u;
    if (pp || pos_arr) n_blocks = min(n_vis, stride);      /* device position: the bound is derived here */
    const uint32_t buf0 = (uint32_t)__cvta_generic_to_shared(sc_smem + IX_HD * sizeof(float4)) + warp * 2u * SC_TILE_BYTES;
    const uint32_t lim = min(n_blocks, n_vis);                       /* rows to score */
    const uint32_t n_tiles = (lim + 31u) / 32u;
    const uint32_t step = gridDim.x * SC_WARPS, first = blockIdx.x * SC_WARPS + warp;
    auto fetch = [&](uint32_t tile, uint32_t which) {
        if (tile < n_tiles) {
            const uint32_t r0 = tile * 32u, rows = min(32u, lim - r0);
            const uint32_t dst = buf0 + which * SC_TILE_BYTES + lane * 16u;
            const float *src = pool + (size_t)r0 * IX_HD + lane * 4u;
            for (uint32_t r = 0; r < rows; r++)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + r * SC_ROW_FLOATS * 4u),
                             "l"(src + (size_t)r * IX_HD) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");   /* one group per call keeps the wait count uniform */
    };
    fetch(first, 0);
    /* the query is staged while the first tile is in flight */
    for (uint32_t d = threadIdx.x; d < IX_HD; d += SC_WARPS * 32u) {
        const float *qt = q + (size_t)t * n_head * IX_HD + d;
        qs[d] = make_float4(qt[0], n_head > 1 ? qt[IX_HD] : 0.f, n_head > 2 ? qt[2 * IX_HD] : 0.f,
                            n_head > 3 ? qt[3 * IX_HD] : 0.f);
    }
    __syncthreads();
    uint32_t which = 0;
    for (uint32_t tile = first; tile < n_tiles; tile += step, which ^= 1u) {
        fetch(tile + step, which ^ 1u);
        asm volatile("cp.async.wait_group 1;" ::: "memory");   /* this tile has landed, the next may be in flight */
        __syncwarp();
        const uint32_t b = tile * 32u + lane;
        if (b < lim) {
            const uint32_t row = buf0 + which * SC_TILE_BYTES + lane * SC_ROW_FLOATS * 4u;
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
            /* the row is read two steps ahead of the multiply-adds that use it */
            float4 kq[3];
            asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(kq[0].x), "=f"(kq[0].y), "=f"(kq[0].z), "=f"(kq[0].w) : "r"(row));
            asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(kq[1].x), "=f"(kq[1].y), "=f"(kq[1].z), "=f"(kq[1].w) : "r"(row + 16u));
#pragma unroll
            for (uint32_t i = 0; i < IX_HD / 4; i++) {
                if (i + 2 < IX_HD / 4)
                    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                                 : "=f"(kq[(i + 2) % 3].x), "=f"(kq[(i + 2) % 3].y), "=f"(kq[(i + 2) % 3].z), "=f"(kq[(i + 2) % 3].w)
                                 : "r"(row + 16u * (i + 2)));
                const float4 k = kq[i % 3];
                const float4 q0 = qs[4 * i], q1 = qs[4 * i + 1], q2 = qs[4 * i + 2], q3 = qs[4 * i + 3];
                d0 = __fmaf_rn(q0.x, k.x, d0); d1 = __fmaf_rn(q0.y, k.x, d1); d2 = __fmaf_rn(q0.z, k.x, d2); d3 = __fmaf_rn(q0.w, k.x, d3);
                d0 = __fmaf_rn(q1.x, k.y, d0); d1 = __fmaf_rn(q1.y, k.y, d1); d2 = __fmaf_rn(q1.z, k.y, d2); d3 = __fmaf_rn(q1.w, k.y, d3);
                d0 = __fmaf_rn(q2.x, k.z, d0); d1 = __fmaf_rn(q2.y, k.z, d1); d2 = __fmaf_rn(q2.z, k.z, d2); d3 = __fmaf_rn(q2.w, k.z, d3);
                d0 = __fmaf_rn(q3.x, k.w, d0); d1 = __fmaf_rn(q3.y, k.w, d1); d2 = __fmaf_rn(q3.z, k.w, d2); d3 = __fmaf_rn(q3.w, k.w, d3);
            }
            float sc = __fadd_rn(0.f, fmaxf(d0, 0.f));          /* s = 0; s += relu(dot_h) in head order */
            if (n_head > 1) sc = __fadd_rn(sc, fmaxf(d1, 0.f));
            if (n_head > 2) sc = __fadd_rn(sc, fmaxf(d2, 0.f));
            if (n_head > 3) sc = __fadd_rn(sc, fmaxf(d3, 0.f));
            score[(size_t)t * stride + b] = sc;
        }
        __syncwarp();   /* every lane is done with this buffer before the fetch after next refills it */
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    /* blocks the token cannot see (host-position form only): -1e30 */
    for (uint32_t b = n_vis + blockIdx.x * (SC_WARPS * 32u) + threadIdx.x; b < n_blocks; b += gridDim.x * SC_WARPS * 32u)
        score[(size_t)t * stride + b] = -1.0e30f;
}
bool score_launch(const float *q, const float *pool, float *score, uint32_t n_tok, uint32_t n_blocks, uint32_t stride,
                  uint32_t n_head, uint32_t pos0, uint32_t ratio, const int32_t *pp,
                  const float *const *pools = nullptr, const int32_t *pos_arr = nullptr) {
    static bool done = false;
    if (!done) {
        if (!q4i_check(cudaFuncSetAttribute(q4_ix_score_k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SC_SMEM),
                       "qsa_score smem attribute"))
            return false;
        done = true;
    }
    /* persistent grid: 3 blocks of 2 warps per SM share 227 KB; fewer when the row is short */
    const uint32_t rows = pp || pos_arr ? stride : n_blocks;
    uint32_t gx = (uint32_t)g_q4.sm_count * 3u;
    const uint32_t need = (rows + SC_WARPS * 32u - 1u) / (SC_WARPS * 32u);
    if (n_tok > 1) gx = (gx + n_tok - 1u) / n_tok;
    if (gx > need) gx = need;
    if (gx < 1) gx = 1;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(gx, n_tok);
    cfg.blockDim = dim3(SC_WARPS * 32);
    cfg.dynamicSmemBytes = SC_SMEM;
    cfg.stream = g_q4.stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = ix_pdl() ? 1 : 0;
    return q4i_check(cudaLaunchKernelEx(&cfg, q4_ix_score_k, q, pool, score, n_blocks, stride, n_head, pos0, ratio, pp, pools, pos_arr),
                     "qsa_score launch");
}

/* ---- selection: one block per token */
__device__ __forceinline__ uint32_t ix_key(float f) {   /* order-preserving uint of a float (:7464-7467) */
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
/* exclusive prefix sum of one value per thread over the block; returns the block total */
__device__ uint32_t block_excl_scan(uint32_t v, uint32_t &excl, uint32_t *warp_tot /* [33] shared */) {
    const uint32_t lane = threadIdx.x & 31u, w = threadIdx.x >> 5;
    uint32_t x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= (uint32_t)o) x += y;
    }
    __syncthreads();   /* warp_tot may still be read from the previous scan */
    if (lane == 31) warp_tot[w] = x;
    __syncthreads();
    if (w == 0) {
        uint32_t t = lane < IX_TK_THREADS / 32 ? warp_tot[lane] : 0u, s = t;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t y = __shfl_up_sync(0xffffffffu, s, o);
            if (lane >= (uint32_t)o) s += y;
        }
        warp_tot[lane] = s - t;
        if (lane == 31) warp_tot[32] = s;
    }
    __syncthreads();
    excl = warp_tot[w] + x - v;
    return warp_tot[32];
}

/* A warp walks its contiguous share of the row in batches of IX_BATCH x 32 keys: the IX_BATCH loads of
 * a batch are independent (one memory round trip per batch instead of one per key), lane l of load k
 * holds index base + 32 k + l, so (batch, k, lane) is ascending index order inside the warp. */
constexpr uint32_t IX_BATCH = 16;
template <typename F>
__device__ __forceinline__ void ix_walk(const float *row, uint32_t n_vis, uint32_t per_warp, F f) {
    const uint32_t lane = threadIdx.x & 31u, w0 = (threadIdx.x >> 5) * per_warp;
    const uint32_t w1 = min(w0 + per_warp, n_vis);
    for (uint32_t base = w0; base < w1; base += 32u * IX_BATCH) {
        uint32_t key[IX_BATCH];
#pragma unroll
        for (uint32_t k = 0; k < IX_BATCH; k++) {
            const uint32_t b = base + 32u * k + lane;
            key[k] = b < w1 ? ix_key(__ldcg(row + b)) : 0u;
        }
#pragma unroll
        for (uint32_t k = 0; k < IX_BATCH; k++) {
            const uint32_t b = base + 32u * k + lane;
            f(b, key[k], b < w1);
        }
    }
}

__global__ void __launch_bounds__(IX_TK_THREADS) q4_ix_topk1_k(const float *score, int32_t *sel, uint32_t stride,
                                                              uint32_t k_blk, uint32_t ratio, uint32_t pos0,
                                                              uint32_t width, const int32_t *pp, const int32_t *pos_arr) {
    __shared__ uint32_t hist[256], warp_tot[33], st_prefix, st_hi;
    __shared__ int32_t chosen[IX_MAX_KBLK];
    const uint32_t t = blockIdx.x, tx = threadIdx.x, lane = tx & 31u;
    const uint32_t pos = pos_arr ? (uint32_t)pos_arr[t] : (pp ? (uint32_t)*pp : pos0) + t;
    const uint32_t n_vis = ratio ? (pos + 1u) / ratio : 0u;
    const uint32_t need = n_vis < k_blk ? n_vis : k_blk;
    const float *row = score + (size_t)t * stride;
    int32_t *out = sel + (size_t)t * width;
    if (need == n_vis) {   /* every complete block fits: the dense prefix */
        for (uint32_t w = tx; w < width; w += IX_TK_THREADS) out[w] = w <= pos ? (int32_t)w : -1;
        return;
    }
    /* contiguous share of each of the 32 warps, a whole number of batches */
    const uint32_t per_warp = ((n_vis + 31u) / 32u + 32u * IX_BATCH - 1u) / (32u * IX_BATCH) * (32u * IX_BATCH);

    /* exact need-th largest key: 4 passes over the 8-bit digits, most significant first */
    if (tx == 0) { st_prefix = 0u; st_hi = 0u; }
    for (int p = 0; p < 4; p++) {
        if (tx < 256) hist[tx] = 0u;
        __syncthreads();
        const uint32_t sh = 24u - 8u * p, pre = st_prefix;
        ix_walk(row, n_vis, per_warp, [&](uint32_t, uint32_t u, bool live) {
            const bool in = live && (p == 0 || (u >> (sh + 8u)) == pre);
            const uint32_t bin = (u >> sh) & 255u;
            /* Keys often share a digit (the leading digits of non-negative scores, relu zeros, padding):
             * when every participating lane has the same bin one lane adds the count; otherwise the bins
             * are spread and each lane adds for itself. */
            const uint32_t m = __ballot_sync(0xffffffffu, in);
            if (m) {
                const uint32_t first = __shfl_sync(0xffffffffu, bin, __ffs(m) - 1);
                if (__all_sync(0xffffffffu, !in || bin == first)) {
                    if (lane == (uint32_t)(__ffs(m) - 1)) atomicAdd(&hist[first], (uint32_t)__popc(m));
                } else if (in) {
                    atomicAdd(&hist[bin], 1u);
                }
            }
        });
        __syncthreads();
        if (tx < 32) {
            /* digit = the highest bin whose count, added to those above it, reaches the target: lane l owns
             * bins 255 - 8 l .. 248 - 8 l, a warp scan gives the count above each lane's bins */
            const uint32_t target = need - st_hi;
            uint32_t c[8], tot = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) { c[j] = hist[255 - 8 * (int)lane - j]; tot += c[j]; }
            uint32_t incl = tot;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t y = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= (uint32_t)o) incl += y;
            }
            uint32_t above = incl - tot;
            if (above < target && incl >= target) {   /* exactly one lane */
                uint32_t dg = 0;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (above + c[j] >= target) { dg = 255u - 8u * lane - (uint32_t)j; break; }
                    above += c[j];
                }
                st_hi += above;
                st_prefix = (pre << 8) | dg;
            }
        }
        __syncthreads();
    }
    const uint32_t thr = st_prefix, n_gt = st_hi;   /* keys above the threshold: n_gt < need <= n_gt + ties */

    /* ordered compaction: blocks above the threshold in ascending index order, then threshold ties in
     * ascending index order until `need` is full.  Per-warp counts, a scan over the warps, then ranks
     * by ballots. */
    uint32_t ng = 0, ne = 0;
    ix_walk(row, n_vis, per_warp, [&](uint32_t, uint32_t u, bool live) {
        ng += __popc(__ballot_sync(0xffffffffu, live && u > thr));
        ne += __popc(__ballot_sync(0xffffffffu, live && u == thr));
    });
    uint32_t og, oe;
    (void)block_excl_scan(lane == 0 ? ng : 0u, og, warp_tot);
    (void)block_excl_scan(lane == 0 ? ne : 0u, oe, warp_tot);
    og = __shfl_sync(0xffffffffu, og, 0);
    oe = __shfl_sync(0xffffffffu, oe, 0);
    const uint32_t lt = (1u << lane) - 1u;
    ix_walk(row, n_vis, per_warp, [&](uint32_t b, uint32_t u, bool live) {
        const bool gt = live && u > thr, eq = live && u == thr;
        const uint32_t mg = __ballot_sync(0xffffffffu, gt), me = __ballot_sync(0xffffffffu, eq);
        if (gt) {
            const uint32_t at = og + __popc(mg & lt);
            if (at < IX_MAX_KBLK) chosen[at] = (int32_t)b;
        } else if (eq) {
            const uint32_t at = n_gt + oe + __popc(me & lt);
            if (at < need) chosen[at] = (int32_t)b;
        }
        og += __popc(mg);
        oe += __popc(me);
    });
    __syncthreads();
    const uint32_t ncs = need * ratio;
    for (uint32_t w = tx; w < width; w += IX_TK_THREADS) {
        int32_t v;
        if (w < ncs) {
            const uint32_t i = w / ratio, j = w - i * ratio;
            v = (int32_t)((uint32_t)chosen[i] * ratio + j);
        } else {
            const uint32_t tail = n_vis * ratio + (w - ncs);
            v = tail <= pos ? (int32_t)tail : -1;
        }
        out[w] = v;
    }
}

/* ---- selection by a cluster of 8 blocks (rows of up to 65 536 pooled blocks = ctx 262 144): every
 * thread keeps its 8 keys in registers (block r, warp w, step i, lane l holds index 8192 r + 256 w +
 * 32 i + l, so (r, w, i, l) is ascending index order), the per-pass histograms are summed into block
 * 0 through distributed shared memory, every block picks the digit from that sum (copied back with one
 * load per thread: one warp reading its bins from block 0 itself was 3 us slower), and the ordered emit ranks by ballots, one scan over the warps and the other
 * blocks' counts, and writes the positions straight into the list.  One cluster barrier and three block
 * barriers per pass, one cluster barrier for the counts, none after the last remote access; 8 SMs
 * instead of one. */
constexpr uint32_t TKC_BLOCKS = 8, TKC_KPT = 8, TKC_MAX_ROW = TKC_BLOCKS * IX_TK_THREADS * TKC_KPT;
constexpr uint32_t TKC_CAND = 256;   /* most keys sharing a 16-bit prefix that are ranked directly */
__device__ __forceinline__ uint32_t tkc_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void tkc_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t tkc_remote(const void *p, uint32_t rank) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(p), r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ uint32_t tkc_ld(uint32_t ra) {
    uint32_t v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(ra) : "memory");
    return v;
}
__device__ __forceinline__ void tkc_st(uint32_t ra, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(ra), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t tkc_atom_add(uint32_t ra, uint32_t v) {
    uint32_t old;
    asm volatile("atom.relaxed.cluster.shared::cluster.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(ra), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void tkc_red_add(uint32_t ra, uint32_t v) {
    asm volatile("red.relaxed.cluster.shared::cluster.add.u32 [%0], %1;" ::"r"(ra), "r"(v) : "memory");
}

__global__ void __launch_bounds__(IX_TK_THREADS) q4_ix_topkc_k(const float *score, int32_t *sel, uint32_t stride,
                                                               uint32_t k_blk, uint32_t ratio, uint32_t pos0,
                                                               uint32_t width, const int32_t *pp, const int32_t *pos_arr) {
    __shared__ uint32_t lhist[4][256];            /* this block's histogram of every pass, zeroed once */
    __shared__ uint32_t ghist[4][256];            /* block 0's copy is the cluster-wide sum, one per pass */
    __shared__ uint32_t cta_cnt[TKC_BLOCKS];      /* (ties << 16 | above) of every block, pushed by its owner */
    __shared__ uint32_t warp_tot[33], st_prefix, st_hi, st_cnt;
    __shared__ uint32_t cand[TKC_CAND], cand_n;   /* block 0's copy collects the keys that share the 16-bit prefix */
    const uint32_t t = blockIdx.y, tx = threadIdx.x, lane = tx & 31u, warp = tx >> 5, rank = tkc_rank();
    /* The block's own shared memory is prepared, and the cluster has met once, before the launch waits for
     * the previous kernel: with programmatic dependent launch this part runs under that kernel's tail. */
    (&lhist[0][0])[tx] = 0u;                      /* 4 x 256 words, one per thread */
    if (rank == 0) (&ghist[0][0])[tx] = 0u;
    static_assert(IX_TK_THREADS == 4 * 256, "one histogram word per thread");
    if (tx == 0) { st_prefix = 0u; st_hi = 0u; cand_n = 0u; }
    tkc_sync();   /* block 0's sums are zero before anyone adds to them */
    ix_pdl_sync();
    const uint32_t pos = pos_arr ? (uint32_t)pos_arr[t] : (pp ? (uint32_t)*pp : pos0) + t;
    const uint32_t n_vis = ratio ? (pos + 1u) / ratio : 0u;
    const uint32_t need = n_vis < k_blk ? n_vis : k_blk;
    const float *row = score + (size_t)t * stride;
    int32_t *out = sel + (size_t)t * width;
    const uint32_t w_per = (width + TKC_BLOCKS - 1u) / TKC_BLOCKS;
    const uint32_t w0 = min(rank * w_per, width), w1 = min(w0 + w_per, width);   /* this block's slice of the list */
    if (need == n_vis) {   /* every complete block fits: the dense prefix (same decision in all blocks) */
        for (uint32_t w = w0 + tx; w < w1; w += IX_TK_THREADS) out[w] = w <= pos ? (int32_t)w : -1;
        return;
    }
    const uint32_t base = rank * (IX_TK_THREADS * TKC_KPT) + warp * (32u * TKC_KPT) + lane;
    uint32_t key[TKC_KPT];
#pragma unroll
    for (uint32_t i = 0; i < TKC_KPT; i++) {
        const uint32_t b = base + 32u * i;
        key[i] = b < n_vis ? ix_key(__ldcg(row + b)) : 0u;
    }
    /* the tail of the list (positions behind the last complete block) does not depend on the selection */
    const uint32_t ncs = need * ratio;
    for (uint32_t w = max(w0, ncs) + tx; w < w1; w += IX_TK_THREADS) {
        const uint32_t tail = n_vis * ratio + (w - ncs);
        out[w] = tail <= pos ? (int32_t)tail : -1;
    }

    bool ranked = false;   /* the threshold came from ranking the last candidates, st_cnt holds the count above it */
    for (int p = 0; p < 4; p++) {
        const uint32_t sh = 24u - 8u * p, pre = st_prefix;
#pragma unroll
        for (uint32_t i = 0; i < TKC_KPT; i++) {
            const uint32_t u = key[i];
            const bool in = base + 32u * i < n_vis && (p == 0 || (u >> (sh + 8u)) == pre);
            const uint32_t bin = (u >> sh) & 255u;
            const uint32_t m = __ballot_sync(0xffffffffu, in);
            if (m) {   /* one add per warp where the lanes agree, else one per lane */
                const uint32_t first = __shfl_sync(0xffffffffu, bin, __ffs(m) - 1);
                if (__all_sync(0xffffffffu, !in || bin == first)) {
                    if (lane == (uint32_t)(__ffs(m) - 1)) atomicAdd(&lhist[p][first], (uint32_t)__popc(m));
                } else if (in) {
                    atomicAdd(&lhist[p][bin], 1u);
                }
            }
        }
        __syncthreads();
        if (tx < 256 && lhist[p][tx]) tkc_red_add(tkc_remote(&ghist[p][tx], 0), lhist[p][tx]);
        tkc_sync();
        if (tx < 256) lhist[p][tx] = tkc_ld(tkc_remote(&ghist[p][tx], 0));   /* the cluster-wide sum, one load per thread */
        __syncthreads();
        if (tx < 32) {
            /* digit = the highest bin whose count, added to those above it, reaches the target: lane l owns
             * bins 255 - 8 l .. 248 - 8 l of the cluster-wide sum */
            const uint32_t target = need - st_hi;
            uint32_t c[8], tot = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) { c[j] = lhist[p][255 - 8 * (int)lane - j]; tot += c[j]; }
            uint32_t incl = tot;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t y = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= (uint32_t)o) incl += y;
            }
            uint32_t above = incl - tot;
            if (above < target && incl >= target) {   /* exactly one lane */
                uint32_t dg = 0, cnt = 0;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (above + c[j] >= target) { dg = 255u - 8u * lane - (uint32_t)j; cnt = c[j]; break; }
                    above += c[j];
                }
                st_hi += above;
                st_prefix = (pre << 8) | dg;
                st_cnt = cnt;   /* keys that share the prefix chosen so far */
            }
        }
        __syncthreads();
        if (p == 1 && st_cnt <= TKC_CAND) {
            /* After 16 bits only a handful of keys still share the prefix (the same decision in every
             * block: the counts are cluster-wide).  They are collected in block 0, and every block ranks
             * them itself: the key with fewer than `target` keys above it and at least `target` at or
             * above it is the threshold.  One cluster barrier instead of the two remaining passes. */
            const uint32_t pre16 = st_prefix, target = need - st_hi;
#pragma unroll
            for (uint32_t i = 0; i < TKC_KPT; i++)
                if (base + 32u * i < n_vis && (key[i] >> 16) == pre16) {
                    const uint32_t slot = tkc_atom_add(tkc_remote(&cand_n, 0), 1u);
                    if (slot < TKC_CAND) tkc_st(tkc_remote(&cand[slot], 0), key[i]);
                }
            tkc_sync();
            const uint32_t n = st_cnt;   /* exactly the keys just collected */
            if (rank != 0 && tx < n) cand[tx] = tkc_ld(tkc_remote(&cand[tx], 0));
            __syncthreads();
            if (tx < n) {
                const uint32_t mine = cand[tx];
                uint32_t gt = 0, ge = 0;
                for (uint32_t j = 0; j < n; j++) {
                    const uint32_t o = cand[j];
                    gt += o > mine;
                    ge += o >= mine;
                }
                if (gt < target && ge >= target) {   /* every copy of the threshold key writes the same values */
                    st_prefix = mine;
                    st_cnt = st_hi + gt;
                }
            }
            __syncthreads();
            ranked = true;
            break;
        }
    }
    const uint32_t thr = st_prefix, n_gt = ranked ? st_cnt : st_hi;

    /* counts: per warp by ballots, per block by one scan over the warps (ties in the high half-word: a
     * block holds at most 8192 keys), per cluster by every block pushing its pair to all the others */
    uint32_t ng = 0, ne = 0;
#pragma unroll
    for (uint32_t i = 0; i < TKC_KPT; i++) {
        const bool live = base + 32u * i < n_vis;
        ng += __popc(__ballot_sync(0xffffffffu, live && key[i] > thr));
        ne += __popc(__ballot_sync(0xffffffffu, live && key[i] == thr));
    }
    static_assert(IX_TK_THREADS * TKC_KPT < 65536, "two counts share a word");
    uint32_t off;
    const uint32_t tot = block_excl_scan(lane == 0 ? (ne << 16 | ng) : 0u, off, warp_tot);
    off = __shfl_sync(0xffffffffu, off, 0);
    if (tx < TKC_BLOCKS) tkc_st(tkc_remote(&cta_cnt[rank], tx), tot);
    tkc_sync();   /* the last access to another block's shared memory is behind this point */
    for (uint32_t r = 0; r < rank; r++) off += cta_cnt[r];   /* neither half carries: at most 7 x 8192 + 8191 keys precede a thread */
    uint32_t og = off & 0xffffu, oe = off >> 16;
    /* ordered emit, straight into the list: above the threshold in index order, then ties until `need` is full */
    const uint32_t lt = (1u << lane) - 1u;
#pragma unroll
    for (uint32_t i = 0; i < TKC_KPT; i++) {
        const uint32_t b = base + 32u * i;
        const bool live = b < n_vis, gt = live && key[i] > thr, eq = live && key[i] == thr;
        const uint32_t mg = __ballot_sync(0xffffffffu, gt), me = __ballot_sync(0xffffffffu, eq);
        uint32_t at = need;
        if (gt) at = og + __popc(mg & lt);
        else if (eq) at = n_gt + oe + __popc(me & lt);
        if (at < need)
            for (uint32_t j = 0; j < ratio && at * ratio + j < width; j++) out[at * ratio + j] = (int32_t)(b * ratio + j);
        og += __popc(mg);
        oe += __popc(me);
    }
}

/* rows that fit the cluster kernel go there, longer ones to the single block */
bool launch_topk(const float *score, int32_t *sel, uint32_t n_tok, uint32_t stride, uint32_t k_blk, uint32_t ratio,
                 uint32_t pos0, uint32_t width, const int32_t *pp, const int32_t *pos_arr = nullptr) {
    if (stride <= TKC_MAX_ROW) {
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3(TKC_BLOCKS, n_tok);
        cfg.blockDim = dim3(IX_TK_THREADS);
        cfg.stream = g_q4.stream;
        cudaLaunchAttribute at[2];
        at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[1].val.programmaticStreamSerializationAllowed = 1;
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = TKC_BLOCKS;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        cfg.attrs = at;
        cfg.numAttrs = ix_pdl() ? 2 : 1;
        return q4i_check(cudaLaunchKernelEx(&cfg, q4_ix_topkc_k, score, sel, stride, k_blk, ratio, pos0, width, pp, pos_arr),
                         "qsa_topk launch");
    }
    q4_ix_topk1_k<<<n_tok, IX_TK_THREADS, 0, g_q4.stream>>>(score, sel, stride, k_blk, ratio, pos0, width, pp, pos_arr);
    return q4i_check(cudaGetLastError(), "qsa_topk launch");
}

}  // namespace

/* ======================================================================= reference ABI ===== */
extern "C" bool q4_hip_qsa_pool(const void *raw_f16, float *pool, const float *wn, uint32_t hd, uint32_t ratio,
                                uint32_t b0, uint32_t b1, uint32_t n_rot, float rope_base, float eps) {
    if (!g_q4.ok || !raw_f16 || !pool || b1 <= b0 || hd != IX_HD || ratio == 0) return false;
    q4_ix_pool_k<<<(b1 - b0 + 3u) / 4u, 128, 0, g_q4.stream>>>((const __half *)raw_f16, pool, wn, ratio, b0, b1, n_rot,
                                                             rope_base, eps, nullptr);
    return q4i_check(cudaGetLastError(), "qsa_pool launch");
}
extern "C" bool q4_hip_qsa_pool_d(const void *raw, float *pool, const float *wn, uint32_t hd, uint32_t ratio,
                                  uint32_t n_rot, float rope_base, float eps) {
    if (!g_q4.ok || !g_q4.pos_d || !raw || !pool || hd != IX_HD || ratio == 0) return false;
    q4_ix_pool_k<<<1, 128, 0, g_q4.stream>>>((const __half *)raw, pool, wn, ratio, 0, 0, n_rot, rope_base, eps, g_q4.pos_d);
    return q4i_check(cudaGetLastError(), "qsa_pool_d launch");
}
extern "C" bool q4_hip_qsa_score(const float *q, const float *pool, float *score, uint32_t n_tok, uint32_t n_blocks,
                                 uint32_t stride, uint32_t n_head, uint32_t hd, uint32_t pos0, uint32_t ratio) {
    if (!g_q4.ok || !q || !pool || !score || n_tok == 0 || hd != IX_HD || n_head == 0 || n_head > 4) return false;
    if (n_blocks == 0) return true;
    return score_launch(q, pool, score, n_tok, n_blocks, stride, n_head, pos0, ratio, nullptr);
}
/* Device position (graph-captured decode): the grid covers `stride` blocks, the bound comes from the
 * position word inside the kernel. */
extern "C" bool q4_hip_qsa_score_d(const float *q, const float *pool, float *score, uint32_t stride, uint32_t n_head,
                                   uint32_t hd, uint32_t ratio) {
    if (!g_q4.ok || !g_q4.pos_d || !q || !pool || !score || hd != IX_HD || n_head == 0 || n_head > 4 || stride == 0)
        return false;
    return score_launch(q, pool, score, 1, 0, stride, n_head, 0, ratio, g_q4.pos_d);
}
extern "C" bool q4_hip_qsa_topk(const float *score, int32_t *sel, uint32_t n_tok, uint32_t n_blocks, uint32_t stride,
                                uint32_t k_blk, uint32_t ratio, uint32_t pos0, uint32_t width) {
    (void)n_blocks;
    if (!g_q4.ok || !score || !sel || n_tok == 0 || k_blk == 0 || k_blk > IX_MAX_KBLK || width == 0) return false;
    return launch_topk(score, sel, n_tok, stride, k_blk, ratio, pos0, width, nullptr);
}
extern "C" bool q4_hip_qsa_topk_d(const float *score, int32_t *sel, uint32_t stride, uint32_t k_blk, uint32_t ratio,
                                  uint32_t width) {
    if (!g_q4.ok || !g_q4.pos_d || !score || !sel || k_blk == 0 || k_blk > IX_MAX_KBLK || width == 0) return false;
    return launch_topk(score, sel, 1, stride, k_blk, ratio, 0, width, g_q4.pos_d);
}

/* Batched form for concurrent sessions (additive): row t of q / score / sel belongs to session t, which
 * has its own pool (pools[t], device array of device pointers) and its own position (pos[t], device
 * array); scoring and selection of all sessions in two launches.  Every session must have at most
 * `stride` visible blocks.  Same arithmetic and the same lists as one q4_hip_qsa_score_d +
 * q4_hip_qsa_topk_d pair per session. */
extern "C" bool q4_gpu_qsa_select_batch(const float *const *pools, const int32_t *pos, const float *q, float *score,
                                        int32_t *sel, uint32_t n_sess, uint32_t stride, uint32_t n_head, uint32_t hd,
                                        uint32_t k_blk, uint32_t ratio, uint32_t width) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "qsa_select_batch: library not initialised");
    Q4_REQUIRE(pools && pos && q && score && sel && n_sess && stride && ratio && width, "qsa_select_batch: bad argument");
    Q4_REQUIRE(hd == IX_HD && n_head >= 1 && n_head <= 4 && k_blk >= 1 && k_blk <= IX_MAX_KBLK,
               "qsa_select_batch: unsupported shape");
    return score_launch(q, nullptr, score, n_sess, 0, stride, n_head, 0, ratio, nullptr, pools, pos) &&
           launch_topk(score, sel, n_sess, stride, k_blk, ratio, 0, width, nullptr, pos);
}
