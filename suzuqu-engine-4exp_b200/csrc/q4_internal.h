/* Internal declarations shared by the libq4gpu translation units (not installed). */
#ifndef Q4_INTERNAL_H
#define Q4_INTERNAL_H

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/q4_gpu.h"

/* KV kinds of the public ABI, plus the two q8_0 layouts the kernels distinguish. */
enum { Q4K_F32 = 0, Q4K_F16 = 1, Q4K_Q8 = 2 };
enum { LAY_F32 = 0, LAY_F16 = 1, LAY_Q8P = 2 /* native store: 16-byte aligned records */, LAY_Q8R = 3 /* reference 34-byte blocks */ };

enum {
    Q4E_ARG = 1, Q4E_CUDA = 2, Q4E_RANGE = 4, Q4E_SCRATCH = 8, Q4E_INIT = 16,
    Q4E_PEER = 32,   /* a peer's record did not arrive within the time limit */
};

/* One cache as the kernels see it.  Row (layer, kv head kh, token p) of the K plane lives at
 * k + layer*layer_stride + kh*kvh_stride + p*tok_stride (same for v); for the native q8_0 store the
 * scale row is at s + layer*s_layer_stride + kh*s_kvh_stride + p*s_tok_stride and holds the K block
 * scales followed by the V block scales (fp16).  The native q8_0 layout is always the record
 * {K codes hd | V codes hd | scales}: v = k + hd, s = k + 2*hd, equal strides (kernels rely on it). */
struct Q4Cache {
    const uint8_t *k, *v, *s;
    uint64_t layer_stride, kvh_stride, s_layer_stride, s_kvh_stride;
    uint32_t tok_stride, s_tok_stride;
    uint32_t max_kv, pad;
};

struct q4_gpu_kv {
    uint32_t n_layers, n_kvh, hd, max_kv;
    int kind;
    uint8_t *k, *v, *s;          /* device planes (s only for q8_0) */
    uint64_t plane_bytes, s_bytes;
    uint32_t rec_bytes;          /* bytes per (kv head, position): q8_0 record, or fp16 / fp32 row */
    Q4Cache view;                /* host copy of the kernel view */
    Q4Cache *d_view;             /* same, in device memory (for batched launches) */
};

/* runtime state (q4_runtime.cu) */
struct Q4State {
    bool ok;
    int device, sm_count;
    cudaStream_t own_stream, stream, copy_stream, down_stream;   /* compute, uploads, downloads */
    int capturing;
    int32_t *pos_d, *pos_h;
    uint32_t *err_d;             /* device-side sticky error bits */
    uint32_t err_h;
    uint32_t last_graph_nodes;
    /* attention scratch: split-KV partial records + per-unit arrival counters */
    float *part;
    size_t part_floats;
    uint32_t *counters;
    size_t n_counters;
};
extern Q4State g_q4;

bool q4i_fail(uint32_t bit, const char *what);
bool q4i_check(cudaError_t e, const char *what);
bool q4i_scratch(size_t part_floats, size_t n_counters); /* grows outside capture, fails inside */

#define Q4_REQUIRE(cond, what)                    \
    do {                                          \
        if (!(cond)) return q4i_fail(Q4E_ARG, what); \
    } while (0)

#ifdef __CUDACC__
/* ---- the q8_0 quantiser, one copy for every kernel that writes a cache row.  8 lanes share a block
 * of 32 values (4 each): d = amax / 127 and id = 1 / d as IEEE fp32 divisions, codes =
 * clamp(rint(x * id), +-127), stored scale = fp16(d) (quantize_row_q8_0's arithmetic,
 * src/q4_quant.c / src/q4_rocm.cu f32_to_q8 kernels). */
__device__ __forceinline__ uint32_t q4d_quant4(const float4 x, float id) {
    int q0 = __float2int_rn(__fmul_rn(x.x, id)), q1 = __float2int_rn(__fmul_rn(x.y, id));
    int q2 = __float2int_rn(__fmul_rn(x.z, id)), q3 = __float2int_rn(__fmul_rn(x.w, id));
    q0 = max(-127, min(127, q0)); q1 = max(-127, min(127, q1));
    q2 = max(-127, min(127, q2)); q3 = max(-127, min(127, q3));
    return (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) |
           ((uint32_t)(q3 & 0xff) << 24);
}
/* amax over the 8 lanes that share a block (all 32 lanes of the warp must call), then d and 1/d */
__device__ __forceinline__ void q4d_block_scale(const float4 x, float &d, float &id) {
    float a = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 4));
    d = __fdiv_rn(a, 127.f);
    id = d > 0.f ? __fdiv_rn(1.f, d) : 0.f;
}
#endif

/* ---- record exchange between the ranks of a sequence-sharded decode -----------------------------
 * Every rank owns one window in its own memory that all peers can write.  It starts with this header;
 * the records follow at XCHG_REC_OFFSET: packet rec[2][units][world][slot_floats], one slot per
 * (parity of the call count, unit = kv head, writing rank).  A slot is the kernel's internal record
 * for the unit's heads, {acc[hd], m (log2 units, scale folded in), l, 2 pad} per head, each fp32
 * value stored as an 8-byte packet {value, epoch of the call that wrote it}. */
constexpr uint32_t XCHG_MAX_WORLD = 16, XCHG_MAX_UNITS = 16;
constexpr size_t XCHG_REC_OFFSET = 4096;
struct Q4XchgWin {
    uint32_t epoch[XCHG_MAX_UNITS];                       /* calls completed by the owner, per unit */
};
/* who and where, in the owner's device memory (never written by peers) */
struct Q4XchgDev {
    uint32_t rank, world, units, slot_floats;
    unsigned long long timeout_ns;
    Q4XchgWin *win[XCHG_MAX_WORLD];                       /* win[rank] is the local window */
};
enum { XCHG_FUSED = 0, XCHG_PUSH = 1, XCHG_MERGE = 2 };
struct q4_gpu_xchg {
    uint32_t n_head, n_kvh, hd;
    size_t win_bytes;
    Q4XchgWin *win;
    Q4XchgDev host, *dev;
    uint8_t attached[XCHG_MAX_WORLD];                     /* 1 = opened from an IPC handle, 2 = caller's pointer */
};
/* wait-and-merge half alone (q4_decode.cu): the records of the latest push on every rank -> out */
bool q4i_xchg_merge(const q4_gpu_xchg *x, const float *gate, float *out);

/* frees the prefill staging buffer (q4_prefill.cu) / the session-file staging (q4_sess.cu); called at shutdown */
void q4i_prefill_release();
void q4i_sess_release();

/* decode attention launcher (q4_decode.cu) */
struct Q4DecodeArgs {
    Q4Cache one;                 /* used when many == nullptr */
    const Q4Cache *many;         /* device array of cache views, one per session */
    int layout;                  /* LAY_* */
    uint32_t layer, n_units;     /* units = sessions (many) or tokens (one) */
    uint32_t n_head, n_kvh, hd;
    const void *q;
    int q_bf16;
    const float *gate;
    float *out, *part_out;
    const int32_t *idx;
    uint32_t width, idx_kvh_stride, idx_unit_stride;
    const int32_t *pos;          /* device positions: per session (many) or one word (one); may be null */
    uint32_t kv_base;            /* used when pos == nullptr: unit u attends kv_base + u + 1 rows */
    uint32_t hint_rows;          /* host's estimate of rows per unit, to size the split */
    int idx_bound_nkv;           /* list entries >= the unit's row count (newest + 1) are out of range (stores:
                                  * rows beyond it were never written); 0 = only max_kv bounds them (reference ABI) */
    float scale;
    /* optional caller-provided scratch (no-allocation entry point); null = library scratch */
    float *scratch_part;
    uint32_t *scratch_counters;
    size_t scratch_part_floats, scratch_n_counters;
    int scratch_clamp;           /* reduce the split count until the records fit the caller's scratch */
    /* sequence-sharded decode: leave the unit's record in the exchange window, push it to the peers and
     * (XCHG_FUSED) wait for theirs and write the merged output; null = single-rank decode */
    const Q4XchgDev *xchg;
    int xchg_phase;
    /* fused append (native q8_0 store only): the new K and V rows [unit][n_kvh*hd] (fp32) are quantised
     * and stored at each unit's position by the attention kernel itself before it reads the cache */
    const float *new_k, *new_v;
};
bool q4i_decode(const Q4DecodeArgs &a);

#endif
