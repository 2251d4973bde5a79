/* Exchange windows for sequence-sharded decode: one context split by position over the GPUs of a
 * node, every rank attends its own rows and the (acc, m, l) records are merged on every rank.
 *
 * The reference merges split-KV records inside one GPU (gqa_dec_comb_k, src/q4_rocm.cu:6968-7012);
 * this file is the same merge across GPUs.  Each rank allocates one small window with cudaMalloc and
 * hands its CUDA IPC handle to the other ranks through whatever channel the host has (64 bytes per
 * rank, once); after that the decode kernel itself stores its record into the peers' windows over
 * NVLink and reads theirs from its own, so a layer costs one launch and no host round trip.  The
 * device side (push, bounded wait, merge) is in q4_decode.cu. */
#include "q4_internal.h"

#include <stdlib.h>
#include <string.h>

namespace {
bool upload(q4_gpu_xchg *x) {
    /* synchronous on purpose: windows are attached during start-up, and a launch that follows must
     * see the complete table */
    return q4i_check(cudaMemcpy(x->dev, &x->host, sizeof(Q4XchgDev), cudaMemcpyHostToDevice), "xchg table upload");
}
bool all_attached(const q4_gpu_xchg *x) {
    for (uint32_t r = 0; r < x->host.world; r++)
        if (!x->host.win[r]) return false;
    return true;
}
}  // namespace

extern "C" q4_gpu_xchg *q4_gpu_xchg_create(uint32_t rank, uint32_t world, uint32_t n_head, uint32_t n_kvh, uint32_t hd) {
    if (!g_q4.ok) { q4i_fail(Q4E_INIT, "xchg_create: library not initialised"); return nullptr; }
    const bool shape_ok = world && world <= XCHG_MAX_WORLD && rank < world && n_kvh && n_kvh <= XCHG_MAX_UNITS &&
                          n_head && n_head % n_kvh == 0 && n_head / n_kvh <= 16 &&
                          (hd == 32 || hd == 64 || hd == 128 || hd == 256);
    if (!shape_ok || g_q4.capturing) { q4i_fail(Q4E_ARG, "xchg_create: bad argument"); return nullptr; }
    q4_gpu_xchg *x = (q4_gpu_xchg *)calloc(1, sizeof(q4_gpu_xchg));
    if (!x) return nullptr;
    x->n_head = n_head; x->n_kvh = n_kvh; x->hd = hd;
    const uint32_t heads = n_head / n_kvh <= 8 ? 8u : 16u;
    x->host.rank = rank; x->host.world = world; x->host.units = n_kvh;
    x->host.slot_floats = heads * (hd + 4);
    x->host.timeout_ns = 2000ull * 1000ull * 1000ull;
    x->win_bytes = XCHG_REC_OFFSET + (size_t)2 * n_kvh * world * x->host.slot_floats * 8u;   /* 8-byte packets */
    bool ok = cudaMalloc(&x->win, x->win_bytes) == cudaSuccess && cudaMalloc(&x->dev, sizeof(Q4XchgDev)) == cudaSuccess &&
              cudaMemset(x->win, 0, x->win_bytes) == cudaSuccess;
    if (ok) {
        x->host.win[rank] = x->win;
        ok = upload(x);
    }
    if (!ok) {
        (void)cudaGetLastError();
        q4i_fail(Q4E_CUDA, "xchg_create: allocation failed");
        q4_gpu_xchg_destroy(x);
        return nullptr;
    }
    return x;
}

extern "C" void q4_gpu_xchg_destroy(q4_gpu_xchg *x) {
    if (!x) return;
    if (g_q4.ok) (void)cudaStreamSynchronize(g_q4.stream);   /* no launch of ours still uses the windows */
    for (uint32_t r = 0; r < XCHG_MAX_WORLD; r++)
        if (x->attached[r] == 1 && x->host.win[r]) (void)cudaIpcCloseMemHandle(x->host.win[r]);
    if (x->win) cudaFree(x->win);
    if (x->dev) cudaFree(x->dev);
    free(x);
}

extern "C" bool q4_gpu_xchg_handle(q4_gpu_xchg *x, void *handle64) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "xchg_handle: library not initialised");
    Q4_REQUIRE(x && handle64, "xchg_handle: bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the IPC handle is documented as 64 bytes");
    cudaIpcMemHandle_t h;
    if (!q4i_check(cudaIpcGetMemHandle(&h, x->win), "xchg_handle")) return false;
    memcpy(handle64, &h, sizeof(h));
    return true;
}

extern "C" void *q4_gpu_xchg_window(q4_gpu_xchg *x) { return x ? (void *)x->win : nullptr; }

extern "C" bool q4_gpu_xchg_attach(q4_gpu_xchg *x, uint32_t peer_rank, const void *handle64) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "xchg_attach: library not initialised");
    Q4_REQUIRE(x && handle64 && peer_rank < x->host.world && peer_rank != x->host.rank && !x->host.win[peer_rank] &&
                   !g_q4.capturing,
               "xchg_attach: bad argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void *p = nullptr;
    if (!q4i_check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "xchg_attach: open peer window"))
        return false;
    x->host.win[peer_rank] = (Q4XchgWin *)p;
    x->attached[peer_rank] = 1;
    return upload(x);
}

extern "C" bool q4_gpu_xchg_attach_ptr(q4_gpu_xchg *x, uint32_t peer_rank, void *peer_window) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "xchg_attach_ptr: library not initialised");
    Q4_REQUIRE(x && peer_window && peer_rank < x->host.world && peer_rank != x->host.rank && !x->host.win[peer_rank] &&
                   !g_q4.capturing,
               "xchg_attach_ptr: bad argument");
    x->host.win[peer_rank] = (Q4XchgWin *)peer_window;
    x->attached[peer_rank] = 2;
    return upload(x);
}

extern "C" bool q4_gpu_xchg_set_timeout_ms(q4_gpu_xchg *x, uint32_t ms) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "xchg_set_timeout_ms: library not initialised");
    Q4_REQUIRE(x && ms && ms <= 10000 && !g_q4.capturing, "xchg_set_timeout_ms: 1..10000 ms");
    x->host.timeout_ns = (unsigned long long)ms * 1000000ull;
    return upload(x);
}

extern "C" bool q4_gpu_kv_decode_xchg(const q4_gpu_kv *kv, q4_gpu_xchg *x, uint32_t layer, const void *q, int q_bf16,
                                      const float *gate, float *out, uint32_t n_kv, float scale, int phase) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "kv_decode_xchg: library not initialised");
    Q4_REQUIRE(x && out && phase >= XCHG_FUSED && phase <= XCHG_MERGE, "kv_decode_xchg: bad argument");
    if (!all_attached(x)) return q4i_fail(Q4E_ARG, "kv_decode_xchg: a peer window is not attached");
    if (phase == XCHG_MERGE) return q4i_xchg_merge(x, gate, out);
    Q4_REQUIRE(kv && q && layer < kv->n_layers && n_kv && n_kv <= kv->max_kv, "kv_decode_xchg: bad argument");
    Q4_REQUIRE(kv->n_kvh == x->n_kvh && kv->hd == x->hd, "kv_decode_xchg: store and window shapes differ");
    Q4DecodeArgs a;
    memset(&a, 0, sizeof(a));
    a.one = kv->view;
    a.layout = kv->kind == Q4K_Q8 ? LAY_Q8P : kv->kind == Q4K_F16 ? LAY_F16 : LAY_F32;
    a.layer = layer;
    a.n_units = 1;
    a.n_head = x->n_head;
    a.n_kvh = kv->n_kvh;
    a.hd = kv->hd;
    a.q = q;
    a.q_bf16 = q_bf16;
    a.gate = gate;
    a.out = out;
    a.kv_base = n_kv - 1;
    a.hint_rows = n_kv;
    a.scale = scale;
    a.xchg = x->dev;
    a.xchg_phase = phase;
    return q4i_decode(a);
}
