/*
 * Runtime glue behind the reference's device ABI: one device, one compute stream, allocation,
 * copies, the decode position word, stream capture, scratch.  Restates the conventions of
 * src/q4_rocm.cu:20-120,202-322,5656-5670,6218-6227,8156-8246,8417-8432 on the CUDA runtime.
 */
#include <stdlib.h>
#include <string.h>

#include "q4_internal.h"

Q4State g_q4 = {};

bool q4i_fail(uint32_t bit, const char *what) {
    g_q4.err_h |= bit;
    fprintf(stderr, "q4 gpu: %s\n", what);
    return false;
}
bool q4i_check(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return true;
    g_q4.err_h |= Q4E_CUDA;
    fprintf(stderr, "q4 gpu: %s: %s\n", what, cudaGetErrorString(e));
    return false;
}

/* Scratch for the split-KV records and arrival counters.  Grows only outside capture (an
 * allocation would invalidate the capture, src/q4_rocm.cu:55-57); counters start at zero and every
 * kernel leaves them at zero. */
bool q4i_scratch(size_t part_floats, size_t n_counters) {
    if (part_floats > g_q4.part_floats) {
        if (g_q4.capturing) return q4i_fail(Q4E_SCRATCH, "attention scratch too small inside a capture");
        if (!q4i_check(cudaStreamSynchronize(g_q4.stream), "scratch sync")) return false;
        if (g_q4.part) cudaFree(g_q4.part);
        g_q4.part = nullptr;
        g_q4.part_floats = 0;
        size_t want = part_floats + part_floats / 4;
        if (!q4i_check(cudaMalloc(&g_q4.part, want * sizeof(float)), "scratch alloc")) return false;
        g_q4.part_floats = want;
    }
    if (n_counters > g_q4.n_counters) {
        if (g_q4.capturing) return q4i_fail(Q4E_SCRATCH, "attention counters too small inside a capture");
        if (!q4i_check(cudaStreamSynchronize(g_q4.stream), "scratch sync")) return false;
        if (g_q4.counters) cudaFree(g_q4.counters);
        g_q4.counters = nullptr;
        g_q4.n_counters = 0;
        size_t want = n_counters * 2;
        if (!q4i_check(cudaMalloc(&g_q4.counters, want * sizeof(uint32_t)), "counter alloc")) return false;
        if (!q4i_check(cudaMemset(g_q4.counters, 0, want * sizeof(uint32_t)), "counter clear")) return false;
        g_q4.n_counters = want;
    }
    return true;
}

extern "C" bool q4_hip_init(void) {
    if (g_q4.ok) return true;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        return false;
    }
    int dev = 0;
    const char *e = getenv("Q4_GPU_DEVICE");
    if (!e) e = getenv("LOCAL_RANK");
    if (e) dev = atoi(e);
    if (dev < 0 || dev >= n) dev = 0;
    if (cudaSetDevice(dev) != cudaSuccess) return false;
    g_q4.device = dev;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return false;
    if (prop.major < 10) {
        fprintf(stderr, "q4 gpu: device %d is sm_%d%d; this library is built for sm_100a only\n", dev,
                prop.major, prop.minor);
        return false;
    }
    g_q4.sm_count = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&g_q4.own_stream, cudaStreamNonBlocking) != cudaSuccess) return false;
    g_q4.stream = g_q4.own_stream;
    if (cudaStreamCreateWithFlags(&g_q4.copy_stream, cudaStreamNonBlocking) != cudaSuccess)
        g_q4.copy_stream = nullptr;
    if (cudaStreamCreateWithFlags(&g_q4.down_stream, cudaStreamNonBlocking) != cudaSuccess)
        g_q4.down_stream = nullptr;
    if (cudaMalloc(&g_q4.pos_d, sizeof(int32_t)) != cudaSuccess) return false;
    if (cudaMemset(g_q4.pos_d, 0, sizeof(int32_t)) != cudaSuccess) return false;
    if (cudaMallocHost(&g_q4.pos_h, sizeof(int32_t) * 64) != cudaSuccess) return false;
    if (cudaMalloc(&g_q4.err_d, sizeof(uint32_t)) != cudaSuccess) return false;
    if (cudaMemset(g_q4.err_d, 0, sizeof(uint32_t)) != cudaSuccess) return false;
    g_q4.ok = true;
    return true;
}

extern "C" void q4_hip_shutdown(void) {
    if (!g_q4.ok) return;
    cudaDeviceSynchronize();
    if (g_q4.part) cudaFree(g_q4.part);
    if (g_q4.counters) cudaFree(g_q4.counters);
    if (g_q4.pos_d) cudaFree(g_q4.pos_d);
    if (g_q4.pos_h) cudaFreeHost(g_q4.pos_h);
    q4i_prefill_release();
    q4i_sess_release();
    if (g_q4.err_d) cudaFree(g_q4.err_d);
    if (g_q4.own_stream) cudaStreamDestroy(g_q4.own_stream);
    if (g_q4.copy_stream) cudaStreamDestroy(g_q4.copy_stream);
    if (g_q4.down_stream) cudaStreamDestroy(g_q4.down_stream);
    memset(&g_q4, 0, sizeof(g_q4));
}

extern "C" bool q4_hip_ok(void) { return g_q4.ok; }
extern "C" int q4_gpu_device(void) { return g_q4.ok ? g_q4.device : -1; }
extern "C" void *q4_gpu_stream(void) { return g_q4.ok ? (void *)g_q4.stream : nullptr; }
extern "C" bool q4_gpu_set_stream(void *s) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "set_stream: library not initialised");
    if (g_q4.capturing) return q4i_fail(Q4E_ARG, "set_stream: a capture is open");
    g_q4.stream = s ? (cudaStream_t)s : g_q4.own_stream;
    return true;
}
extern "C" const int32_t *q4_gpu_pos_word(void) { return g_q4.pos_d; }

extern "C" uint32_t q4_gpu_last_error(void) {
    uint32_t e = g_q4.err_h;
    g_q4.err_h = 0;
    if (g_q4.ok && !g_q4.capturing) {
        uint32_t d = 0;
        if (cudaMemcpyAsync(&d, g_q4.err_d, sizeof(d), cudaMemcpyDeviceToHost, g_q4.stream) == cudaSuccess &&
            cudaStreamSynchronize(g_q4.stream) == cudaSuccess) {
            if (d) (void)cudaMemsetAsync(g_q4.err_d, 0, sizeof(d), g_q4.stream);
            e |= d;
        } else {
            e |= Q4E_CUDA;
        }
    }
    return e;
}

extern "C" void *q4_hip_malloc(size_t n) {
    if (!g_q4.ok || n == 0) return nullptr;
    void *p = nullptr;
    if (cudaMalloc(&p, n) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return p;
}
extern "C" void q4_hip_free(void *p) {
    if (p) (void)cudaFree(p);
}

/* Copy ordered after the compute stream's work; waited for unless a capture is open, in which case
 * it becomes a memcpy node (src/q4_rocm.cu:202-214). */
static bool sync_copy(void *dst, const void *src, size_t n, cudaMemcpyKind kind) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "copy: library not initialised");
    if (!q4i_check(cudaMemcpyAsync(dst, src, n, kind, g_q4.stream), "copy")) return false;
    if (g_q4.capturing) return true;
    return q4i_check(cudaStreamSynchronize(g_q4.stream), "copy sync");
}
extern "C" bool q4_hip_h2d(void *d, const void *h, size_t n) {
    if (!d || !h || n == 0) return false;
    return sync_copy(d, h, n, cudaMemcpyHostToDevice);
}
extern "C" bool q4_hip_d2h(void *h, const void *d, size_t n) {
    if (!d || !h || n == 0) return false;
    return sync_copy(h, d, n, cudaMemcpyDeviceToHost);
}
extern "C" bool q4_hip_d2h_async(void *h, const void *d, uint64_t n) {
    if (!g_q4.ok || !h || !d || !n) return false;
    return q4i_check(cudaMemcpyAsync(h, d, (size_t)n, cudaMemcpyDeviceToHost, g_q4.stream), "d2h_async");
}
extern "C" bool q4_hip_h2d_async(void *d, const void *h, uint64_t n) {
    if (!g_q4.ok || !d || !h || !n) return false;
    return q4i_check(cudaMemcpyAsync(d, h, (size_t)n, cudaMemcpyHostToDevice, g_q4.stream), "h2d_async");
}
/* Copies on the separate copy stream, so uploads for the next step overlap the current step's
 * kernels (src/q4.h:832,887; src/q4_rocm.cu:247-250,3270-3275).  The caller orders them against the
 * compute stream with q4_hip_copy_wait (blocking) or with events on q4_gpu_copy_stream(). */
extern "C" bool q4_hip_copy_h2d(void *dst, const void *src, size_t n) {
    if (!g_q4.ok || !dst || !src || !n) return false;
    cudaStream_t st = g_q4.copy_stream ? g_q4.copy_stream : g_q4.stream;
    return q4i_check(cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, st), "copy_h2d");
}
extern "C" void q4_hip_copy_wait(void) {
    if (!g_q4.ok) return;
    if (g_q4.copy_stream) (void)cudaStreamSynchronize(g_q4.copy_stream);
    else (void)cudaDeviceSynchronize();
}
extern "C" void *q4_gpu_copy_stream(void) { return g_q4.ok ? (void *)g_q4.copy_stream : nullptr; }
/* Results back to the host on a third stream, so that a download uses the device-to-host copy engine
 * while the next step computes and the step after uploads.  Ordered by the caller with events on
 * q4_gpu_download_stream(). */
extern "C" bool q4_gpu_copy_d2h(void *dst, const void *src, size_t n) {
    if (!g_q4.ok || !dst || !src || !n) return false;
    cudaStream_t st = g_q4.down_stream ? g_q4.down_stream : g_q4.stream;
    return q4i_check(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToHost, st), "copy_d2h");
}
extern "C" void *q4_gpu_download_stream(void) { return g_q4.ok ? (void *)g_q4.down_stream : nullptr; }
extern "C" bool q4_hip_stream_sync(void) {
    if (!g_q4.ok) return false;
    return q4i_check(cudaStreamSynchronize(g_q4.stream), "stream_sync");
}
extern "C" void q4_hip_sync(void) {
    if (g_q4.ok) (void)cudaDeviceSynchronize();
}
extern "C" void q4_hip_clear(void) { (void)cudaGetLastError(); }

/* Device-to-device copy of n floats, stream-ordered.  The reference also waits for it outside
 * capture (sync_copy); a stream-ordered consumer never needs that wait, so it is not reproduced. */
extern "C" bool q4_hip_copy(float *d, const float *s, uint64_t n) {
    if (!g_q4.ok || !d || !s || n == 0) return false;
    return q4i_check(cudaMemcpyAsync(d, s, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, g_q4.stream),
                     "copy d2d");
}
__global__ static void q4_fill_k(float *d, float v, uint64_t n) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) d[i] = v;
}
extern "C" bool q4_hip_fill(float *d, float v, uint64_t n) {
    if (!g_q4.ok || !d || n == 0) return false;
    if (v == 0.f)
        return q4i_check(cudaMemsetAsync(d, 0, (size_t)n * sizeof(float), g_q4.stream), "fill");
    uint64_t blocks = (n + 255) / 256;
    uint64_t cap = (uint64_t)g_q4.sm_count * 16;
    q4_fill_k<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, g_q4.stream>>>(d, v, n);
    return q4i_check(cudaGetLastError(), "fill launch");
}

/* Decode position for graph-captured kernels: a stream-ordered one-word store.  The value travels
 * as a launch argument, so a host that runs many steps ahead of the device has no staging word that
 * a later push could overwrite before the device has read it. */
__global__ void q4_set_word_k(int32_t *dst, int32_t v) { *dst = v; }
extern "C" void q4_hip_pos_push(int32_t pos) {
    if (!g_q4.ok) return;
    q4_set_word_k<<<1, 1, 0, g_q4.stream>>>(g_q4.pos_d, pos);
    (void)q4i_check(cudaGetLastError(), "pos_push launch");
}
extern "C" int q4_hip_capturing(void) { return g_q4.capturing; }
extern "C" int q4_hip_pos_dev_ok(void) { return g_q4.ok && g_q4.pos_d && g_q4.pos_h; }

extern "C" int q4_hip_graph_begin(void) {
    if (!g_q4.ok || g_q4.capturing) return 0;
    if (g_q4.stream == cudaStreamLegacy || g_q4.stream == nullptr) {
        /* the legacy default stream cannot be captured: a host that adopted it (q4_gpu_set_stream) has to
         * hand over a real stream, or NULL to go back to the library's own, before it opens a capture */
        q4i_fail(Q4E_ARG, "graph_begin: the adopted stream is the legacy default stream, which cannot be captured; "
                          "call q4_gpu_set_stream(NULL) or adopt a created stream first");
        return 0;
    }
    if (cudaStreamBeginCapture(g_q4.stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    g_q4.capturing = 1;
    return 1;
}
extern "C" void *q4_hip_graph_end(void) {
    if (!g_q4.ok || !g_q4.capturing) return nullptr;
    g_q4.capturing = 0;
    cudaGraph_t g = nullptr;
    if (cudaStreamEndCapture(g_q4.stream, &g) != cudaSuccess || !g) {
        (void)cudaGetLastError();
        return nullptr;
    }
    size_t nn = 0;
    (void)cudaGraphGetNodes(g, nullptr, &nn);
    g_q4.last_graph_nodes = (uint32_t)nn;
    cudaGraphExec_t ex = nullptr;
    cudaError_t e = cudaGraphInstantiate(&ex, g, 0);
    (void)cudaGraphDestroy(g);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    (void)cudaGraphUpload(ex, g_q4.stream);
    return (void *)ex;
}
extern "C" uint32_t q4_hip_graph_nodes(void *exec) {
    (void)exec;
    return g_q4.last_graph_nodes;
}
extern "C" bool q4_hip_graph_launch(void *exec) {
    if (!g_q4.ok || !exec) return false;
    return q4i_check(cudaGraphLaunch((cudaGraphExec_t)exec, g_q4.stream), "graph launch");
}
extern "C" void q4_hip_graph_free(void *exec) {
    if (exec) (void)cudaGraphExecDestroy((cudaGraphExec_t)exec);
}

/* ---- a pipelined step loop over one set of step buffers -------------------------------------------
 * A host that decodes step after step from host buffers keeps two or three sets of device input / output
 * buffers, each with a captured graph that reads and writes them, and overlaps the upload of step i + 1 and the
 * download of step i - 1 with the kernels of step i.  A pipe holds the three events that order one set's
 * upload (copy stream), graph (compute stream) and download (download stream), so that a step costs the host
 * two calls and no event bookkeeping of its own. */
struct q4_gpu_pipe {
    cudaEvent_t in_done, run_done, out_done;
    bool has_run, has_out;
};
extern "C" q4_gpu_pipe *q4_gpu_pipe_create(void) {
    if (!g_q4.ok) { q4i_fail(Q4E_INIT, "pipe_create: library not initialised"); return nullptr; }
    q4_gpu_pipe *p = (q4_gpu_pipe *)calloc(1, sizeof(q4_gpu_pipe));
    if (!p) return nullptr;
    if (cudaEventCreateWithFlags(&p->in_done, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&p->run_done, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&p->out_done, cudaEventDisableTiming) != cudaSuccess) {
        q4i_fail(Q4E_CUDA, "pipe_create: event");
        if (p->in_done) cudaEventDestroy(p->in_done);
        if (p->run_done) cudaEventDestroy(p->run_done);
        free(p);
        return nullptr;
    }
    return p;
}
extern "C" void q4_gpu_pipe_destroy(q4_gpu_pipe *p) {
    if (!p) return;
    cudaEventDestroy(p->in_done);
    cudaEventDestroy(p->run_done);
    cudaEventDestroy(p->out_done);
    free(p);
}
/* The step's inputs, pinned host memory -> the set's device buffer, on the copy stream, once the set's previous
 * graph launch (which read that buffer) has run. */
extern "C" bool q4_gpu_pipe_upload(q4_gpu_pipe *p, void *dst_d, const void *src_h, size_t n) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "pipe_upload: library not initialised");
    Q4_REQUIRE(p && dst_d && src_h && n, "pipe_upload: bad argument");
    if (p->has_run && !q4i_check(cudaStreamWaitEvent(g_q4.copy_stream, p->run_done, 0), "pipe_upload wait")) return false;
    return q4i_check(cudaMemcpyAsync(dst_d, src_h, n, cudaMemcpyHostToDevice, g_q4.copy_stream), "pipe_upload copy") &&
           q4i_check(cudaEventRecord(p->in_done, g_q4.copy_stream), "pipe_upload record");
}
/* The set's graph on the compute stream, once its upload has landed and its previous download has left the output
 * buffer; then the outputs, device -> pinned host memory, on the download stream.  Returns at once. */
extern "C" bool q4_gpu_pipe_run(q4_gpu_pipe *p, void *graph_exec, void *dst_h, const void *src_d, size_t n) {
    if (!g_q4.ok) return q4i_fail(Q4E_INIT, "pipe_run: library not initialised");
    Q4_REQUIRE(p && graph_exec, "pipe_run: bad argument");
    if (!q4i_check(cudaStreamWaitEvent(g_q4.stream, p->in_done, 0), "pipe_run wait")) return false;
    if (p->has_out && !q4i_check(cudaStreamWaitEvent(g_q4.stream, p->out_done, 0), "pipe_run wait")) return false;
    if (!q4i_check(cudaGraphLaunch((cudaGraphExec_t)graph_exec, g_q4.stream), "pipe_run launch") ||
        !q4i_check(cudaEventRecord(p->run_done, g_q4.stream), "pipe_run record"))
        return false;
    p->has_run = true;
    if (dst_h && src_d && n) {
        if (!q4i_check(cudaStreamWaitEvent(g_q4.down_stream, p->run_done, 0), "pipe_run wait") ||
            !q4i_check(cudaMemcpyAsync(dst_h, src_d, n, cudaMemcpyDeviceToHost, g_q4.down_stream), "pipe_run copy") ||
            !q4i_check(cudaEventRecord(p->out_done, g_q4.down_stream), "pipe_run record"))
            return false;
        p->has_out = true;
    }
    return true;
}
/* Blocks until the set's last download has landed in host memory. */
extern "C" bool q4_gpu_pipe_sync(q4_gpu_pipe *p) {
    if (!g_q4.ok || !p) return false;
    return q4i_check(cudaEventSynchronize(p->has_out ? p->out_done : p->run_done), "pipe_sync");
}

extern "C" bool q4_hip_qsa_topk_alloc(void) {
    if (!g_q4.ok) return false;
    /* 32 MB of records + 64 Ki counters: one session at the largest supported shape (4 kv heads x
     * 272 records x 16 heads x 258 floats) or a batch of a few hundred sessions at the usual one;
     * the same role as g_attn_part, src/q4_rocm.cu:7705-7706 */
    return q4i_scratch((size_t)8 << 20, (size_t)64 << 10);
}
