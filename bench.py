#!/usr/bin/env python
"""Benchmark of the KV-cache + decode-attention hot path.

Headline workload (`config.workload`): multi-session batched QSA decode -- 64 concurrent sessions
with seeded context lengths uniform in [1024, 131072], q8_0 KV, 12 attention layers, 16 query / 2
kv heads, head_dim 128, 2051 selected positions per session, layer and kv head (4 sink + 1024
recent + 1023 random).  One step = one decoded token for every session: for each layer the fused
K/V append (quantise + scatter) and the sparse decode attention, as one CUDA graph.  Sessions are
sharded round-robin over the ranks with no collective (strong scaling: 64 sessions in total).

`value` = sessions x tokens / s with every input resident in HBM; `e2e` = the same step with q, new
K/V rows, selection lists and positions copied from pinned host memory and the outputs copied back
inside the timed region.  L2 is defeated by rotation: consecutive steps run on different replicas
of the session group (own caches, own lists), sized so that >= 512 MB of distinct rows pass between
two uses of the same row.

Extra objects on the same JSON line (rank 0, 1 GPU): `single_session_ctx262144` (QSA decode, batch
1, us per layer under graph replay), `dense_ctx262144` (full attention over 262144 rows for q8_0 /
f16 / f32), `roofline` for the dominant kernel and `cpu_baseline` (the CPU oracle on host cores).

`--impl reference` times the reference's own CPU arithmetic for the same step (the oracle port:
q8_0 quantise of the new rows + scalar attention over the dequantised selected rows) on all host
threads, on a bounded sample of the sessions.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "suzuqu-engine-4exp_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

N_LAYERS, N_HEAD, N_KVH, HD, WIDTH = 12, 16, 2, 128, 2051
SINK, RECENT, NRAND = 4, 1024, 1023
KVW = N_KVH * HD
ROW_BYTES = 136                       # one (token, kv head) q8_0 row: 128 codes + 4 fp16 scales
SCALE = 1.0 / math.sqrt(HD)
SEED = 20261125
PAD = 64                              # token slots a session can append between two rewinds (raised to fit --steps)
L2_BYTES = 126e6
# dram bytes (read + write) per algorithmic byte of the batched decode kernel, from one ncu capture of the
# kernel on a small case: 81.1 MB of dram traffic for 71.1 MB gathered (272-byte records are 16-byte, not
# sector aligned); traffic grows with the rows gathered, so a full launch scales by the same ratio
DECODE_TRAFFIC_RATIO = 1.14
TIMED_BLOCKS = 15              # the --steps block is timed this many times; the median block is reported


def draw_contexts(n, lo=1024, hi=131072, seed=SEED + 4):
    return np.random.default_rng(seed).integers(lo, hi + 1, n).astype(np.int64)


def selection(rng, ctx):
    """sorted unique {0..3} + 1023 random of [4, ctx-1024) + the last 1024; everything when ctx <= 2051"""
    out = np.full(WIDTH, -1, np.int32)
    if ctx <= WIDTH:
        out[:ctx] = np.arange(ctx)
        return out
    mid = rng.choice(ctx - RECENT - SINK, NRAND, replace=False) + SINK
    out[:] = np.sort(np.concatenate([np.arange(SINK), mid, np.arange(ctx - RECENT, ctx)]))
    return out


def gathered_bytes(ctx):
    """algorithmic bytes one layer's decode reads for one session: rows x kv heads x (K + V)"""
    return min(int(ctx), WIDTH) * N_KVH * ROW_BYTES * 2


class ClockSampler:
    """SM clock and throttle reasons while the timed steps run.  Reads NVML in a thread every ~2 ms (the
    timed region of a default run lasts tens of milliseconds, shorter than one nvidia-smi poll); falls
    back to an `nvidia-smi -lms` child when NVML cannot be opened.  Read-only: no setting is touched."""
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index, uuid=None):
        self.samples = []          # (t, sm_mhz, reasons bitmask)
        self.sm_max = None
        self.thread = self.proc = None
        self.stop_flag = False
        try:
            import pynvml as nv
            import threading
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByUUID(uuid) if uuid else nv.nvmlDeviceGetHandleByIndex(gpu_index)
            self.sm_max = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            bits = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
                    "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                    "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
                    "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
            self.bits = bits

            def poll():
                while not self.stop_flag:
                    try:
                        self.samples.append((time.perf_counter(),
                                             float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)),
                                             int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))))
                    except Exception:
                        pass
                    time.sleep(0.002)
            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        self.path = "/tmp/q4_bench_clocks_%d.csv" % os.getpid()
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, windows=()):
        """windows: (t0, t1) host-clock intervals of the timed regions; samples outside them are used only
        when fewer than three fall inside (then "window" says so)."""
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.thread:
            self.stop_flag = True
            self.thread.join(timeout=2)
            inside = [s for s in self.samples if any(a <= s[0] <= b for a, b in windows)]
            use, out["window"] = (inside, "timed regions") if len(inside) >= 3 else \
                                 (self.samples, "warm-up through the last timed step")
            if use:
                out["sm_mhz"] = float(np.median([s[1] for s in use]))
                out["sm_max_mhz"] = self.sm_max
                out["samples"] = len(use)
                mask = 0
                for s in use:
                    mask |= s[2]
                out["reasons"] = sorted(n for n, bit in self.bits.items() if mask & bit)
            out["source"] = "nvml"
            return out
        if not self.proc:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, v in zip(self.NAMES, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if sm:
            out["sm_mhz"] = float(np.median(sm))
            out["sm_max_mhz"] = float(max(mx))
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        out["source"] = "nvidia-smi"
        return out


# ------------------------------------------------------------------------------------------ CPU arm
def cpu_sample_problem(ctxs, n_sessions, seed):
    """Host-side copy of the step for the first n_sessions sessions: per (session, layer) the selected
    rows only, quantised by the oracle into a compact cache with the lists remapped onto it (same rows
    dequantised and dotted as on the full cache; the full 27 GB of caches is not materialised)."""
    from oracle import q4_oracle as oracle
    rng = np.random.default_rng(seed)
    items, news = [], []
    for s in range(n_sessions):
        ctx = int(ctxs[s])
        for layer in range(N_LAYERS):
            idx = np.stack([selection(rng, ctx) for _ in range(N_KVH)])
            live = np.unique(idx[idx >= 0])
            remap = np.full(ctx, -1, np.int32)
            remap[live] = np.arange(len(live), dtype=np.int32)
            cidx = np.where(idx >= 0, remap[np.maximum(idx, 0)], -1).astype(np.int32)
            rows = rng.standard_normal((2, len(live), KVW), dtype=np.float32)
            kc, vc = oracle.kv_write(rows[0], 2), oracle.kv_write(rows[1], 2)
            q = oracle.bf16_to_f32(oracle.f32_to_bf16(rng.standard_normal(N_HEAD * HD, dtype=np.float32)))
            items.append(dict(q=q, kc=kc, vc=vc, out=np.empty(N_HEAD * HD, np.float32), idx=cidx, width=WIDTH,
                              idx_kvh_stride=WIDTH, kv_base=0, max_kv=len(live)))
            news.append(rng.standard_normal((2, KVW), dtype=np.float32))
    return items, news


def cpu_step(items, news, threads):
    """one decoded token for the sampled sessions: quantise the new K and V rows of every layer
    (kv_write), then sparse attention of every (session, layer) on `threads` host threads"""
    from oracle import q4_oracle as oracle
    for nw in news:
        oracle.kv_write(nw[0], 2)
        oracle.kv_write(nw[1], 2)
    oracle.attn_items(items, N_HEAD, N_KVH, HD, SCALE, 2, threads)


def cpu_baseline(ctxs, budget_s, n_sessions=4):
    """the oracle port on all host processors, and on one thread (the reference's CPU attention loop is
    serial, src/q4_fwd.c:369-397), each on the same bounded sample"""
    from oracle import q4_oracle as oracle
    threads = max(1, oracle.host_procs())
    items, news = cpu_sample_problem(ctxs, n_sessions, SEED + 9)

    def run(n_threads, budget):
        cpu_step(items, news, n_threads)            # warm-up
        t0 = time.perf_counter()
        reps = 0
        while reps < 2 or time.perf_counter() - t0 < budget:
            cpu_step(items, news, n_threads)
            reps += 1
            if time.perf_counter() - t0 > 3 * budget:
                break
        return n_sessions * reps / (time.perf_counter() - t0), reps, time.perf_counter() - t0
    v, reps, dt = run(threads, budget_s)
    v1, reps1, dt1 = run(1, budget_s / 2)
    return {"value": v, "unit": "session*tok/s", "cores": threads, "kind": "port",
            "sample": "%d of the 64 sessions x 12 layers x %d reps (%.1f s); compact caches of the selected rows"
                      % (n_sessions, reps, dt),
            "value_1_thread": v1, "sample_1_thread": "same sample, %d reps (%.1f s) on one thread" % (reps1, dt1)}


def run_reference_arm(args, rank):
    if rank != 0:
        return
    from oracle import q4_oracle as oracle
    ctxs = draw_contexts(args.sessions)
    n_s = 4
    threads = max(1, oracle.host_procs())
    items, news = cpu_sample_problem(ctxs, n_s, SEED + 9)
    for _ in range(args.warmup):
        cpu_step(items, news, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(items, news, threads)
    dt = time.perf_counter() - t0
    v = n_s * args.steps / dt
    line = {"impl": "reference", "metric": "decode_attn_session_tok_per_s", "value": v, "unit": "session*tok/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "q8_0+f32",
            "data": "synthetic", "config": workload_config(args.sessions),
            "cpu_baseline": {"value": v, "unit": "session*tok/s", "cores": threads, "kind": "port",
                             "sample": "each step = %d of the 64 sessions x 12 layers (compact caches of the "
                                       "selected rows), all host threads" % n_s},
            "e2e": {"value": v, "unit": "session*tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(sessions):
    return {"workload": "configs[3]: multi-session batched QSA decode, %d sessions, ctx ~ U[1024,131072], "
                        "q8_0 KV, 12 layers x (fused K/V append + sparse decode attention), 16 Q / 2 KV heads, "
                        "hd 128, 2051 selected positions per kv head" % sessions,
            "sessions": sessions, "layers": N_LAYERS, "selected_positions": WIDTH, "kv": "q8_0", "q": "bf16",
            "parallelism": "sessions sharded round-robin, no collective",
            "l2": "rotation over replicas of the session group (>=512 MB of distinct rows between two uses of a row)"}


# ------------------------------------------------------------------------------------------ GPU arm
class Group:
    """One replica of this rank's session group: caches, selection lists, per-step inputs, graph."""

    def __init__(self, q4gpu, torch, ctxs, seed, fill=True):
        self.torch, self.q4gpu = torch, q4gpu
        self.ctxs = [int(c) for c in ctxs]
        n = len(self.ctxs)
        self.n = n
        rng = np.random.default_rng(seed)
        self.stores = [q4gpu.KVStore(N_LAYERS, N_KVH, HD, c + PAD, q4gpu.KIND_Q8) for c in self.ctxs]
        if fill:
            for st, c in zip(self.stores, self.ctxs):
                fill_store(torch, st, c)
        self.batch = q4gpu.Batch(self.stores)
        idx = np.empty((N_LAYERS, n, N_KVH, WIDTH), np.int32)
        for layer in range(N_LAYERS):
            for s, c in enumerate(self.ctxs):
                for kh in range(N_KVH):
                    idx[layer, s, kh] = selection(rng, c)
        # The step's inputs live in ONE pinned host buffer and ONE device buffer (q | k | v | lists, each part
        # 256-byte aligned), so the upload of a step is a single copy; the tensors below are views into them.
        parts = [("q", torch.bfloat16, (N_LAYERS, n, N_HEAD, HD)), ("k", torch.float32, (N_LAYERS, n, KVW)),
                 ("v", torch.float32, (N_LAYERS, n, KVW)), ("idx", torch.int32, (N_LAYERS, n, N_KVH, WIDTH))]
        offs, total = {}, 0
        for name, dt, shape in parts:
            offs[name] = total
            total += (int(np.prod(shape)) * torch.empty(0, dtype=dt).element_size() + 255) // 256 * 256
        self.in_h = torch.empty(total, dtype=torch.uint8).pin_memory()
        self.in_d = torch.empty(total, dtype=torch.uint8, device="cuda")

        def view(buf, name, dt, shape):
            nbytes = int(np.prod(shape)) * torch.empty(0, dtype=dt).element_size()
            return buf[offs[name]:offs[name] + nbytes].view(dt).view(*shape)
        for name, dt, shape in parts:
            setattr(self, name + "_h", view(self.in_h, name, dt, shape))
            setattr(self, name, view(self.in_d, name, dt, shape))
        self.idx_h.copy_(torch.from_numpy(idx))
        self.q_h.copy_(torch.randn(N_LAYERS, n, N_HEAD, HD).to(torch.bfloat16))
        self.k_h.copy_(torch.randn(N_LAYERS, n, KVW))
        self.v_h.copy_(torch.randn(N_LAYERS, n, KVW))
        self.in_d.copy_(self.in_h)
        self.out_h = torch.empty(N_LAYERS, n, N_HEAD, HD).pin_memory()
        self.out = torch.empty(N_LAYERS, n, N_HEAD, HD, device="cuda")
        self.t = 0
        self.graph = None
        self.pipe = None                      # events of this group's upload / graph / download (q4_gpu_pipe)

    def enqueue_layers(self):
        # one launch per layer: the attention kernel quantises and stores each session's new K/V row itself
        for layer in range(N_LAYERS):
            self.batch.append_decode(layer, self.k[layer], self.v[layer], self.q[layer], self.out[layer], N_HEAD,
                                     SCALE, idx=self.idx[layer], width=WIDTH, idx_kvh_stride=WIDTH,
                                     idx_sess_stride=N_KVH * WIDTH, q_bf16=True)

    def capture(self, L):
        """one decode step = one graph: every session's position moves on by one on the device, then the layers"""
        assert L.q4_hip_graph_begin() == 1
        self.batch.advance(1)
        self.enqueue_layers()
        self.graph = L.q4_hip_graph_end()
        assert self.graph, "graph capture failed"

    def rewind(self):
        """positions back to one before the first free slot, so that the next step appends at slot ctx; called
        between timed blocks (the stores have room for PAD appended tokens)"""
        self.batch.set_pos([c - 1 for c in self.ctxs])
        self.t = 0

    def step(self, L):
        """the token at slot ctx + t of every session: a graph replay, nothing else"""
        assert self.t < PAD, "more steps than the stores have room for between two rewinds"
        self.t += 1
        assert L.q4_hip_graph_launch(self.graph)

    def copy_in(self, L):
        """this step's inputs from pinned host memory, on the library's copy stream, after the previous step
        that read these device buffers (the pipe orders it)"""
        if self.pipe is None:
            self.pipe = L.q4_gpu_pipe_create()
            assert self.pipe
        assert L.q4_gpu_pipe_upload(self.pipe, self.in_d.data_ptr(), self.in_h.data_ptr(), self.in_h.numel())

    def run_e2e(self, L):
        """the step's graph on the library's stream once the inputs are in and the previous result of this
        group is out; the result goes back on the download stream"""
        assert self.t < PAD, "more steps than the stores have room for between two rewinds"
        self.t += 1
        assert L.q4_gpu_pipe_run(self.pipe, self.graph, self.out_h.data_ptr(), self.out.data_ptr(), self.out.numel() * 4)

    def e2e_bytes(self):
        h2d = self.in_h.numel()                       # the packed inputs (positions advance on the device)
        return h2d, self.out_h.numel() * 4

    def algorithmic_bytes_per_layer(self):
        return sum(gathered_bytes(c) for c in self.ctxs)


def fill_store(torch, st, rows, chunk=32768):
    """cache contents N(0,1) before quantisation: rows generated on the device and appended (quantised)
    through the library"""
    for layer in range(st.n_layers):
        for p0 in range(0, rows, chunk):
            n = min(chunk, rows - p0)
            k = torch.randn(n, st.n_kvh * st.hd, device="cuda")
            v = torch.randn(n, st.n_kvh * st.hd, device="cuda")
            st.append(layer, k, v, p0, n)


def close_enough(got, ref, extra_rel=0.0):
    """the stated tolerance of the path: 2e-3 max-abs + 1e-3 relative against the fp32 oracle (extra_rel: one
    bf16 rounding of the result where the output type is bf16); returns (ok, max abs error)"""
    got, ref = np.asarray(got, np.float64).reshape(-1), np.asarray(ref, np.float64).reshape(-1)
    err = np.abs(got - ref)
    ok = bool(np.isfinite(got).all() and (err <= 2e-3 + (1e-3 + extra_rel) * np.abs(ref)).all())
    return ok, float(err.max())


def export_layer(torch, L, st, layer, rows):
    """rows [0, rows) of one layer of a store as the reference-layout bytes the oracle reads (K, V)"""
    out = []
    for which in (0, 1):
        buf = torch.empty(rows * st.token_bytes, dtype=torch.uint8, device="cuda")
        st.export(layer, which, 0, rows, buf)
        assert L.q4_hip_stream_sync()
        out.append(buf.cpu().numpy())
    return out


def verify_decode(torch, L, st, layer, q_bf16_t, out_t, rows, idx=None, kind=2, n_kv=None):
    """one decode result (out_t, computed from the bf16 query q_bf16_t over the store's layer) against the
    CPU oracle on the exported cache bytes: a list of positions per kv head (idx [N_KVH][WIDTH]) or dense"""
    from oracle import q4_oracle as oracle
    kc, vc = export_layer(torch, L, st, layer, rows)
    assert L.q4_hip_stream_sync()
    torch.cuda.synchronize()
    q = q_bf16_t.float().cpu().numpy().reshape(-1)
    threads = max(1, oracle.host_procs())
    if idx is not None:
        ref = oracle.attn(q, kc, vc, None, N_HEAD, N_KVH, HD, 1, 0, rows, SCALE, kind, idx=np.ascontiguousarray(idx, np.int32),
                          width=idx.shape[-1], idx_kvh_stride=idx.shape[-1] if idx.ndim > 1 else 0, threads=threads)[0]
    else:
        ref = oracle.attn(q, kc, vc, None, N_HEAD, N_KVH, HD, 1, n_kv - 1, rows, SCALE, kind, threads=threads)[0]
    return close_enough(out_t.float().cpu().numpy(), ref)


def timed(torch, ext, fn, reps):
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(ext)
    for i in range(reps):
        fn(i)
    ev1.record(ext)
    ev1.synchronize()
    return ev0.elapsed_time(ev1) * 1e-3


def extras_single_session(torch, q4gpu, L, ext, peak_gbs):
    """configs[1]: one session at ctx 262144, batch 1, 12 layers; us per layer under graph replay"""
    ctx, R = 262144, 24
    g = []
    st = q4gpu.KVStore(N_LAYERS, N_KVH, HD, ctx + PAD, q4gpu.KIND_Q8)
    q4gpu.use_torch_stream()
    fill_store(torch, st, ctx)
    torch.cuda.synchronize()
    L.q4_gpu_set_stream(None)
    rng = np.random.default_rng(SEED + 2)
    idx = np.empty((R, N_LAYERS, N_KVH, WIDTH), np.int32)
    for r in range(R):                      # every replica selects around a different virtual end
        for layer in range(N_LAYERS):
            for kh in range(N_KVH):
                idx[r, layer, kh] = selection(rng, ctx - r * 2048)
    idx_d = torch.from_numpy(idx).cuda()
    q = torch.randn(R, N_LAYERS, N_HEAD, HD, device="cuda").to(torch.bfloat16)
    k = torch.randn(N_LAYERS, KVW, device="cuda")
    v = torch.randn(N_LAYERS, KVW, device="cuda")
    out = torch.empty(N_LAYERS, N_HEAD, HD, device="cuda")
    torch.cuda.synchronize()
    graphs, graphs_attn = [], []
    for with_append, dst in ((True, graphs), (False, graphs_attn)):
        for r in range(R):
            assert L.q4_hip_graph_begin() == 1
            for layer in range(N_LAYERS):
                if with_append:      # append fused into the attention launch
                    st.append_decode_d(layer, k[layer], v[layer], q[r, layer], out[layer], N_HEAD, SCALE,
                                       idx=idx_d[r, layer], width=WIDTH, idx_kvh_stride=WIDTH, q_bf16=True)
                else:
                    st.decode(layer, q[r, layer], out[layer], N_HEAD, SCALE, idx=idx_d[r, layer], width=WIDTH,
                              idx_kvh_stride=WIDTH, n_kv=0, q_bf16=True)
            gr = L.q4_hip_graph_end()
            assert gr
            dst.append(gr)
    res = {}
    for name, gl in (("us_per_layer", graphs), ("us_per_layer_attn_only", graphs_attn)):
        def one(i, gl=gl):
            L.q4_hip_pos_push(ctx + (i % PAD))
            assert L.q4_hip_graph_launch(gl[i % R])
        timed(torch, ext, one, R)
        n = 10 * R
        dt = timed(torch, ext, one, n)
        res[name] = 1e6 * dt / (n * N_LAYERS)
    # check: one layer of one replica, recomputed outside the graph, against the oracle on the exported rows
    L.q4_hip_pos_push(ctx)
    st.decode(3, q[5, 3], out[3], N_HEAD, SCALE, idx=idx_d[5, 3], width=WIDTH, idx_kvh_stride=WIDTH, n_kv=0, q_bf16=True)
    ok, err = verify_decode(torch, L, st, 3, q[5, 3], out[3], ctx + PAD, idx=idx[5, 3])
    res["verified"], res["max_err"] = ok, err
    by = gathered_bytes(ctx)
    gbs = by / (res["us_per_layer"] * 1e-6) / 1e9
    res.update({"workload": "configs[1]: single-session QSA decode, ctx 262144, batch 1, 12 layers, graph replay, "
                            "%d rotating selections" % R,
                "gathered_bytes_per_layer": by, "achieved_gbs": gbs, "frac_of_measured_hbm": gbs / peak_gbs,
                "tok_per_s": 1e6 / (res["us_per_layer"] * N_LAYERS),
                "note": "latency-bound: 1.1 MB per dependent layer is 0.17 us of HBM time"})
    for gr in graphs + graphs_attn:
        L.q4_hip_graph_free(gr)
    st.close()
    return res


def extras_prefill(torch, q4gpu, L, ext, peaks):
    """configs[2]: append 8192 new tokens (fp32 N(0,1), quantised to q8_0) into a 16384-token q8_0 cache, then
    causal dense attention of the 8192 bf16 queries over all 24576 keys on the tensor cores, bf16 out"""
    base, n_tok, n_layers = 16384, 8192, 4       # 4 layers rotate so Q/out (67 MB per layer) do not sit in L2
    st = q4gpu.KVStore(n_layers, N_KVH, HD, base + n_tok, q4gpu.KIND_Q8)
    q4gpu.use_torch_stream()
    fill_store(torch, st, base)
    knew = torch.randn(n_tok, KVW, device="cuda")
    vnew = torch.randn(n_tok, KVW, device="cuda")
    q = torch.randn(n_layers, n_tok, N_HEAD, HD, device="cuda").to(torch.bfloat16)
    out = torch.empty(n_layers, n_tok, N_HEAD, HD, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    L.q4_gpu_set_stream(None)

    def app(i):
        st.append(i % n_layers, knew, vnew, base, n_tok)

    def att(i):
        st.prefill(i % n_layers, q[i % n_layers], out[i % n_layers], N_HEAD, n_tok, base, SCALE)
    timed(torch, ext, app, n_layers)
    t_app = timed(torch, ext, app, 4 * n_layers) / (4 * n_layers)
    timed(torch, ext, att, n_layers)
    t_att = timed(torch, ext, att, 2 * n_layers) / (2 * n_layers)
    # check: sampled queries of the last call against the oracle (bf16 result: one more rounding allowed)
    from oracle import q4_oracle as oracle
    lay = (2 * n_layers - 1) % n_layers
    kc, vc = export_layer(torch, L, st, lay, base + n_tok)
    ok, err = True, 0.0
    for t in (0, 4097, n_tok - 1):
        ref = oracle.attn(q[lay, t].float().cpu().numpy().reshape(-1), kc, vc, None, N_HEAD, N_KVH, HD, 1, base + t, base + n_tok,
                          SCALE, 2, threads=max(1, oracle.host_procs()))[0]
        o, e = close_enough(out[lay, t].float().cpu().numpy(), ref, extra_rel=2.0 ** -8)
        ok, err = ok and o, max(err, e)
    pairs = sum(base + t + 1 for t in range(n_tok))
    flop = pairs * 4 * HD * N_HEAD
    peak_tf = float(peaks.get("bf16_tflops", 1590.0))
    st.close()
    return {"workload": "configs[2]: chunked prefill, 8192 new tokens over a 16384-token q8_0 cache, 16 Q / 2 KV heads, "
                        "hd 128, bf16 Q and out",
            "append_us": t_app * 1e6, "append_gbs": 2 * n_tok * (KVW * 4 + N_KVH * ROW_BYTES) / t_app / 1e9,
            "attn_ms_per_layer": t_att * 1e3, "flop_per_layer": flop, "achieved_tflops": flop / t_att / 1e12,
            "peak_tflops_measured_bf16": peak_tf, "frac_of_measured_tensor": flop / t_att / 1e12 / peak_tf,
            "queries_per_s": n_tok / (t_app + t_att), "verified": ok, "max_err": err}


def extras_indexer(torch, q4gpu, L, ext, peak_gbs):
    """QSA indexer at ctx 262144 (the step that produces the lists): per layer, score 65536 pooled blocks
    (4 indexer heads, fp32 pool = 33.5 MB) and select the top 512 + tail into a 2051-wide list, at the device
    position word; 12 layers x (score + select) captured in one graph, pools of the 12 layers 402 MB >> L2"""
    pos, ratio, n_head, k_blk = 262143, 4, 4, 512
    nb = (pos + 1) // ratio
    pool = torch.randn(N_LAYERS, nb, HD, device="cuda")
    q = torch.randn(N_LAYERS, n_head, HD, device="cuda")
    score = torch.empty(N_LAYERS, nb, device="cuda")
    sel = torch.empty(N_LAYERS, WIDTH, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    L.q4_hip_pos_push(pos)

    def enqueue(with_select):
        for l in range(N_LAYERS):
            assert L.q4_hip_qsa_score_d(q[l].data_ptr(), pool[l].data_ptr(), score[l].data_ptr(), nb, n_head, HD, ratio)
            if with_select:
                assert L.q4_hip_qsa_topk_d(score[l].data_ptr(), sel[l].data_ptr(), nb, k_blk, ratio, WIDTH)
    res = {}
    for name, with_select in (("score_plus_select_us_per_layer", True), ("score_us_per_layer", False)):
        enqueue(with_select)
        assert L.q4_hip_graph_begin() == 1
        enqueue(with_select)
        gr = L.q4_hip_graph_end()
        assert gr

        def one(i, gr=gr):
            assert L.q4_hip_graph_launch(gr)
        timed(torch, ext, one, 3)
        res[name] = 1e6 * timed(torch, ext, one, 10) / (10 * N_LAYERS)
        L.q4_hip_graph_free(gr)
    # check: the last layer's list against the oracle's selection on the oracle's scores (exact equality)
    from oracle import q4_oracle as oracle
    enqueue(True)
    assert L.q4_hip_stream_sync()
    torch.cuda.synchronize()
    l_chk = N_LAYERS - 1
    sc_ref = oracle.ix_score(q[l_chk].cpu().numpy(), pool[l_chk].cpu().numpy(), 1, nb, nb, n_head, pos, ratio)
    sel_ref = oracle.ix_topk(sc_ref, 1, nb, k_blk, ratio, pos, WIDTH)[0]
    res["verified"] = bool(np.array_equal(sel[l_chk].cpu().numpy(), sel_ref) and
                           np.array_equal(score[l_chk].cpu().numpy().view(np.uint32), sc_ref[0].view(np.uint32)))
    # ---- the whole decode-attention step of one session at ctx 262144, selection included: per layer score,
    # select, then the fused append + sparse decode over the list just produced (one list shared by both kv
    # heads, as the reference's); 24 graphs with different indexer queries rotate so that the gathered rows
    # (13 MB per graph) do not stay in L2
    R = 24
    st = q4gpu.KVStore(N_LAYERS, N_KVH, HD, pos + 1, q4gpu.KIND_Q8)
    q4gpu.use_torch_stream()
    fill_store(torch, st, pos + 1)
    torch.cuda.synchronize()
    L.q4_gpu_set_stream(None)
    qix = torch.randn(R, N_LAYERS, n_head, HD, device="cuda")
    qa = torch.randn(N_LAYERS, N_HEAD, HD, device="cuda").to(torch.bfloat16)
    knew = torch.randn(N_LAYERS, KVW, device="cuda")
    vnew = torch.randn(N_LAYERS, KVW, device="cuda")
    out = torch.empty(N_LAYERS, N_HEAD, HD, device="cuda")
    torch.cuda.synchronize()
    L.q4_hip_pos_push(pos)

    def layer_step(r, l):
        assert L.q4_hip_qsa_score_d(qix[r, l].data_ptr(), pool[l].data_ptr(), score[l].data_ptr(), nb, n_head, HD, ratio)
        assert L.q4_hip_qsa_topk_d(score[l].data_ptr(), sel[l].data_ptr(), nb, k_blk, ratio, WIDTH)
        st.append_decode_d(l, knew[l], vnew[l], qa[l], out[l], N_HEAD, SCALE, idx=sel[l], width=WIDTH, idx_kvh_stride=0,
                           q_bf16=True)
    graphs = []
    for r in range(R):
        if r == 0:
            for l in range(N_LAYERS):
                layer_step(r, l)
        assert L.q4_hip_graph_begin() == 1
        for l in range(N_LAYERS):
            layer_step(r, l)
        gr = L.q4_hip_graph_end()
        assert gr
        graphs.append(gr)

    def one(i):
        assert L.q4_hip_graph_launch(graphs[i % R])
    timed(torch, ext, one, R)
    res["select_plus_attend_us_per_layer"] = 1e6 * timed(torch, ext, one, 2 * R) / (2 * R * N_LAYERS)
    status = L.q4_gpu_last_error()
    assert status == 0, "device status %#x" % status
    for gr in graphs:
        L.q4_hip_graph_free(gr)
    st.close()
    # ---- batched form: 8 sessions at ctx 262144, one score launch and one selection launch per layer for all of
    # them (q4_gpu_qsa_select_batch); 4 rotating pool sets of 8 x 33.5 MB, far beyond L2
    n_sess, sets = 8, 4
    del pool, score, sel
    torch.cuda.empty_cache()
    bpool = torch.randn(sets, n_sess, nb, HD, device="cuda")
    ptrs = torch.tensor([[bpool[g, i].data_ptr() for i in range(n_sess)] for g in range(sets)], dtype=torch.int64, device="cuda")
    bpos = torch.full((n_sess,), pos, dtype=torch.int32, device="cuda")
    bq = torch.randn(n_sess, n_head, HD, device="cuda")
    bscore = torch.empty(n_sess, nb, device="cuda")
    bsel = torch.empty(n_sess, WIDTH, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()

    def batch_one(i):
        assert L.q4_gpu_qsa_select_batch(ptrs[i % sets].data_ptr(), bpos.data_ptr(), bq.data_ptr(), bscore.data_ptr(),
                                         bsel.data_ptr(), n_sess, nb, n_head, HD, k_blk, ratio, WIDTH)
    timed(torch, ext, batch_one, sets)
    dtb = timed(torch, ext, batch_one, 6 * sets) / (6 * sets)
    by = nb * HD * 4
    res["batch8_score_plus_select_us_per_layer"] = dtb * 1e6
    res["batch8_pool_gbs"] = n_sess * by / dtb / 1e9
    res["batch8_pool_frac_of_measured_hbm"] = n_sess * by / dtb / 1e9 / peak_gbs
    del bpool
    res.update({"workload": "QSA indexer, ctx 262144: 65536 pooled blocks x 4 heads scored, exact top-512 + tail -> 2051 positions; "
                            "select_plus_attend = score + select + fused append + sparse decode over the produced list",
                "pool_bytes_per_layer": by, "score_gbs": by / res["score_us_per_layer"] / 1e3,
                "score_frac_of_measured_hbm": by / res["score_us_per_layer"] / 1e3 / peak_gbs})
    return res


def extras_dense(torch, q4gpu, L, ext, peak_gbs, kinds=("q8_0", "f16", "f32")):
    """configs[4] on one GPU: full attention over 262144 rows, q8_0 / f16 / f32 KV, 12 layers"""
    ctx = 262144
    res = {}
    for name, kind, rowb in (("q8_0", 2, 136), ("f16", 1, 256), ("f32", 0, 512)):
        if name not in kinds:
            continue
        st = q4gpu.KVStore(N_LAYERS, N_KVH, HD, ctx, kind)
        q4gpu.use_torch_stream()
        fill_store(torch, st, ctx)
        torch.cuda.synchronize()
        L.q4_gpu_set_stream(None)
        q = torch.randn(N_LAYERS, N_HEAD, HD, device="cuda").to(torch.bfloat16)
        out = torch.empty(N_LAYERS, N_HEAD, HD, device="cuda")
        torch.cuda.synchronize()

        def one(i):
            layer = i % N_LAYERS
            st.decode(layer, q[layer], out[layer], N_HEAD, SCALE, n_kv=ctx, q_bf16=True)
        timed(torch, ext, one, N_LAYERS)
        n = 4 * N_LAYERS
        dt = timed(torch, ext, one, n)
        by = ctx * N_KVH * rowb * 2
        us = 1e6 * dt / n
        ok, err = verify_decode(torch, L, st, N_LAYERS - 1, q[N_LAYERS - 1], out[N_LAYERS - 1], ctx, kind=kind, n_kv=ctx)
        res[name] = {"us_per_layer": us, "bytes_per_layer": by, "achieved_gbs": by / us / 1e3,
                     "frac_of_measured_hbm": by / us / 1e3 / peak_gbs, "verified": ok, "max_err": err}
        st.close()
    res["workload"] = "configs[4] on 1 GPU: dense decode over ctx 262144, 12 layers, inputs 12 x bytes_per_layer >> L2"
    return res


def extras_snapshot(torch, q4gpu, L, ext):
    """session prefix save / restore at configs[3]'s mean context (66048 rows x 12 layers, q8_0): bulk strided
    copies to a device pool and to pinned host memory, and the reference session-file byte order streamed
    through a file descriptor (an in-memory file, so the figure is the library's, not a disk's)"""
    n_kv, max_kv = 66048, 131072
    st = q4gpu.KVStore(N_LAYERS, N_KVH, HD, max_kv, q4gpu.KIND_Q8)
    q4gpu.use_torch_stream()
    fill_store(torch, st, n_kv)
    torch.cuda.synchronize()
    L.q4_gpu_set_stream(None)
    by = st.snapshot_bytes(n_kv)
    pool = torch.empty(4, by, dtype=torch.uint8, device="cuda")     # 4 slots > L2 between two uses of one
    host = torch.empty(by, dtype=torch.uint8).pin_memory()
    res = {"workload": "one session, %d rows x %d layers q8_0 (K and V)" % (n_kv, N_LAYERS), "bytes": by}
    for name, fn, reps, moved in (
            ("save_device", lambda i: st.save(n_kv, pool[i % 4]), 8, 2 * by),
            ("restore_device", lambda i: st.restore(n_kv, pool[i % 4]), 8, 2 * by),
            ("save_pinned_host", lambda i: st.save(n_kv, host, host=True), 3, by),
            ("restore_pinned_host", lambda i: st.restore(n_kv, host, host=True), 3, by)):
        timed(torch, ext, fn, 2)
        dt = timed(torch, ext, fn, reps) / reps
        res[name] = {"ms": dt * 1e3, "gbs": moved / dt / 1e9}
    fd = os.memfd_create("q4_session_kv")
    try:
        st.write_fd(n_kv, fd)                                        # warm-up: staging buffers, page faults
        os.lseek(fd, 0, os.SEEK_SET)
        t0 = time.perf_counter()
        st.write_fd(n_kv, fd)
        t1 = time.perf_counter()
        file_bytes = os.lseek(fd, 0, os.SEEK_CUR)
        os.lseek(fd, 0, os.SEEK_SET)
        st.read_fd(n_kv, fd)
        os.lseek(fd, 0, os.SEEK_SET)
        t2 = time.perf_counter()
        st.read_fd(n_kv, fd)
        t3 = time.perf_counter()
    finally:
        os.close(fd)
    # check: the restored store (device pool, host, file: the last restore was the file's) exports the bytes it held
    probe = torch.empty(512 * st.token_bytes, dtype=torch.uint8, device="cuda")
    st.export(7, 1, n_kv - 512, 512, probe)
    before = probe.clone()
    st.save(n_kv, pool[0])
    z = torch.zeros(512, KVW, device="cuda")
    q4gpu.use_torch_stream()
    st.append(7, z, z, n_kv - 512, 512)
    torch.cuda.synchronize()
    L.q4_gpu_set_stream(None)
    st.restore(n_kv, pool[0])
    st.export(7, 1, n_kv - 512, 512, probe)
    assert L.q4_hip_stream_sync()
    res["verified"] = bool(torch.equal(before, probe))
    res["write_fd"] = {"ms": (t1 - t0) * 1e3, "gbs": file_bytes / (t1 - t0) / 1e9, "file_bytes": file_bytes}
    res["read_fd"] = {"ms": (t3 - t2) * 1e3, "gbs": file_bytes / (t3 - t2) / 1e9}
    st.close()
    return res


def extras_sparse_prefill(torch, q4gpu, L, ext, peak_gbs):
    """sparse prefill (the n_tok > 1 indexed form): 512 queries at the end of a 262144-row context, each
    with its own 2051-entry list per kv head (4 sink + 1024 recent + 1023 spread over the rest, one random
    row per stratum), one launch per layer on the q8_0 store"""
    ctx, n_tok = 262144, 512
    st = q4gpu.KVStore(N_LAYERS, N_KVH, HD, ctx, q4gpu.KIND_Q8)
    q4gpu.use_torch_stream()
    fill_store(torch, st, ctx)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(SEED + 9)
    pos = torch.arange(ctx - n_tok, ctx, device="cuda").view(n_tok, 1, 1)             # the query's own row
    sink = torch.arange(4, device="cuda").view(1, 1, 4).expand(n_tok, N_KVH, 4)
    recent = pos - 1023 + torch.arange(1024, device="cuda").view(1, 1, 1024)
    span = (pos - 1023 - 4).to(torch.float64)                                          # rows [4, pos - 1023)
    u = torch.rand(n_tok, N_KVH, 1023, device="cuda", dtype=torch.float64, generator=gen)
    spread = 4 + ((torch.arange(1023, device="cuda").view(1, 1, 1023) + u) * span / 1023).long()
    idx = torch.cat([sink, spread, recent.expand(n_tok, N_KVH, 1024)], 2).to(torch.int32).contiguous()
    assert idx.shape[2] == WIDTH and int(idx.max()) < ctx and int(idx.min()) >= 0
    q = torch.randn(N_LAYERS, n_tok, N_HEAD, HD, device="cuda").to(torch.bfloat16)
    out = torch.empty(N_LAYERS, n_tok, N_HEAD, HD, device="cuda")
    torch.cuda.synchronize()
    L.q4_gpu_set_stream(None)

    def one(i):
        layer = i % N_LAYERS
        st.decode_idx_n(layer, q[layer], out[layer], N_HEAD, SCALE, idx, WIDTH, n_tok,
                        idx_tok_stride=N_KVH * WIDTH, idx_kvh_stride=WIDTH, q_bf16=True)
    timed(torch, ext, one, N_LAYERS)
    n = 2 * N_LAYERS
    dt = timed(torch, ext, one, n) / n
    gathered = n_tok * N_KVH * WIDTH * 272
    distinct = int(torch.unique(idx[:, 0]).numel() + torch.unique(idx[:, 1]).numel()) * 272
    lay = (2 * N_LAYERS - 1) % N_LAYERS
    ok, err = verify_decode(torch, L, st, lay, q[lay, 17], out[lay, 17], ctx, idx=idx[17].cpu().numpy())
    st.close()
    return {"workload": "512 queries x 2051 rows per kv head over ctx 262144, q8_0, one launch per layer",
            "us_per_layer": dt * 1e6, "us_per_query": dt * 1e6 / n_tok, "gathered_bytes_per_layer": gathered,
            "distinct_row_bytes_per_layer": distinct, "gathered_gbs": gathered / dt / 1e9,
            "distinct_gbs": distinct / dt / 1e9, "distinct_frac_of_measured_hbm": distinct / dt / 1e9 / peak_gbs,
            "verified": ok, "max_err": err,
            "note": "lists of neighbouring queries overlap, so most gathers hit L2; the HBM floor is the distinct rows"}


def measure_seqshard(args, torch, q4gpu, L, dist, rank, world, peak_gbs):
    """configs[4]: one session at ctx 262144, dense attention; rank r owns an even contiguous slice of the
    rows and attends them; the (acc, m, l) records are exchanged and merged on every rank, either inside the
    decode kernel (peer stores over NVLink, q4_gpu_kv_decode_xchg: the product) or by an NCCL all-gather
    plus a merge kernel (timed beside it; the two results must agree).  One step = 12 layers; time = max over
    ranks, on the device.  Returns {kind: {...}} (the same on every rank)."""
    from q4gpu import shard
    ctx = 262144
    b, e = shard.rows_for_rank(ctx, rank, world)
    rows = e - b
    res = {}
    stream = torch.cuda.Stream()
    xw = q4gpu.Exchange(rank, world, N_HEAD, N_KVH, HD)
    comm = None
    if world > 1:
        xw.attach_all(dist)
        comm = q4gpu.Comm(rank, world, dist)
    for name, kind, rowb in (("q8_0", 2, 136), ("f16", 1, 256), ("f32", 0, 512)):
        if name not in args.dense_kinds.split(","):
            continue
        st = q4gpu.KVStore(N_LAYERS, N_KVH, HD, rows, kind)
        with torch.cuda.stream(stream):
            q4gpu.use_torch_stream()
            torch.manual_seed(SEED + rank)
            fill_store(torch, st, rows)
            torch.manual_seed(SEED)                       # the query is the same on every rank
            q = torch.randn(N_LAYERS, N_HEAD, HD, device="cuda").to(torch.bfloat16)
            part = torch.empty(N_LAYERS, N_HEAD, HD + 2, device="cuda")
            out = torch.empty(N_LAYERS, N_HEAD, HD, device="cuda")

            def step_nccl():
                for layer in range(N_LAYERS):
                    st.decode_partial(layer, q[layer], part[layer], N_HEAD, SCALE, n_kv=rows, q_bf16=True)
                    if world > 1:
                        allp = shard.exchange_records(part[layer])
                    else:
                        allp = part[layer:layer + 1]
                    q4gpu.check(L.q4_gpu_lse_merge(allp.data_ptr(), world, N_HEAD, HD, None, out[layer].data_ptr()),
                                "q4_gpu_lse_merge")

            def step_fused():
                # one launch per layer: attend the local rows, store the record into every peer's window
                # over NVLink, wait for theirs, merge
                for layer in range(N_LAYERS):
                    xw.decode(st, layer, q[layer], out_f[layer], SCALE, rows, q_bf16=True)

            def time_graph(step):
                for _ in range(max(args.warmup, 3)):
                    step()
                stream.synchronize()
                # the 12-layer step as one CUDA graph (NCCL and the library's launches are all captured on
                # this stream), so the host is out of the timed loop
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    q4gpu.use_torch_stream()
                    step()
                q4gpu.use_torch_stream()
                for _ in range(3):
                    graph.replay()
                stream.synchronize()
                if dist is not None:
                    dist.barrier()
                torch.cuda.synchronize()
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record(stream)
                for _ in range(args.steps):
                    graph.replay()
                ev1.record(stream)
                ev1.synchronize()
                dt = ev0.elapsed_time(ev1) * 1e-3
                del graph
                if dist is not None:
                    t = torch.tensor([dt], device="cuda", dtype=torch.float64)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    dt = float(t.item())
                return 1e6 * dt / (args.steps * N_LAYERS)

            def step_comm():
                # the library's own communicator (q4_gpu_comm_*): all-gather + merge behind one C call per layer
                for layer in range(N_LAYERS):
                    st.decode_partial(layer, q[layer], part[layer], N_HEAD, SCALE, n_kv=rows, q_bf16=True)
                    comm.allgather_merge(part[layer], parts_all[layer], N_HEAD, HD, out_c[layer])

            out_f = torch.zeros_like(out)
            out_c = torch.zeros_like(out)
            parts_all = torch.empty(N_LAYERS, world, N_HEAD, HD + 2, device="cuda")
            us_comm = time_graph(step_comm) if world > 1 else None
            us_nccl = time_graph(step_nccl) if world > 1 else None
            us = time_graph(step_fused)
            stream.synchronize()
            status = L.q4_gpu_last_error()
            assert status == 0, "device status %#x" % status
            agree = None
            if world > 1:      # the two exchanges must agree (same records, same merge arithmetic up to rounding)
                agree = max(float((out_f - out).abs().max()), float((out_c - out).abs().max()))
                assert agree < 2e-3, "the exchanges differ: %g" % agree
        by = ctx * N_KVH * rowb * 2
        res[name] = {"us_per_layer": us, "us_per_layer_nccl_allgather": us_nccl, "us_per_layer_library_nccl": us_comm,
                     "bytes_per_layer_all_ranks": by,
                     "achieved_gbs_all_ranks": by / us / 1e3,
                     "frac_of_measured_hbm_x_ranks": by / us / 1e3 / (peak_gbs * world),
                     "max_abs_diff_in_kernel_vs_nccl": agree}
        st.close()
    L.q4_gpu_set_stream(None)
    xw.close()
    if comm is not None:
        comm.close()
    res["exchange"] = ("in-kernel: %d B of {value, epoch} packets stored per peer per layer over NVLink, polled and merged "
                       "by the same launch; us_per_layer_nccl_allgather is the same step with torch.distributed's NCCL all-gather + "
                       "the merge kernel, us_per_layer_library_nccl with the library's own communicator (q4_gpu_comm_*)" % (N_HEAD * (HD + 4) * 8))
    return res


def measure_sessions(args, torch, q4gpu, L, dist, rank, world, local, mine, seed0, blocks, e2e=True, verify=True):
    """Times the batched decode step of this rank's sessions (`mine`: their context lengths): `blocks` blocks of
    --steps steps, each block bracketed by a barrier + synchronize on both sides and timed with CUDA events on
    the library's stream, max over ranks per block; the median block is reported.  Then the same with host
    buffers (uploads, downloads inside the timed region), then one session's output of the last step against
    the CPU oracle.  Returns a dict; frees everything it built."""
    global PAD
    PAD = max(PAD, args.steps + args.warmup + 8)      # a group takes at most that many steps between two rewinds
    step_bytes = N_LAYERS * sum(gathered_bytes(c) for c in mine)
    groups_n = args.groups or max(2, int(math.ceil(512e6 / max(step_bytes, 1))))
    torch.manual_seed(seed0)
    q4gpu.use_torch_stream()
    groups = [Group(q4gpu, torch, mine, seed0 + g) for g in range(groups_n)]
    torch.cuda.synchronize()
    L.q4_gpu_set_stream(None)                 # capture and timing on the library's own stream
    ext = torch.cuda.ExternalStream(L.q4_gpu_stream())
    for g in groups:
        g.batch.set_pos(g.ctxs)
        g.enqueue_layers()                    # eager once: scratch grows outside the capture
        g.capture(L)
        g.rewind()
    assert L.q4_hip_stream_sync()

    def barrier():
        L.q4_hip_stream_sync()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing
    sampler = ClockSampler(local, "GPU-" + str(torch.cuda.get_device_properties(local).uuid)) if rank == 0 else None
    for i in range(args.warmup):
        groups[i % groups_n].step(L)
    windows, block_dt = [], []
    step_no = args.warmup
    for blk in range(blocks):
        for g in groups:
            g.rewind()
        barrier()
        w0 = time.perf_counter()
        if blk == 0:
            torch.cuda.profiler.start()       # profilers started with capture off see one timed block only
        base = step_no
        dt = timed(torch, ext, lambda i: groups[(base + i) % groups_n].step(L), args.steps)
        if blk == 0:
            torch.cuda.profiler.stop()
        windows.append((w0, time.perf_counter()))
        step_no += args.steps
        barrier()
        block_dt.append(max_over_ranks(dt))
    dt = float(np.median(block_dt))
    res = {"dt": dt, "block_ms": [1e3 * x for x in block_dt], "groups": groups_n, "sessions_here": len(mine),
           "algorithmic_bytes_per_launch": groups[0].algorithmic_bytes_per_layer()}
    # ---- end to end: host buffers in, outputs out, every step
    # Uploads ride the library's copy stream and downloads its download stream, ordered against the compute
    # stream by the events of a q4_gpu_pipe per group (two C calls per step), so the inputs of step i+1 travel
    # while step i computes; every step's copies in and out are inside the timed region.
    if e2e:
        cs = torch.cuda.ExternalStream(L.q4_gpu_copy_stream())
        ds = torch.cuda.ExternalStream(L.q4_gpu_download_stream())

        def e2e_loop(n):
            groups[0].copy_in(L)
            for i in range(n):
                if i + 1 < n and groups_n > 1:
                    groups[(i + 1) % groups_n].copy_in(L)
                groups[i % groups_n].run_e2e(L)
                if i + 1 < n and groups_n == 1:          # one set of device buffers: no overlap possible
                    groups[0].copy_in(L)
        for g in groups:
            g.rewind()
        e2e_loop(3)
        e2e_dt = []
        for blk in range(max(3, blocks // 3)):
            for g in groups:
                g.rewind()
            barrier()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            w0 = time.perf_counter()
            ev0.record(ext)
            cs.wait_event(ev0)                     # no copy starts before the clock does
            e2e_loop(args.steps)
            ext.wait_stream(ds)                    # the last result is on the host before the clock stops
            ev1.record(ext)
            ev1.synchronize()
            windows.append((w0, time.perf_counter()))
            barrier()
            e2e_dt.append(max_over_ranks(ev0.elapsed_time(ev1) * 1e-3))
        res["dt_e2e"] = float(np.median(e2e_dt))
        res["e2e_block_ms"] = [1e3 * x for x in e2e_dt]
        res["h2d"], res["d2h"] = groups[0].e2e_bytes()
    res["clocks"] = sampler.stop(windows) if sampler else None
    status = L.q4_gpu_last_error()
    assert status == 0, "device status %#x" % status
    # ---- check: the shortest session's output of the last step of group 0, one layer, against the oracle
    if verify and rank == 0:
        g = groups[0]
        s_i = int(np.argmin(g.ctxs))
        layer = 5
        ok, err = verify_decode(torch, L, g.stores[s_i], layer, g.q[layer, s_i], g.out[layer, s_i], g.ctxs[s_i] + PAD,
                                idx=g.idx_h[layer, s_i].numpy())
        res["verified"], res["max_err"] = ok, err
    for g in groups:
        L.q4_hip_graph_free(g.graph)
        if g.pipe:
            L.q4_gpu_pipe_destroy(g.pipe)
        g.batch.close()
        for st in g.stores:
            st.close()
    groups.clear()
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sessions", type=int, default=64)
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--groups", type=int, default=0, help="replicas of the session group (0 = enough to defeat L2)")
    ap.add_argument("--blocks", type=int, default=TIMED_BLOCKS, help="how many times the --steps block is timed (median reported)")
    ap.add_argument("--ctx-max", type=int, default=131072, help="upper end of the context-length draw (profiling: small)")
    ap.add_argument("--only", default="", choices=["", "single", "dense", "prefill", "indexer", "snapshot", "sparse_prefill"],
                    help="run just one of the ctx-262144 extras (for profiler captures)")
    ap.add_argument("--dense-kinds", default="q8_0,f16,f32")
    ap.add_argument("--mode", default="sessions", choices=["sessions", "seqshard"],
                    help="sessions: the headline (sessions sharded over ranks); seqshard: one ctx-262144 "
                         "session, dense attention, rows sharded over ranks, records all-gathered (configs[4])")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import q4gpu
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: libq4gpu has no CPU path")
    torch.cuda.set_device(local)
    os.environ.setdefault("Q4_GPU_DEVICE", str(local))
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    L = q4gpu.init()
    assert L.q4_hip_qsa_topk_alloc()
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured (MEASURED_PEAKS.json)" if "hbm_gbs" in peaks else "fallback 6.65 TB/s"

    if args.mode == "seqshard":
        res = measure_seqshard(args, torch, q4gpu, L, dist, rank, world, peak_gbs)
        if rank == 0:
            print(json.dumps({"metric": "dense_decode_us_per_layer_ctx262144", "mode": "seqshard", "n_gpus": world,
                              "steps": args.steps, "exchange": res.pop("exchange"), "result": res}), flush=True)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return
    if args.only:
        ext = torch.cuda.ExternalStream(L.q4_gpu_stream())
        torch.manual_seed(SEED)
        if args.only == "single":
            res = extras_single_session(torch, q4gpu, L, ext, peak_gbs)
        elif args.only == "prefill":
            res = extras_prefill(torch, q4gpu, L, ext, peaks)
        elif args.only == "indexer":
            res = extras_indexer(torch, q4gpu, L, ext, peak_gbs)
        elif args.only == "snapshot":
            res = extras_snapshot(torch, q4gpu, L, ext)
        elif args.only == "sparse_prefill":
            res = extras_sparse_prefill(torch, q4gpu, L, ext, peak_gbs)
        else:
            res = extras_dense(torch, q4gpu, L, ext, peak_gbs, args.dense_kinds.split(","))
        print(json.dumps({"only": args.only, "result": res}), flush=True)
        return

    # ---- headline: the sessions of the whole job, sharded round-robin over the ranks (strong scaling)
    ctxs = draw_contexts(args.sessions, hi=args.ctx_max)
    mine = [int(c) for i, c in enumerate(ctxs) if i % world == rank]
    m = measure_sessions(args, torch, q4gpu, L, dist, rank, world, local, mine, SEED + 100 * rank, args.blocks)
    dt, dt_e2e = m["dt"], m["dt_e2e"]
    extras = {}
    if world > 1 and not args.no_extras:
        # weak scaling beside it: the full 64-session batch on EVERY rank (own contexts per rank), so the curve
        # separates the fixed per-launch time (which strong scaling of 64 sessions runs into) from anything else
        wctx = [int(c) for c in draw_contexts(args.sessions, hi=args.ctx_max, seed=SEED + 4 + 1000 * (rank + 1))]
        w = measure_sessions(args, torch, q4gpu, L, dist, rank, world, local, wctx, SEED + 7000 + 100 * rank,
                             max(3, args.blocks // 3), e2e=False, verify=False)
        extras["weak_scaling"] = {"scaling": "weak", "sessions_per_gpu": args.sessions, "n_gpus": world,
                                  "value": world * args.sessions * args.steps / w["dt"], "unit": "session*tok/s",
                                  "ms_per_step": 1e3 * w["dt"] / args.steps,
                                  "us_per_launch": 1e6 * w["dt"] / (args.steps * N_LAYERS)}
        # configs[4]: the sequence-sharded dense decode on the same ranks
        seq = measure_seqshard(args, torch, q4gpu, L, dist, rank, world, peak_gbs)
        if rank == 0:          # the one-GPU figure beside it, while the other ranks wait
            one = extras_dense(torch, q4gpu, L, torch.cuda.ExternalStream(L.q4_gpu_stream()), peak_gbs)
            for kname in ("q8_0", "f16", "f32"):
                if kname in seq and kname in one:
                    seq[kname]["us_per_layer_1_gpu"] = one[kname]["us_per_layer"]
                    seq[kname]["verified_1_gpu"] = one[kname]["verified"]
        dist.barrier()
        seq["workload"] = "configs[4]: one session, ctx 262144, dense attention, rows sharded evenly over %d GPUs" % world
        extras["seqshard_ctx262144"] = seq
    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel.  A step is 12 launches of one kernel (append fused into the sparse
    # decode), so its average launch duration is the device-timed region divided by the launches in it.
    dt_dec = dt / (args.steps * N_LAYERS)
    alg = m["algorithmic_bytes_per_launch"]
    achieved = alg / dt_dec / 1e9
    roofline = {"kernel": "q4_decode_k<q8_0 records, hd 128> (fused append + batched sparse decode, %d sessions per launch)" % len(mine),
                "bound": "hbm", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s", "frac": achieved / peak_gbs,
                "peak_source": peak_src, "algorithmic_bytes_per_launch": alg, "us_per_launch": dt_dec * 1e6,
                "traffic": (alg * DECODE_TRAFFIC_RATIO) if DECODE_TRAFFIC_RATIO else None}
    line = {"metric": "decode_attn_session_tok_per_s", "value": args.sessions * args.steps / dt,
            "unit": "session*tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "q8_0 KV, f16 tensor-core products, f32 accumulate", "data": "synthetic",
            "config": workload_config(args.sessions), "l2_replicas": m["groups"],
            "timing": {"blocks": len(m["block_ms"]), "steps_per_block": args.steps, "reported": "median block",
                       "block_ms_min": min(m["block_ms"]), "block_ms_max": max(m["block_ms"]),
                       "e2e_blocks": len(m["e2e_block_ms"])},
            "e2e": {"value": args.sessions * args.steps / dt_e2e, "unit": "session*tok/s",
                    "h2d_bytes_per_step": m["h2d"] * world, "d2h_bytes_per_step": m["d2h"] * world,
                    "ms_per_step": 1e3 * dt_e2e / args.steps},
            "gpu_launches": args.steps * (N_LAYERS + 1) * world,   # per step: the position advance + one kernel per layer
             "clocks": m["clocks"], "roofline": roofline,
            "us_per_layer": 1e6 * dt / (args.steps * N_LAYERS),
            "attn_roofline_session_tok_per_s": args.sessions / (N_LAYERS * sum(gathered_bytes(c) for c in ctxs)
                                                                / world / (peak_gbs * 1e9))}
    checks = {"headline": {"verified": m.get("verified"), "max_err": m.get("max_err"),
                           "what": "one session x one layer of the last step against the CPU oracle on the exported cache"}}
    line.update(extras)
    if world == 1 and not args.no_extras:
        ext = torch.cuda.ExternalStream(L.q4_gpu_stream())
        line["single_session_ctx262144"] = extras_single_session(torch, q4gpu, L, ext, peak_gbs)
        line["dense_ctx262144"] = extras_dense(torch, q4gpu, L, ext, peak_gbs)
        line["prefill_8192_over_16384"] = extras_prefill(torch, q4gpu, L, ext, peaks)
        line["indexer_ctx262144"] = extras_indexer(torch, q4gpu, L, ext, peak_gbs)
        line["sparse_prefill_512_ctx262144"] = extras_sparse_prefill(torch, q4gpu, L, ext, peak_gbs)
        line["session_snapshot"] = extras_snapshot(torch, q4gpu, L, ext)
        line["cpu_baseline"] = cpu_baseline(ctxs, args.cpu_seconds)
        for name in ("single_session_ctx262144", "prefill_8192_over_16384", "indexer_ctx262144", "sparse_prefill_512_ctx262144",
                     "session_snapshot"):
            checks[name] = {"verified": line[name].get("verified"), "max_err": line[name].get("max_err")}
        for kname in ("q8_0", "f16", "f32"):
            d = line["dense_ctx262144"].get(kname)
            if d:
                checks["dense_ctx262144/" + kname] = {"verified": d["verified"], "max_err": d["max_err"]}
    line["checks"] = checks
    line["verified"] = all(c["verified"] is True for c in checks.values())
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
