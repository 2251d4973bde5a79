"""The small entry points of the reference ABI that the attention path leans on, through the C ABI:
q4_hip_fill / q4_hip_copy (session reset and the fp32 append, src/q4_rocm.cu:5656-5670),
q4_hip_f32_to_f16_d (fp16 append at the device position word, :7943-7958), the asynchronous copies
(:8417-8432), the device-position append for rows of any length (:7962-8012), shutdown followed by
a new init, and the behaviours the store entry points promise about sizes and bounds."""
import ctypes

import numpy as np
import pytest
import torch

import q4gpu
from gpu_util import assert_close, dev, host, lib

pytestmark = pytest.mark.gpu


def test_fill_and_copy():
    L = lib()
    n = 100003
    a = torch.empty(n, device="cuda")
    b = torch.empty(n, device="cuda")
    assert L.q4_hip_fill(a.data_ptr(), 2.5, n)
    assert L.q4_hip_copy(b.data_ptr(), a.data_ptr(), n)
    assert torch.equal(b, torch.full((n,), 2.5, device="cuda"))
    assert L.q4_hip_fill(a.data_ptr(), 0.0, n)
    assert not a.any()
    assert L.q4_hip_fill(a.data_ptr() + 4, -1.0, 5)            # a sub-range, not 16-byte aligned
    assert host(a)[:8].tolist() == [0.0, -1.0, -1.0, -1.0, -1.0, -1.0, 0.0, 0.0]
    # rejected like the reference: NULL or zero size
    assert not L.q4_hip_fill(None, 1.0, 4) and not L.q4_hip_fill(a.data_ptr(), 1.0, 0)
    assert not L.q4_hip_copy(b.data_ptr(), None, 4) and not L.q4_hip_copy(b.data_ptr(), a.data_ptr(), 0)


def test_f32_to_f16_at_the_device_position(oracle):
    L = lib()
    stride, rows, n = 96, 7, 80
    x = oracle.normal(5, 0, n)
    base = torch.zeros(rows * stride, dtype=torch.float16, device="cuda")
    for pos in (0, 3, 6):
        L.q4_hip_pos_push(pos)
        assert L.q4_hip_f32_to_f16_d(base.data_ptr(), stride, dev(x).data_ptr(), n)
    got = host(base).view(np.uint16).reshape(rows, stride)
    want = oracle.f32_to_f16(x)
    for r in range(rows):
        if r in (0, 3, 6):
            assert np.array_equal(got[r, :n], want) and not got[r, n:].any()
        else:
            assert not got[r].any()
    assert not L.q4_hip_f32_to_f16_d(None, stride, dev(x).data_ptr(), n)


def test_async_copies_are_stream_ordered():
    L = lib()
    n = 1 << 16
    h_in = torch.arange(n, dtype=torch.float32).pin_memory()
    h_out = torch.zeros(n, dtype=torch.float32).pin_memory()
    d = torch.zeros(n, device="cuda")
    d2 = torch.zeros(n, device="cuda")
    assert L.q4_hip_h2d_async(d.data_ptr(), h_in.data_ptr(), 4 * n)
    assert L.q4_hip_copy(d2.data_ptr(), d.data_ptr(), n)        # ordered after the upload
    assert L.q4_hip_d2h_async(h_out.data_ptr(), d2.data_ptr(), 4 * n)
    assert L.q4_hip_stream_sync()
    assert torch.equal(h_out, h_in)
    # the blocking forms and the copy stream
    d.zero_()
    torch.cuda.synchronize()
    assert L.q4_hip_h2d(d.data_ptr(), h_in.data_ptr(), 4 * n)
    assert torch.equal(d.cpu(), h_in)
    d.zero_()
    torch.cuda.synchronize()
    assert L.q4_hip_copy_h2d(d.data_ptr(), h_in.data_ptr(), 4 * n)
    L.q4_hip_copy_wait()
    assert torch.equal(d.cpu(), h_in)
    assert not L.q4_hip_h2d_async(None, h_in.data_ptr(), 4) and not L.q4_hip_d2h_async(h_out.data_ptr(), d.data_ptr(), 0)


@pytest.mark.parametrize("kind,n", [(0, 40), (1, 40), (0, 100), (1, 36), (1, 256), (0, 256)])
def test_device_position_append_rows_of_any_length(oracle, kind, n):
    """q4_hip_kv_append_d on fp32 / fp16 caches takes rows of any length (the reference needs a multiple
    of 32 only for q8_0), from sources of any 4-byte alignment"""
    L = lib()
    es = 4 if kind == 0 else 2
    bpt, rows = n * es, 5
    k, v = oracle.normal(60, n, n + 1), oracle.normal(61, n, n + 1)
    dk, dv = dev(k), dev(v)
    kc = torch.zeros(rows * bpt, dtype=torch.uint8, device="cuda")
    vc = torch.zeros(rows * bpt, dtype=torch.uint8, device="cuda")
    L.q4_hip_pos_push(2)
    off = 4                                                     # sources one float off a 16-byte boundary
    assert L.q4_hip_kv_append_d(kc.data_ptr(), vc.data_ptr(), dk.data_ptr() + off, dv.data_ptr() + off, n, bpt, kind)
    for cache, src in ((kc, k[1:]), (vc, v[1:])):
        got = host(cache).reshape(rows, bpt)
        want = oracle.kv_write(src, kind)
        assert np.array_equal(got[2], want)
        assert not got[[0, 1, 3, 4]].any()
    # q8_0 still wants whole blocks
    assert not L.q4_hip_kv_append_d(kc.data_ptr(), vc.data_ptr(), dk.data_ptr(), dv.data_ptr(), 40, 40 // 32 * 34, 2)


def test_shutdown_then_init_again(oracle):
    """q4_hip_shutdown releases the library's own state; a new q4_hip_init brings it back and the path
    computes the same bytes as before"""
    L = lib()
    x = oracle.normal(77, 0, 4096)
    dx = dev(x)
    out1 = torch.empty(4096 // 32 * 34, dtype=torch.uint8, device="cuda")
    assert L.q4_hip_f32_to_q8(out1.data_ptr(), dx.data_ptr(), 4096)
    torch.cuda.synchronize()
    L.q4_gpu_set_stream(None)
    L.q4_hip_shutdown()
    assert not L.q4_hip_ok()
    assert not L.q4_hip_f32_to_q8(out1.data_ptr(), dx.data_ptr(), 4096)      # nothing works without init
    assert not L.q4_gpu_kv_create(1, 2, 128, 16, 2)
    assert L.q4_gpu_last_error() & 16                                         # "not initialised" is reported, and cleared by reading
    L = lib()                                                                 # q4_hip_init again
    assert L.q4_hip_ok()
    out2 = torch.empty_like(out1)
    assert L.q4_hip_f32_to_q8(out2.data_ptr(), dx.data_ptr(), 4096)
    assert torch.equal(out1, out2) and np.array_equal(host(out2), oracle.quant_q8_0(x))
    st = q4gpu.KVStore(1, 2, 128, 64, 2)                                     # scratch, position word, status word: all new
    k = oracle.normal(78, 0, 64 * 256).reshape(64, 256)
    st.append(0, dev(k), dev(k), 0, 64)
    q = oracle.normal(78, 1, 16 * 128)
    out = torch.empty(16 * 128, device="cuda")
    st.decode(0, dev(q), out, 16, 0.0884, n_kv=64)
    kc = oracle.kv_write(k, 2)
    assert_close(host(out).reshape(16, 128), oracle.attn(q, kc, kc, None, 16, 2, 128, 1, 63, 64, 0.0884, 2)[0], "after re-init")
    assert L.q4_gpu_last_error() == 0
    st.close()


@pytest.mark.parametrize("hd", [32, 64, 128, 256])
@pytest.mark.parametrize("kind", [0, 1, 2])
def test_kv_bytes_is_what_the_store_allocates(hd, kind):
    L = lib()
    n_layers, n_kvh, max_kv = 3, 2, 100
    st = q4gpu.KVStore(n_layers, n_kvh, hd, max_kv, kind)
    assert st.bytes() == st.snapshot_bytes(max_kv)              # a snapshot of every row is the whole allocation
    ref_total = n_layers * max_kv * 2 * (n_kvh * hd // 32 * 34 if kind == 2 else n_kvh * hd * (2 if kind == 1 else 4))
    if kind != 2 or hd >= 128:
        assert st.bytes() == ref_total                          # the reference's q4_qsa_kv_bytes
    else:
        assert st.bytes() == n_layers * max_kv * n_kvh * {32: 80, 64: 144}[hd] > ref_total
    st.close()


def test_batch_launches_cover_the_sessions_of_the_last_set_pos(oracle):
    """four bound slots, positions published for two: the launch reads and writes two rows of every array"""
    lib()
    n_head, n_kvh, hd, ctx = 16, 2, 128, 40
    kvw = n_kvh * hd
    stores, ks = [], []
    for s in range(4):
        k = oracle.normal(300 + s, 0, (ctx + 1) * kvw).reshape(ctx + 1, kvw)
        st = q4gpu.KVStore(1, n_kvh, hd, ctx + 1, 2)
        st.append(0, dev(k[:ctx]), dev(k[:ctx]), 0, ctx)
        stores.append(st)
        ks.append(k)
    b = q4gpu.Batch(stores)
    b.set_pos([ctx, ctx])
    q = oracle.normal(310, 0, 2 * n_head * hd).reshape(2, n_head * hd)
    out = torch.full((4, n_head * hd), 7.0, device="cuda")      # rows 2, 3 must stay untouched
    newk = np.stack([ks[0][ctx], ks[1][ctx]])
    b.append_decode(0, dev(newk), dev(newk), dev(q), out, n_head, 0.0884)
    got = host(out)
    for s in range(2):
        kc = oracle.kv_write(ks[s], 2)
        assert_close(got[s].reshape(n_head, hd), oracle.attn(q[s], kc, kc, None, n_head, n_kvh, hd, 1, ctx, ctx + 1, 0.0884, 2)[0],
                     "session %d" % s)
    assert (got[2:] == 7.0).all()
    # sessions 2 and 3 were not appended to: their slot ctx still holds what the allocation held, and a
    # decode over their first ctx rows is unaffected
    for s in (2, 3):
        o = torch.empty(n_head * hd, device="cuda")
        stores[s].decode(0, dev(q[0]), o, n_head, 0.0884, n_kv=ctx)
        kc = oracle.kv_write(ks[s][:ctx], 2)
        assert_close(host(o).reshape(n_head, hd), oracle.attn(q[0], kc, kc, None, n_head, n_kvh, hd, 1, ctx - 1, ctx, 0.0884, 2)[0],
                     "untouched session %d" % s)
    assert q4gpu.load().q4_gpu_last_error() == 0
    b.close()
    for st in stores:
        st.close()


def test_list_entries_beyond_the_rows_written_are_reported(oracle):
    """a store is not cleared when it is created: an entry >= n_kv is skipped and raises status bit 4"""
    L = lib()
    n_head, n_kvh, hd, ctx, max_kv = 16, 2, 128, 50, 200
    k = oracle.normal(320, 0, ctx * 256).reshape(ctx, 256)
    st = q4gpu.KVStore(1, n_kvh, hd, max_kv, 2)
    st.append(0, dev(k), dev(k), 0, ctx)
    q = oracle.normal(321, 0, n_head * hd)
    idx = np.array([0, 3, 49, 50, 120, -1, 7, 199], np.int32)  # 50, 120, 199: inside the allocation, never written
    out = torch.empty(n_head * hd, device="cuda")
    assert L.q4_gpu_last_error() == 0
    st.decode(0, dev(q), out, n_head, 0.0884, idx=dev(idx), width=len(idx), idx_kvh_stride=0, n_kv=ctx)
    assert L.q4_gpu_last_error() == 4
    kc = oracle.kv_write(k, 2)
    good = np.where(idx < ctx, idx, -1).astype(np.int32)
    ref = oracle.attn(q, kc, kc, None, n_head, n_kvh, hd, 1, 0, ctx, 0.0884, 2, idx=good, width=len(idx))[0]
    assert_close(host(out).reshape(n_head, hd), ref, "entries beyond n_kv skipped")
    st.close()


def test_graph_capture_on_the_legacy_default_stream_is_refused_with_a_reason():
    L = lib()
    assert L.q4_gpu_set_stream(ctypes.c_void_p(1))              # cudaStreamLegacy
    assert L.q4_gpu_last_error() == 0
    assert L.q4_hip_graph_begin() == 0
    assert L.q4_gpu_last_error() & 1
    assert L.q4_gpu_set_stream(None)
    assert L.q4_hip_graph_begin() == 1
    assert L.q4_hip_capturing() == 1
    g = L.q4_hip_graph_end()
    if g:
        L.q4_hip_graph_free(g)
    q4gpu.use_torch_stream()


def test_pipelined_steps_over_two_buffer_sets():
    """q4_gpu_pipe_*: upload on the copy stream, a captured graph on the compute stream, download on the download
    stream, ordered by the pipe's events alone; two sets of buffers alternate, every step's result must be that
    step's input (the graph copies input to output on the device)"""
    L = lib()
    assert L.q4_gpu_set_stream(None)
    n = 1 << 18
    sets = []
    for _ in range(2):
        in_h = torch.empty(n, dtype=torch.float32).pin_memory()
        out_h = torch.zeros(n, dtype=torch.float32).pin_memory()
        in_d = torch.zeros(n, device="cuda")
        out_d = torch.zeros(n, device="cuda")
        torch.cuda.synchronize()
        assert L.q4_hip_graph_begin() == 1
        assert L.q4_hip_copy(out_d.data_ptr(), in_d.data_ptr(), n)
        g = L.q4_hip_graph_end()
        assert g
        pipe = L.q4_gpu_pipe_create()
        assert pipe
        sets.append((in_h, out_h, in_d, out_d, g, pipe))
    steps = 9
    expect = [None, None]
    def upload(i):
        in_h, _, in_d, _, _, pipe = sets[i % 2]
        if expect[i % 2] is not None:                     # the set's previous result must be read before its input is reused
            assert L.q4_gpu_pipe_sync(pipe)
            assert (sets[i % 2][1] == expect[i % 2]).all(), "step %d" % (i - 2)
        in_h.fill_(float(i + 1))
        in_h[i] = -3.0
        expect[i % 2] = in_h.clone()
        assert L.q4_gpu_pipe_upload(pipe, in_d.data_ptr(), in_h.data_ptr(), 4 * n)
    upload(0)
    for i in range(steps):
        if i + 1 < steps:
            upload(i + 1)
        _, out_h, _, out_d, g, pipe = sets[i % 2]
        assert L.q4_gpu_pipe_run(pipe, g, out_h.data_ptr(), out_d.data_ptr(), 4 * n)
    for k in range(2):
        assert L.q4_gpu_pipe_sync(sets[k][5])
        assert (sets[k][1] == expect[k]).all()
    assert L.q4_gpu_last_error() == 0
    for in_h, out_h, in_d, out_d, g, pipe in sets:
        L.q4_hip_graph_free(g)
        L.q4_gpu_pipe_destroy(pipe)
    q4gpu.use_torch_stream()
