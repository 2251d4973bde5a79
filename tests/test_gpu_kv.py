"""GPU parity of the KV path through the C ABI: quantiser bits, layouts, append variants,
reference-layout export/import, prefix save/restore."""
import numpy as np
import pytest
import torch

import q4gpu
from gpu_util import dev, dev_bytes, host, lib

pytestmark = pytest.mark.gpu


def edge_rows(oracle, n):
    x = oracle.normal(21, 0, n)
    x[:32] = 0.0
    x[32:64] = np.float32(1e-9) * np.arange(32)
    x[64:96] = 0.0
    x[64] = -3.0
    x[96:128] *= np.float32(1e4)
    x[128:160] *= np.float32(1e-5)
    x[160] = 127.5
    x[161] = -127.49999
    return x


@pytest.mark.parametrize("n", [32, 64, 32 * 257, 4096 * 256])
def test_f32_to_q8_bit_exact(oracle, n):
    L = lib()
    x = edge_rows(oracle, max(n, 192))[:n] if n >= 192 else oracle.normal(21, 1, n)
    src = dev(x)
    dst = torch.empty(n // 32 * 34, dtype=torch.uint8, device="cuda")
    assert L.q4_hip_f32_to_q8(dst.data_ptr(), src.data_ptr(), n)
    assert np.array_equal(host(dst), oracle.quant_q8_0(x))


def test_f32_to_q8_rejects_bad_arguments(oracle):
    L = lib()
    src = torch.zeros(64, device="cuda")
    dst = torch.empty(68, dtype=torch.uint8, device="cuda")
    assert not L.q4_hip_f32_to_q8(dst.data_ptr(), src.data_ptr(), 33)
    assert not L.q4_hip_f32_to_q8(None, src.data_ptr(), 32)
    assert not L.q4_hip_f32_to_q8(dst.data_ptr(), src.data_ptr(), 0)
    # unaligned source still quantises correctly
    x = oracle.normal(3, 3, 65)
    s2 = dev(x)
    assert L.q4_hip_f32_to_q8(dst.data_ptr(), s2.data_ptr() + 4, 64)
    assert np.array_equal(host(dst), oracle.quant_q8_0(x[1:]))


def test_f32_to_f16(oracle):
    L = lib()
    x = edge_rows(oracle, 4096)
    dst = torch.empty(4096, dtype=torch.float16, device="cuda")
    assert L.q4_hip_f32_to_f16(dst.data_ptr(), dev(x).data_ptr(), 4096)
    assert np.array_equal(host(dst).view(np.uint16), oracle.f32_to_f16(x))


@pytest.mark.parametrize("kind", [2, 1, 0])
@pytest.mark.parametrize("n_kvh,hd", [(2, 128), (1, 32), (2, 256), (4, 64)])
def test_store_append_export_matches_reference_bytes(oracle, kind, n_kvh, hd):
    """rows appended in ragged chunks, exported in the reference layout == oracle's kv_write bytes"""
    lib()
    n_layers, max_kv, n = 3, 300, 257
    st = q4gpu.KVStore(n_layers, n_kvh, hd, max_kv, kind)
    kvw = n_kvh * hd
    for layer in (0, 2):
        k = edge_rows(oracle, n * kvw).reshape(n, kvw) if layer == 0 else oracle.normal(5, layer, n * kvw).reshape(n, kvw)
        v = oracle.normal(6, layer, n * kvw).reshape(n, kvw)
        pos = 0
        for chunk in (1, 31, 33, 100, 92):
            st.append(layer, dev(k[pos:pos + chunk]), dev(v[pos:pos + chunk]), pos, chunk)
            pos += chunk
        assert pos == n
        tb = st.token_bytes
        for which, rows in ((0, k), (1, v)):
            out = torch.empty(n * tb, dtype=torch.uint8, device="cuda")
            st.export(layer, which, 0, n, out)
            assert np.array_equal(host(out), oracle.kv_write(rows, kind)), (layer, which)
            part = torch.empty(7 * tb, dtype=torch.uint8, device="cuda")
            st.export(layer, which, 250, 7, part)
            assert np.array_equal(host(part), oracle.kv_write(rows[250:257], kind))
    # layer 1 was never touched by the appends to layers 0 and 2
    st.close()


def test_store_import_is_inverse_of_export(oracle):
    lib()
    a = q4gpu.KVStore(2, 2, 128, 64, 2)
    b = q4gpu.KVStore(2, 2, 128, 64, 2)
    k = oracle.normal(8, 0, 50 * 256).reshape(50, 256)
    v = oracle.normal(8, 1, 50 * 256).reshape(50, 256)
    a.append(1, dev(k), dev(v), 3, 50)
    buf = torch.empty(50 * a.token_bytes, dtype=torch.uint8, device="cuda")
    for which in (0, 1):
        a.export(1, which, 3, 50, buf)
        b.import_(1, which, 3, 50, buf)
        back = torch.empty_like(buf)
        b.export(1, which, 3, 50, back)
        assert torch.equal(buf, back)


def test_append_rejects_overflow_and_reports(oracle):
    L = lib()
    st = q4gpu.KVStore(1, 2, 128, 16, 2)
    k = torch.zeros(4, 256, device="cuda")
    assert not L.q4_gpu_kv_append(st.h, 0, k.data_ptr(), k.data_ptr(), 14, 4)
    assert L.q4_gpu_last_error() & 1
    assert not L.q4_gpu_kv_append(st.h, 1, k.data_ptr(), k.data_ptr(), 0, 1)
    L.q4_gpu_last_error()
    # device-position append beyond max_kv: skipped on the device, status bit 4, nothing written
    L.q4_hip_pos_push(16)
    assert L.q4_gpu_kv_append_d(st.h, 0, k.data_ptr(), k.data_ptr())
    assert L.q4_gpu_last_error() & 4


def test_kv_append_d_reference_abi(oracle):
    """q4_hip_kv_append_d on a caller-owned cache in the reference layout, position from the device word."""
    L = lib()
    n_kvh, hd, max_kv = 2, 128, 40
    kvw = n_kvh * hd
    for kind in (2, 1, 0):
        bpt = oracle.kv_token_bytes(n_kvh, hd, kind)
        kc = torch.zeros(max_kv * bpt, dtype=torch.uint8, device="cuda")
        vc = torch.zeros(max_kv * bpt, dtype=torch.uint8, device="cuda")
        want_k = np.zeros(max_kv * bpt, np.uint8)
        want_v = np.zeros(max_kv * bpt, np.uint8)
        for pos in (0, 7, 39):
            k = oracle.normal(30 + kind, pos, kvw)
            v = oracle.normal(40 + kind, pos, kvw)
            L.q4_hip_pos_push(pos)
            assert L.q4_hip_kv_append_d(kc.data_ptr(), vc.data_ptr(), dev(k).data_ptr(), dev(v).data_ptr(), kvw, bpt, kind)
            want_k[pos * bpt:(pos + 1) * bpt] = oracle.kv_write(k, kind)
            want_v[pos * bpt:(pos + 1) * bpt] = oracle.kv_write(v, kind)
        assert np.array_equal(host(kc), want_k) and np.array_equal(host(vc), want_v)


def test_store_append_d_and_graph_replay(oracle):
    """The graph-captured append reads its slot from the position word, so one captured graph
    appends at successive positions (src/q4_fwd.c:891, src/q4_rocm.cu:6216-6223)."""
    L = lib()
    L.q4_gpu_set_stream(None)           # capture runs on the library's own stream
    st = q4gpu.KVStore(1, 2, 128, 32, 2)
    kbuf = torch.zeros(256, device="cuda")
    vbuf = torch.zeros(256, device="cuda")
    torch.cuda.synchronize()
    assert L.q4_hip_graph_begin() == 1
    assert L.q4_hip_capturing() == 1
    assert L.q4_gpu_kv_append_d(st.h, 0, kbuf.data_ptr(), vbuf.data_ptr())
    g = L.q4_hip_graph_end()
    assert g and L.q4_hip_capturing() == 0 and L.q4_hip_graph_nodes(g) >= 1
    rows_k, rows_v = [], []
    for pos in range(5):
        k = oracle.normal(50, pos, 256)
        v = oracle.normal(51, pos, 256)
        rows_k.append(k)
        rows_v.append(v)
        assert L.q4_hip_h2d(kbuf.data_ptr(), k.ctypes.data, 1024)
        assert L.q4_hip_h2d(vbuf.data_ptr(), v.ctypes.data, 1024)
        L.q4_hip_pos_push(pos)
        assert L.q4_hip_graph_launch(g)
    assert L.q4_hip_stream_sync()
    out = torch.empty(5 * st.token_bytes, dtype=torch.uint8, device="cuda")
    st.export(0, 0, 0, 5, out)
    assert L.q4_hip_stream_sync()
    assert np.array_equal(out.cpu().numpy(), oracle.kv_write(np.stack(rows_k), 2))
    st.export(0, 1, 0, 5, out)
    assert L.q4_hip_stream_sync()
    assert np.array_equal(out.cpu().numpy(), oracle.kv_write(np.stack(rows_v), 2))
    L.q4_hip_graph_free(g)
    q4gpu.use_torch_stream()


@pytest.mark.parametrize("n", [77, 199])
@pytest.mark.parametrize("kind", [2, 1, 0])
def test_prefix_save_restore_round_trip(oracle, kind, n):
    """save rows [0,n) -> wipe -> restore == original, to device memory (the library's own copy kernel:
    one partial 32 KB tile per row at 77 rows, several at 199; a buffer that is not 16-byte aligned takes
    the driver's 2-D copy) and to pinned host memory"""
    L = lib()
    n_layers, n_kvh, hd, max_kv = 3, 2, 128, 200
    st = q4gpu.KVStore(n_layers, n_kvh, hd, max_kv, kind)
    kvw = n_kvh * hd
    ref = {}
    for layer in range(n_layers):
        k = oracle.normal(60, layer, n * kvw).reshape(n, kvw)
        v = oracle.normal(61, layer, n * kvw).reshape(n, kvw)
        st.append(layer, dev(k), dev(v), 0, n)
        ref[layer] = (oracle.kv_write(k, kind), oracle.kv_write(v, kind))
    nbytes = st.snapshot_bytes(n)
    assert nbytes == n * n_layers * 2 * st.token_bytes       # same byte count as the reference snapshot
    for host_side, skew in ((False, 0), (False, 8), (True, 0)):
        snap = torch.empty(nbytes, dtype=torch.uint8, device="cpu", pin_memory=True) if host_side else \
            torch.empty(nbytes + 16, dtype=torch.uint8, device="cuda")[skew:skew + nbytes]
        st.save(n, snap, host=host_side)
        torch.cuda.synchronize()
        other = q4gpu.KVStore(n_layers, n_kvh, hd, max_kv, kind)
        other.restore(n, snap, host=host_side)
        for layer in range(n_layers):
            for which in (0, 1):
                out = torch.empty(n * st.token_bytes, dtype=torch.uint8, device="cuda")
                other.export(layer, which, 0, n, out)
                assert np.array_equal(host(out), ref[layer][which]), (host_side, layer, which)
        other.close()
    assert not L.q4_gpu_kv_save(st.h, max_kv + 1, snap.data_ptr(), 0)
    L.q4_gpu_last_error()


def test_prep_kernels(oracle):
    L = lib()
    n_head, n_kvh, hd, n_rot, base, eps, n_tok, pos0 = 16, 2, 128, 64, 1e7, 1e-6, 5, 1000
    qg = oracle.normal(70, 0, n_tok * n_head * 2 * hd)
    kk = oracle.normal(70, 1, n_tok * n_kvh * hd)
    wq = (1 + 0.1 * oracle.normal(70, 2, hd)).astype(np.float32)
    wk = (1 + 0.1 * oracle.normal(70, 3, hd)).astype(np.float32)
    q_ref, g_ref = oracle.q_prep(qg, wq, n_head, hd, n_rot, pos0, base, eps)
    k_ref = oracle.k_prep(kk, wk, n_kvh, hd, n_rot, pos0, base, eps)
    dq = torch.empty(n_tok * n_head * hd, device="cuda")
    dg = torch.empty_like(dq)
    dk = dev(kk)
    assert L.q4_hip_qsa_q_prep_n(dev(qg).data_ptr(), dev(wq).data_ptr(), dq.data_ptr(), dg.data_ptr(), n_head, hd,
                                 n_rot, pos0, base, eps, n_tok)
    assert L.q4_hip_qsa_k_prep_n(dk.data_ptr(), dev(wk).data_ptr(), n_kvh, hd, n_rot, pos0, base, eps, n_tok)
    # libm of the device and of the host differ in the last bits of powf/sinf/cosf at angle ~1e3
    assert np.array_equal(host(dg), g_ref.reshape(-1))
    assert np.abs(host(dq) - q_ref.reshape(-1)).max() < 2e-3
    assert np.abs(host(dk) - k_ref.reshape(-1)).max() < 2e-3
    # untouched tail (partial rotary) is exact up to the norm's rounding
    assert np.allclose(host(dq).reshape(n_tok, n_head, hd)[:, :, n_rot:], q_ref[:, :, n_rot:], rtol=2e-6, atol=1e-7)
    # device-position variants agree with the explicit-position ones
    L.q4_hip_pos_push(pos0)
    dq2 = torch.empty(n_head * hd, device="cuda")
    dg2 = torch.empty_like(dq2)
    assert L.q4_hip_qsa_q_prep_d(dev(qg).data_ptr(), dev(wq).data_ptr(), dq2.data_ptr(), dg2.data_ptr(), n_head, hd,
                                 n_rot, base, eps)
    assert np.array_equal(host(dq2), host(dq)[:n_head * hd])
    dk2 = dev(kk[:n_kvh * hd])
    assert L.q4_hip_qsa_k_prep_d(dk2.data_ptr(), dev(wk).data_ptr(), n_kvh, hd, n_rot, base, eps)
    assert np.array_equal(host(dk2), host(dk)[:n_kvh * hd])


@pytest.mark.parametrize("kind", [2, 1])
def test_session_file_kv_section(oracle, kind, tmp_path):
    """q4_gpu_kv_write_fd writes exactly the KV section of the reference's session file: per layer the
    K rows then the V rows in the reference layout (src/q4_fwd.c:2353-2360); read_fd restores it; a
    truncated file is refused."""
    import os
    L = lib()
    n_layers, n_kvh, hd, max_kv, n = 3, 2, 128, 400, 333
    kvw = n_kvh * hd
    st = q4gpu.KVStore(n_layers, n_kvh, hd, max_kv, kind)
    want = b""
    for layer in range(n_layers):
        k = oracle.normal(90, layer, n * kvw).reshape(n, kvw)
        v = oracle.normal(91, layer, n * kvw).reshape(n, kvw)
        st.append(layer, dev(k), dev(v), 0, n)
        want += oracle.kv_write(k, kind).tobytes() + oracle.kv_write(v, kind).tobytes()
    path = str(tmp_path / "kv.bin")
    fd = os.open(path, os.O_CREAT | os.O_WRONLY | os.O_TRUNC, 0o600)
    os.write(fd, b"HDR!")                      # the caller positions the descriptor (header, ids, ...)
    st.write_fd(n, fd)
    os.close(fd)
    data = open(path, "rb").read()
    assert data[:4] == b"HDR!" and data[4:] == want
    other = q4gpu.KVStore(n_layers, n_kvh, hd, max_kv, kind)
    fd = os.open(path, os.O_RDONLY)
    os.lseek(fd, 4, os.SEEK_SET)
    other.read_fd(n, fd)
    os.close(fd)
    tb = st.token_bytes
    for layer in range(n_layers):
        for which in (0, 1):
            a = torch.empty(n * tb, dtype=torch.uint8, device="cuda")
            b = torch.empty_like(a)
            st.export(layer, which, 0, n, a)
            other.export(layer, which, 0, n, b)
            assert torch.equal(a, b)
    with open(path, "r+b") as f:
        f.truncate(len(data) - 100)
    fd = os.open(path, os.O_RDONLY)
    os.lseek(fd, 4, os.SEEK_SET)
    assert not L.q4_gpu_kv_read_fd(other.h, n, fd)
    os.close(fd)
    L.q4_gpu_last_error()
    st.close()
    other.close()


@pytest.mark.parametrize("kind,hd,n_rot", [(2, 128, 128), (2, 256, 64), (1, 128, 64), (0, 64, 64)])
def test_fused_prep_append_equals_two_launches(oracle, kind, hd, n_rot):
    """RMSNorm + RoPE + quantise + scatter in one launch == q4_hip_qsa_k_prep_n followed by the append,
    byte for byte; and within the documented libm tolerance of the oracle's prep before quantisation."""
    L = lib()
    n_kvh, n_tok, pos0, base, eps = 2, 37, 1000, 1e7, 1e-6
    kvw = n_kvh * hd
    k = oracle.normal(95, hd, n_tok * kvw)
    v = oracle.normal(96, hd, n_tok * kvw)
    w = (1 + 0.1 * oracle.normal(97, hd, hd)).astype(np.float32)
    a = q4gpu.KVStore(1, n_kvh, hd, 1100, kind)
    b = q4gpu.KVStore(1, n_kvh, hd, 1100, kind)
    dk, dv, dw = dev(k), dev(v), dev(w)
    assert L.q4_gpu_kv_prep_append(a.h, 0, dk.data_ptr(), dv.data_ptr(), dw.data_ptr(), n_rot, base, eps, pos0, n_tok)
    assert np.array_equal(host(dk), k)                      # the raw rows are left alone
    dk2 = dev(k)
    assert L.q4_hip_qsa_k_prep_n(dk2.data_ptr(), dw.data_ptr(), n_kvh, hd, n_rot, pos0, base, eps, n_tok)
    b.append(0, dk2, dv, pos0, n_tok)
    tb = a.token_bytes
    for which in (0, 1):
        xa = torch.empty(n_tok * tb, dtype=torch.uint8, device="cuda")
        xb = torch.empty_like(xa)
        a.export(0, which, pos0, n_tok, xa)
        b.export(0, which, pos0, n_tok, xb)
        assert torch.equal(xa, xb), which
    # device-position variant writes the same bytes at the position word
    c = q4gpu.KVStore(1, n_kvh, hd, 1100, kind)
    L.q4_hip_pos_push(pos0 + 5)
    assert L.q4_gpu_kv_prep_append_d(c.h, 0, dk.data_ptr() + 5 * kvw * 4, dv.data_ptr() + 5 * kvw * 4, dw.data_ptr(),
                                     n_rot, base, eps)
    for which in (0, 1):
        xa = torch.empty(tb, dtype=torch.uint8, device="cuda")
        xc = torch.empty_like(xa)
        a.export(0, which, pos0 + 5, 1, xa)
        c.export(0, which, pos0 + 5, 1, xc)
        assert torch.equal(xa, xc)
    for s in (a, b, c):
        s.close()
