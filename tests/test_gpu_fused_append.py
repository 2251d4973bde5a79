"""Append fused into the attention launch (q4_gpu_batch_append_decode, q4_gpu_kv_append_decode_d):
the rows it stores are bit-identical to the append kernel's and to the oracle's q8_0 bytes, and the
attention output equals append-then-decode, for sparse lists that do and do not contain the newest
position, dense ranges, several splits per unit, and other kinds / head dims (two launches inside)."""
import numpy as np
import pytest
import torch

import q4gpu
from gpu_util import assert_close, dev, host, lib

pytestmark = pytest.mark.gpu


def ref_bytes(store, layer, which, tok0, n):
    rb = {2: store.hd // 32 * 34, 1: store.hd * 2, 0: store.hd * 4}[store.kind]
    buf = torch.empty(n * store.n_kvh * rb, dtype=torch.uint8, device="cuda")
    store.export(layer, which, tok0, n, buf)
    return host(buf)


@pytest.mark.parametrize("kind,hd,lens,width", [(2, 128, [1, 17, 300, 2051, 5000, 33, 4096, 2], 64),
                                                (2, 128, [9000, 12000], 2051),
                                                (2, 64, [40, 700, 3], 32), (1, 128, [40, 700, 3], 32),
                                                (0, 128, [5, 200], 16)])
def test_batch_fused_equals_append_then_decode(oracle, kind, hd, lens, width):
    lib()
    n_head, n_kvh, n_layers = 16, 2, 2
    kvw = n_kvh * hd
    max_kv = max(lens) + 8
    pairs = []
    for s, n in enumerate(lens):
        k = oracle.normal(900 + s, 0, n * kvw).reshape(n, kvw)
        v = oracle.normal(900 + s, 1, n * kvw).reshape(n, kvw)
        two = []
        for _ in range(2):
            st = q4gpu.KVStore(n_layers, n_kvh, hd, max_kv, kind)
            if n > 1:
                for layer in range(n_layers):
                    st.append(layer, dev(k[:-1]), dev(v[:-1]), 0, n - 1)
            two.append(st)
        pairs.append((k, v, two))
    ba, bb = q4gpu.Batch([p[2][0] for p in pairs]), q4gpu.Batch([p[2][1] for p in pairs])
    pos = [n - 1 for n in lens]
    ba.set_pos(pos)
    bb.set_pos(pos)
    last_k = dev(np.stack([p[0][-1] for p in pairs]))
    last_v = dev(np.stack([p[1][-1] for p in pairs]))
    q = dev(oracle.normal(901, 0, len(lens) * n_head * hd).reshape(len(lens), n_head, hd))
    gate = dev(oracle.normal(901, 1, len(lens) * n_head * hd).reshape(len(lens), n_head, hd))
    idx = np.full((len(lens), n_kvh, width), -1, np.int32)
    for s, n in enumerate(lens):
        for kh in range(n_kvh):
            sink = 4 if width == 2051 else 2
            recent = (width - sink + 1) // 2
            sel = oracle.select(950 + s, kh, n, width, sink=sink, recent=recent, nrand=width - sink - recent)
            if (s + kh) % 2 and n > 1:
                sel = np.where(sel == n - 1, 0, sel)       # a list without the newest position
            idx[s, kh] = sel
    didx = dev(idx)
    out_a, out_b = torch.zeros(len(lens) * n_head * hd, device="cuda"), torch.zeros(len(lens) * n_head * hd, device="cuda")
    # sparse
    ba.append(1, last_k, last_v)
    ba.decode(1, q, out_a, n_head, 0.0884, gate=gate, idx=didx, width=width, idx_kvh_stride=width, idx_sess_stride=n_kvh * width)
    bb.append_decode(1, last_k, last_v, q, out_b, n_head, 0.0884, gate=gate, idx=didx, width=width, idx_kvh_stride=width,
                     idx_sess_stride=n_kvh * width)
    assert_close(host(out_b), host(out_a), "sparse fused vs two launches")
    for s, n in enumerate(lens):
        for which in (0, 1):
            a = ref_bytes(pairs[s][2][0], 1, which, n - 1, 1)
            b = ref_bytes(pairs[s][2][1], 1, which, n - 1, 1)
            assert np.array_equal(a, b), "stored row differs (session %d plane %d)" % (s, which)
            want = oracle.kv_write(pairs[s][which][-1:], kind).reshape(-1)
            assert np.array_equal(b, want), "stored row differs from the oracle (session %d plane %d)" % (s, which)
    # dense, on the other layer
    ba.append(0, last_k, last_v)
    ba.decode(0, q, out_a, n_head, 0.0884)
    bb.append_decode(0, last_k, last_v, q, out_b, n_head, 0.0884)
    assert_close(host(out_b), host(out_a), "dense fused vs two launches")
    assert q4gpu.load().q4_gpu_last_error() == 0
    ba.close()
    bb.close()
    for p in pairs:
        for st in p[2]:
            st.close()


def test_single_session_fused_at_the_position_word(oracle):
    """q4_gpu_kv_append_decode_d for successive tokens == q4_gpu_kv_append_d + q4_gpu_kv_decode; rows bit-equal;
    also against the oracle over the whole prefix."""
    L = lib()
    n_head, n_kvh, hd, max_kv, steps = 16, 2, 128, 96, 70
    kvw = n_kvh * hd
    k = oracle.normal(960, 0, steps * kvw).reshape(steps, kvw)
    v = oracle.normal(960, 1, steps * kvw).reshape(steps, kvw)
    q = oracle.normal(960, 2, steps * n_head * hd).reshape(steps, n_head, hd)
    a, b = q4gpu.KVStore(1, n_kvh, hd, max_kv, 2), q4gpu.KVStore(1, n_kvh, hd, max_kv, 2)
    oa, ob = torch.zeros(n_head * hd, device="cuda"), torch.zeros(n_head * hd, device="cuda")
    for t in range(steps):
        L.q4_hip_pos_push(t)
        dk, dv, dq = dev(k[t]), dev(v[t]), dev(q[t])
        a.append_d(0, dk, dv)
        a.decode(0, dq, oa, n_head, 0.0884)
        b.append_decode_d(0, dk, dv, dq, ob, n_head, 0.0884)
        assert_close(host(ob), host(oa), "token %d" % t)
    kc, vc = oracle.kv_write(k, 2), oracle.kv_write(v, 2)
    ref = oracle.attn(q[-1], kc, vc, None, n_head, n_kvh, hd, 1, steps - 1, steps, 0.0884, 2)[0]
    assert_close(host(ob).reshape(n_head, hd), ref, "last token vs oracle")
    for which in (0, 1):
        assert np.array_equal(ref_bytes(a, 0, which, 0, steps), ref_bytes(b, 0, which, 0, steps))
    assert L.q4_gpu_last_error() == 0
    a.close()
    b.close()


def test_position_beyond_the_store_is_reported():
    L = lib()
    st = q4gpu.KVStore(1, 2, 128, 16, 2)
    b = q4gpu.Batch([st])
    b.set_pos([16])
    z = torch.zeros(256, device="cuda")
    qq, out = torch.zeros(16 * 128, device="cuda"), torch.zeros(16 * 128, device="cuda")
    b.append_decode(0, z, z, qq, out, 16, 0.1)
    torch.cuda.synchronize()
    assert L.q4_gpu_last_error() & 4
    b.close()
    st.close()
