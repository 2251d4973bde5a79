"""The configurations of the benchmark at their full sizes, checked through properties that do not need
the CPU oracle to chew through them: the tensor-core prefill of 8192 queries over 24 576 rows against
the decode kernel on sampled queries and against itself in two chunks; appends in one call against
appends in ragged chunks (bytes) with a sampled comparison to the oracle; dense attention over 262 144
rows against the merge of its 8 position shards; a 12-layer prefix snapshot round trip."""
import numpy as np
import pytest
import torch

import q4gpu
from gpu_util import assert_close, dev, host, lib
from test_gpu_prefill import check

pytestmark = pytest.mark.gpu

N_HEAD, N_KVH, HD = 16, 2, 128
KVW = N_KVH * HD
SCALE = 1.0 / np.sqrt(HD)


def export_bytes(store, layer, which, tok0, n):
    buf = torch.empty(n * N_KVH * (HD // 32 * 34), dtype=torch.uint8, device="cuda")
    store.export(layer, which, tok0, n, buf)
    return buf


def test_chunked_prefill_full_size_properties(oracle):
    lib()
    base, n_tok = 16384, 8192
    torch.manual_seed(3)
    k = torch.randn(base + n_tok, KVW, device="cuda")
    v = torch.randn(base + n_tok, KVW, device="cuda")
    q = torch.randn(n_tok, N_HEAD, HD, device="cuda").to(torch.bfloat16)
    gate = torch.randn(n_tok, N_HEAD, HD, device="cuda")
    # the same rows appended in one call and in ragged chunks: identical bytes
    a = q4gpu.KVStore(1, N_KVH, HD, base + n_tok, 2)
    b = q4gpu.KVStore(1, N_KVH, HD, base + n_tok, 2)
    a.append(0, k, v, 0, base + n_tok)
    p = 0
    for step in (1, 999, 4097, 7, 16384, 1 << 30):
        n = min(step, base + n_tok - p)
        if n:
            b.append(0, k[p:p + n].contiguous(), v[p:p + n].contiguous(), p, n)
        p += n
    for which in (0, 1):
        assert torch.equal(export_bytes(a, 0, which, 0, base + n_tok), export_bytes(b, 0, which, 0, base + n_tok))
    # sampled rows against the oracle's q8_0 bytes
    rows = [0, 1, 4095, 16383, 16384, 20000, base + n_tok - 1]
    for which, src in ((0, k), (1, v)):
        got = host(export_bytes(a, 0, which, 0, base + n_tok)).reshape(base + n_tok, -1)
        want = oracle.kv_write(host(src[rows]), 2).reshape(len(rows), -1)
        assert np.array_equal(got[rows], want)
    out = torch.empty(n_tok, N_HEAD, HD, dtype=torch.bfloat16, device="cuda")
    a.prefill(0, q, out, N_HEAD, n_tok, base, SCALE, gate=gate)
    # (1) sampled queries == the decode kernel over the same prefix
    dd = torch.empty(N_HEAD * HD, device="cuda")
    for t in (0, 1, 15, 16, 4095, 4096, 8000, n_tok - 1):
        a.decode(0, q[t].contiguous(), dd, N_HEAD, SCALE, gate=gate[t].contiguous(), n_kv=base + t + 1, q_bf16=True)
        check(host(out[t].float()), host(dd).reshape(N_HEAD, HD), "token %d vs decode" % t)
    # (2) the chunk split in two == the chunk in one call
    out2 = torch.empty_like(out)
    half = 4096 + 16 * 3
    a.prefill(0, q[:half].contiguous(), out2[:half], N_HEAD, half, base, SCALE, gate=gate[:half].contiguous())
    a.prefill(0, q[half:].contiguous(), out2[half:], N_HEAD, n_tok - half, base + half, SCALE, gate=gate[half:].contiguous())
    d = (out.float() - out2.float()).abs()
    assert float(d.max()) <= 2e-3 + 2.0 ** -7 * float(out.float().abs().max())
    assert torch.isfinite(out.float()).all()
    assert q4gpu.load().q4_gpu_last_error() == 0
    a.close()
    b.close()


@pytest.mark.parametrize("kind", [2, 1])
def test_dense_262144_equals_merge_of_its_shards(oracle, kind):
    """configs[4]: attention over the whole 262 144-row context == merge of the records of its 8 position
    shards (each shard a store of its own, as on 8 GPUs), for bf16 queries with a gate"""
    L = lib()
    ctx, G = 262144, 8
    torch.manual_seed(4)
    full = q4gpu.KVStore(1, N_KVH, HD, ctx, kind)
    shards = [q4gpu.KVStore(1, N_KVH, HD, ctx // G, kind) for _ in range(G)]
    per = ctx // G
    for r in range(G):
        k = torch.randn(per, KVW, device="cuda")
        v = torch.randn(per, KVW, device="cuda")
        full.append(0, k, v, r * per, per)
        shards[r].append(0, k, v, 0, per)
    q = torch.randn(N_HEAD, HD, device="cuda").to(torch.bfloat16)
    gate = torch.randn(N_HEAD, HD, device="cuda")
    out = torch.empty(N_HEAD * HD, device="cuda")
    full.decode(0, q, out, N_HEAD, SCALE, gate=gate, n_kv=ctx, q_bf16=True)
    parts = torch.empty(G, N_HEAD, HD + 2, device="cuda")
    for r in range(G):
        shards[r].decode_partial(0, q, parts[r], N_HEAD, SCALE, n_kv=per, q_bf16=True)
    merged = torch.empty(N_HEAD * HD, device="cuda")
    assert L.q4_gpu_lse_merge(parts.data_ptr(), G, N_HEAD, HD, gate.data_ptr(), merged.data_ptr())
    assert_close(host(merged), host(out), "merge of shards vs whole, kind %d" % kind)
    assert float(out.abs().max()) > 0
    assert L.q4_gpu_last_error() == 0
    for s in shards + [full]:
        s.close()


def test_prefix_snapshot_round_trip_12_layers(oracle):
    """a 12-layer, 65 536-row prefix: save to a device pool, wipe, restore: exported rows identical"""
    lib()
    n_layers, n_kv = 12, 65536
    torch.manual_seed(5)
    st = q4gpu.KVStore(n_layers, N_KVH, HD, n_kv + 64, 2)
    k = torch.randn(n_kv, KVW, device="cuda")
    v = torch.randn(n_kv, KVW, device="cuda")
    for layer in range(n_layers):
        st.append(layer, k.roll(layer, 0), v.roll(-layer, 0), 0, n_kv)
    before = [export_bytes(st, layer, which, 0, n_kv).clone() for layer in (0, 5, 11) for which in (0, 1)]
    nbytes = st.snapshot_bytes(n_kv)
    assert nbytes == n_layers * n_kv * 2 * N_KVH * (HD // 32 * 34)      # the reference's byte count
    pool = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    st.save(n_kv, pool)
    z = torch.zeros(n_kv, KVW, device="cuda")
    for layer in range(n_layers):
        st.append(layer, z, z, 0, n_kv)
    st.restore(n_kv, pool)
    after = [export_bytes(st, layer, which, 0, n_kv) for layer in (0, 5, 11) for which in (0, 1)]
    for x, y in zip(before, after):
        assert torch.equal(x, y)
    st.close()
