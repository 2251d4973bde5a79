"""The configurations of the benchmark at their full sizes, against the CPU oracle: sampled queries of the
tensor-core prefill of 8192 queries over 24 576 rows; one dense query over 262 144 rows for the three KV
kinds; the 64-session batch with seeded context lengths up to 131 072 and 2051-entry lists per kv head
through the fused append + decode (only the selected rows are materialised); plus size-independent
properties: the prefill in one call == in two chunks, appends in one call == in ragged chunks (bytes),
dense attention over 262 144 rows == the merge of its 8 position shards, a 12-layer prefix snapshot
round trip."""
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
    # (1) sampled queries against the oracle: fp32 attention of query t over rows [0, base + t + 1) of the
    # q8_0 cache the oracle quantises from the same fp32 rows
    kc, vc = oracle.kv_write(host(k), 2), oracle.kv_write(host(v), 2)
    threads = max(1, oracle.host_procs())
    for t in (0, 1, 15, 16, 4095, 4096, 8000, n_tok - 1):
        ref = oracle.attn(host(q[t].float()), kc, vc, host(gate[t]), N_HEAD, N_KVH, HD, 1, base + t, base + n_tok, SCALE, 2,
                          threads=threads)[0]
        check(host(out[t].float()), ref, "token %d vs oracle" % t)
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


@pytest.mark.parametrize("kind", [2, 1, 0])
def test_dense_262144_vs_oracle(oracle, kind):
    """configs[4] on one GPU: one query (bf16, with a gate) over all 262 144 rows of a q8_0 / f16 / f32
    store against the oracle's fp32 attention over the cache bytes it builds from the same fp32 rows"""
    L = lib()
    ctx, chunk = 262144, 32768
    torch.manual_seed(40 + kind)
    st = q4gpu.KVStore(1, N_KVH, HD, ctx, kind)
    kh, vh = np.empty((ctx, KVW), np.float32), np.empty((ctx, KVW), np.float32)
    for p0 in range(0, ctx, chunk):
        k = torch.randn(chunk, KVW, device="cuda")
        v = torch.randn(chunk, KVW, device="cuda")
        st.append(0, k, v, p0, chunk)
        kh[p0:p0 + chunk], vh[p0:p0 + chunk] = host(k), host(v)
    q = torch.randn(N_HEAD, HD, device="cuda").to(torch.bfloat16)
    gate = torch.randn(N_HEAD, HD, device="cuda")
    out = torch.empty(N_HEAD * HD, device="cuda")
    st.decode(0, q, out, N_HEAD, SCALE, gate=gate, n_kv=ctx, q_bf16=True)
    ref = oracle.attn(host(q.float()), oracle.kv_write(kh, kind), oracle.kv_write(vh, kind), host(gate), N_HEAD, N_KVH, HD,
                      1, ctx - 1, ctx, SCALE, kind, threads=max(1, oracle.host_procs()))[0]
    assert_close(host(out).reshape(N_HEAD, HD), ref, "dense 262144, kind %d" % kind)
    assert L.q4_gpu_last_error() == 0
    st.close()


def bench_selection(rng, ctx, width=2051, sink=4, recent=1024, nrand=1023):
    """the benchmark's recipe: sinks + `nrand` random of the middle + the most recent, sorted; -1 padded"""
    out = np.full(width, -1, np.int32)
    if ctx <= width:
        out[:ctx] = np.arange(ctx)
        return out
    mid = rng.choice(ctx - recent - sink, nrand, replace=False) + sink
    out[:] = np.sort(np.concatenate([np.arange(sink), mid, np.arange(ctx - recent, ctx)]))
    return out


def test_batch_64_sessions_2051_wide_vs_oracle(oracle):
    """configs[3]: 64 sessions with seeded context lengths in [1024, 131072], one 2051-entry list per kv head
    whose last entry is the row being appended, through q4_gpu_batch_append_decode (one launch: the kernel
    quantises and stores every session's new row, then attends).  Only the selected rows exist in the
    stores, at their positions; the oracle attends a compact copy of the same rows.  Every session's
    output and every stored new row is compared."""
    L = lib()
    n_sess, width = 64, 2051
    rng = np.random.default_rng(20261125 + 4)
    ctxs = rng.integers(1024, 131072 + 1, n_sess)
    ctxs[0], ctxs[1] = 1024, 131072                       # both ends of the range
    stores, items, lists = [], [], []
    newk = rng.standard_normal((n_sess, KVW), dtype=np.float32)
    newv = rng.standard_normal((n_sess, KVW), dtype=np.float32)
    qb = oracle.f32_to_bf16(rng.standard_normal((n_sess, N_HEAD * HD), dtype=np.float32))
    gate = rng.standard_normal((n_sess, N_HEAD * HD), dtype=np.float32)
    for s_i, ctx in enumerate(int(c) for c in ctxs):
        # the token being decoded sits at position ctx: the lists are drawn over ctx + 1 rows and end with it
        idx = np.stack([bench_selection(rng, ctx + 1) for _ in range(N_KVH)])
        live = np.unique(idx[idx >= 0])
        assert live[-1] == ctx
        rows = rng.standard_normal((2, len(live), KVW), dtype=np.float32)
        rows[0, -1], rows[1, -1] = newk[s_i], newv[s_i]   # the oracle's copy of the appended row
        st = q4gpu.KVStore(1, N_KVH, HD, ctx + 1, 2)
        old = live[:-1]
        dk, dv = dev(rows[0, :-1]), dev(rows[1, :-1])
        for r in np.split(np.arange(len(old)), np.where(np.diff(old) != 1)[0] + 1):
            st.append(0, dk[r[0]:r[-1] + 1], dv[r[0]:r[-1] + 1], int(old[r[0]]), len(r))
        remap = np.full(ctx + 1, -1, np.int32)
        remap[live] = np.arange(len(live), dtype=np.int32)
        cidx = np.where(idx >= 0, remap[np.maximum(idx, 0)], -1).astype(np.int32)
        items.append(dict(q=oracle.bf16_to_f32(qb[s_i]), kc=oracle.kv_write(rows[0], 2), vc=oracle.kv_write(rows[1], 2),
                          gate=gate[s_i], out=np.empty(N_HEAD * HD, np.float32), idx=cidx, width=width,
                          idx_kvh_stride=width, kv_base=0, max_kv=len(live)))
        stores.append(st)
        lists.append(idx)
    oracle.attn_items(items, N_HEAD, N_KVH, HD, SCALE, 2, max(1, oracle.host_procs()))
    batch = q4gpu.Batch(stores)
    batch.set_pos([int(c) for c in ctxs])
    out = torch.empty(n_sess, N_HEAD * HD, device="cuda")
    dq = torch.from_numpy(qb.view(np.int16)).cuda()
    batch.append_decode(0, dev(newk), dev(newv), dq, out, N_HEAD, SCALE, gate=dev(gate), idx=dev(np.stack(lists)),
                        width=width, idx_kvh_stride=width, idx_sess_stride=N_KVH * width, q_bf16=True)
    got = host(out)
    worst = 0.0
    for s_i in range(n_sess):
        worst = max(worst, assert_close(got[s_i], items[s_i]["out"], "session %d (ctx %d)" % (s_i, ctxs[s_i])))
    # the rows the kernel appended: the oracle's q8_0 bytes, bit for bit
    for s_i in (0, 1, 17, 63):
        for which, src in ((0, newk), (1, newv)):
            assert np.array_equal(host(export_bytes(stores[s_i], 0, which, int(ctxs[s_i]), 1)), oracle.kv_write(src[s_i], 2))
    assert L.q4_gpu_last_error() == 0
    assert worst > 0
    batch.close()
    for st in stores:
        st.close()


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
