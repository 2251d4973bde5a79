"""GPU parity of the decode attention through the C ABI against the CPU oracle (fp32), within
2e-3 max-abs + 1e-3 relative: the reference's own fixture, the ctx-4096 reference check, sparse
selections with padding, ragged sizes, every head_dim / GQA shape, partial + merge, batches,
graph replay."""
import numpy as np
import pytest
import torch

import q4gpu
from gpu_util import assert_close, dev, dev_bytes, host, lib
from test_oracle import dense_ref64, ref_fixture

pytestmark = pytest.mark.gpu


def test_reference_fixture_through_reference_abi(oracle):
    """src/q4_test.c:134-238: q4_hip_qsa_decode_n with n_tok = 2 on f32 / f16 / q8_0 caches built by
    q4_hip_f32_to_f16 / q4_hip_f32_to_q8, against the unquantised reference with the tolerances the
    reference asserts (1e-3, 2e-2, 8e-2), and against the oracle on the same cache bytes."""
    L = lib()
    fx = ref_fixture()
    ref = dense_ref64(fx).reshape(-1)
    n = fx["npos"] * fx["hd"]
    dq, dk, dv, dg = dev(fx["q"]), dev(fx["k"]), dev(fx["v"]), dev(fx["gate"])
    dout = torch.empty_like(dq)
    dk16 = torch.empty(n, dtype=torch.float16, device="cuda")
    dv16 = torch.empty_like(dk16)
    dk8 = torch.empty(n // 32 * 34, dtype=torch.uint8, device="cuda")
    dv8 = torch.empty_like(dk8)
    assert L.q4_hip_f32_to_f16(dk16.data_ptr(), dk.data_ptr(), n) and L.q4_hip_f32_to_f16(dv16.data_ptr(), dv.data_ptr(), n)
    assert L.q4_hip_f32_to_q8(dk8.data_ptr(), dk.data_ptr(), n) and L.q4_hip_f32_to_q8(dv8.data_ptr(), dv.data_ptr(), n)
    for kind, kc, vc, tol in ((0, dk, dv, 1e-3), (1, dk16, dv16, 2e-2), (2, dk8, dv8, 8e-2)):
        assert L.q4_hip_qsa_decode_n(dq.data_ptr(), kc.data_ptr(), vc.data_ptr(), dg.data_ptr(), dout.data_ptr(),
                                     fx["n_head"], fx["n_kvh"], fx["hd"], fx["n_tok"], 0, fx["npos"],
                                     float(fx["scale"]), kind)
        got = host(dout)
        assert np.abs(got - ref).max() <= tol, kind
        orc = oracle.attn(fx["q"], oracle.kv_write(fx["k"], kind), oracle.kv_write(fx["v"], kind), fx["gate"],
                          fx["n_head"], fx["n_kvh"], fx["hd"], fx["n_tok"], 0, fx["npos"], float(fx["scale"]), kind)
        assert_close(got, orc.reshape(-1), "fixture kind %d" % kind)
    # NULL gate / zero sizes are rejected like the reference (src/q4_rocm.cu:7254-7255)
    assert not L.q4_hip_qsa_decode_n(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), None, dout.data_ptr(), 2, 1, 32, 2, 0, 4, 1.0, 0)
    assert not L.q4_hip_qsa_decode_n(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(), dout.data_ptr(), 2, 1, 32, 0, 0, 4, 1.0, 0)
    assert not L.q4_hip_qsa_decode(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(), dout.data_ptr(), 2, 1, 32, 0, 4, 1.0, 0)


def make_case(oracle, seed, ctx, n_head, n_kvh, hd, rope=True):
    kvw = n_kvh * hd
    k = oracle.normal(seed, 0, ctx * kvw).reshape(ctx, n_kvh, hd)
    v = oracle.normal(seed, 1, ctx * kvw).reshape(ctx, kvw)
    q = oracle.normal(seed, 2, n_head * hd).reshape(1, n_head, hd)
    if rope:
        k = oracle.rope_rows(k, hd, 0, 1e7)
        q = oracle.rope_rows(q, hd, ctx - 1, 1e7)
    return k.reshape(ctx, kvw), v, q.reshape(n_head, hd)


@pytest.mark.parametrize("kind", [2, 1, 0])
def test_config1_ctx4096_reference_check(oracle, kind):
    """One sequence, ctx 4096, 16 query / 2 kv heads, hd 128, RoPE theta 1e7 on Q and K; append all
    rows, dense decode of the last query, scale 1/sqrt(128) -- store path and reference-ABI path."""
    L = lib()
    ctx, n_head, n_kvh, hd = 4096, 16, 2, 128
    k, v, q = make_case(oracle, 20261125 + 1, ctx, n_head, n_kvh, hd)
    scale = 1.0 / np.sqrt(hd)
    kc, vc = oracle.kv_write(k, kind), oracle.kv_write(v, kind)
    ref = oracle.attn(q, kc, vc, None, n_head, n_kvh, hd, 1, ctx - 1, ctx, scale, kind)[0]
    ref64 = oracle.attn(q, kc, vc, None, n_head, n_kvh, hd, 1, ctx - 1, ctx, scale, kind, acc64=True)[0]
    st = q4gpu.KVStore(1, n_kvh, hd, ctx, kind)
    st.append(0, dev(k), dev(v), 0, ctx)
    if kind == 2:   # quantised bytes are the oracle's, bit for bit
        out = torch.empty(ctx * st.token_bytes, dtype=torch.uint8, device="cuda")
        st.export(0, 0, 0, ctx, out)
        assert np.array_equal(host(out), kc)
        st.export(0, 1, 0, ctx, out)
        assert np.array_equal(host(out), vc)
    dq = dev(q)
    dout = torch.empty(n_head * hd, device="cuda")
    st.decode(0, dq, dout, n_head, scale, n_kv=ctx)
    e1 = assert_close(host(dout).reshape(n_head, hd), ref, "store kind %d" % kind)
    assert_close(host(dout).reshape(n_head, hd), ref64, "store kind %d vs fp64" % kind)
    # the same through the reference ABI on a cache in the reference layout (gate = 0 -> x 0.5)
    gate = torch.zeros(n_head * hd, device="cuda")
    dkc, dvc = dev_bytes(kc), dev_bytes(vc)
    assert L.q4_hip_qsa_decode(dq.data_ptr(), dkc.data_ptr(), dvc.data_ptr(), gate.data_ptr(), dout.data_ptr(),
                               n_head, n_kvh, hd, ctx, ctx, scale, kind)
    assert_close(2 * host(dout).reshape(n_head, hd), ref, "reference ABI kind %d" % kind)
    # bf16 queries (the bench's query type): compare with the oracle run on the rounded queries
    qb = oracle.f32_to_bf16(q)
    refb = oracle.attn(oracle.bf16_to_f32(qb), kc, vc, None, n_head, n_kvh, hd, 1, ctx - 1, ctx, scale, kind)[0]
    dqb = torch.from_numpy(qb.view(np.int16)).cuda()
    st.decode(0, dqb, dout, n_head, scale, n_kv=ctx, q_bf16=True)
    assert_close(host(dout).reshape(n_head, hd), refb, "bf16 q kind %d" % kind)
    st.close()


@pytest.mark.parametrize("ctx", list(range(1, 36)) + [47, 48, 49, 63, 64, 65, 70, 255, 1000, 1025])
def test_dense_ragged_lengths(oracle, ctx):
    """every length around the 16-position step and the split boundaries"""
    lib()
    n_head, n_kvh, hd = 16, 2, 128
    k, v, q = make_case(oracle, 100 + ctx, ctx, n_head, n_kvh, hd)
    st = q4gpu.KVStore(1, n_kvh, hd, 1100, 2)
    st.append(0, dev(k), dev(v), 0, ctx)
    gate = oracle.normal(7, ctx, n_head * hd)
    dout = torch.empty(n_head * hd, device="cuda")
    st.decode(0, dev(q), dout, n_head, 0.0883883, gate=dev(gate), n_kv=ctx)
    ref = oracle.attn(q, oracle.kv_write(k, 2), oracle.kv_write(v, 2), gate, n_head, n_kvh, hd, 1, ctx - 1, ctx,
                      0.0883883, 2)[0]
    assert_close(host(dout).reshape(n_head, hd), ref, "ctx %d" % ctx)
    st.close()


@pytest.mark.parametrize("n_head,n_kvh,hd", [(2, 1, 32), (4, 4, 32), (8, 2, 64), (24, 2, 256), (16, 1, 128),
                                             (12, 1, 64), (32, 4, 128), (5, 1, 128), (16, 2, 256)])
@pytest.mark.parametrize("kind", [2, 1, 0])
def test_shapes_and_kinds(oracle, n_head, n_kvh, hd, kind):
    """head_dim 32..256, GQA group 1..16 (incl. the real model's 24 / 2 / 256), all three KV kinds,
    store layout and reference layout"""
    L = lib()
    ctx = 333
    k, v, q = make_case(oracle, 7 * n_head + hd + kind, ctx, n_head, n_kvh, hd, rope=False)
    scale = 1.0 / np.sqrt(hd)
    kc, vc = oracle.kv_write(k, kind), oracle.kv_write(v, kind)
    gate = oracle.normal(3, n_head + hd, n_head * hd)
    ref = oracle.attn(q, kc, vc, gate, n_head, n_kvh, hd, 1, ctx - 1, ctx, scale, kind)[0]
    st = q4gpu.KVStore(2, n_kvh, hd, 400, kind)
    st.append(1, dev(k), dev(v), 0, ctx)
    dout = torch.empty(n_head * hd, device="cuda")
    dq, dg = dev(q), dev(gate)
    st.decode(1, dq, dout, n_head, scale, gate=dg, n_kv=ctx)
    assert_close(host(dout).reshape(n_head, hd), ref, "store")
    dkc, dvc = dev_bytes(kc), dev_bytes(vc)
    assert L.q4_hip_qsa_decode_n(dq.data_ptr(), dkc.data_ptr(), dvc.data_ptr(), dg.data_ptr(), dout.data_ptr(),
                                 n_head, n_kvh, hd, 1, ctx - 1, ctx, scale, kind)
    assert_close(host(dout).reshape(n_head, hd), ref, "reference ABI")
    st.close()


def selection(oracle, seed, ctx, n_kvh, width=2051):
    return np.stack([oracle.select(seed, kh, ctx, width) for kh in range(n_kvh)])


@pytest.mark.parametrize("ctx", [262144, 65536, 2052, 2051, 1500])
def test_qsa_sparse_decode_per_kv_head_lists(oracle, ctx):
    """The benchmark's selection recipe (4 sink + 1024 recent + 1023 random, sorted, one list per kv
    head) at the full context length: only the selected rows are materialised, at their positions."""
    lib()
    n_head, n_kvh, hd, width = 16, 2, 128, 2051
    idx = selection(oracle, 20261125 + 2, ctx, n_kvh)
    live = np.unique(idx[idx >= 0])
    kvw = n_kvh * hd
    krows = oracle.normal(31, 0, len(live) * kvw).reshape(len(live), kvw)
    vrows = oracle.normal(31, 1, len(live) * kvw).reshape(len(live), kvw)
    q = oracle.normal(31, 2, n_head * hd)
    st = q4gpu.KVStore(1, n_kvh, hd, ctx, 2)
    # scatter row by row at the selected positions (runs of consecutive positions in one call)
    runs = np.split(np.arange(len(live)), np.where(np.diff(live) != 1)[0] + 1)
    dk, dv = dev(krows), dev(vrows)
    for r in runs:
        st.append(0, dk[r[0]:r[-1] + 1], dv[r[0]:r[-1] + 1], int(live[r[0]]), len(r))
    # oracle: compact cache of the live rows, lists remapped to compact indices
    remap = {int(p): i for i, p in enumerate(live)}
    cidx = np.vectorize(lambda p: remap[int(p)] if p >= 0 else -1)(idx).astype(np.int32)
    kc, vc = oracle.kv_write(krows, 2), oracle.kv_write(vrows, 2)
    scale = 1.0 / np.sqrt(hd)
    ref = oracle.attn(q, kc, vc, None, n_head, n_kvh, hd, 1, 0, len(live), scale, 2, idx=cidx, width=width,
                      idx_kvh_stride=width)[0]
    dout = torch.empty(n_head * hd, device="cuda")
    st.decode(0, dev(q), dout, n_head, scale, idx=dev(idx), width=width, idx_kvh_stride=width, n_kv=ctx)
    assert_close(host(dout).reshape(n_head, hd), ref, "sparse ctx %d" % ctx)
    st.close()


@pytest.mark.parametrize("width", [1, 15, 16, 17, 31, 32, 33, 100])
def test_indexed_padding_edges(oracle, width):
    """-1 padding anywhere in the list, tile-edge widths, a shared list (the reference's form), an
    all-padding list -> zeros, out-of-range positions -> skipped and reported"""
    L = lib()
    n_head, n_kvh, hd, ctx = 16, 2, 128, 120
    k, v, q = make_case(oracle, 900 + width, ctx, n_head, n_kvh, hd, rope=False)
    kc, vc = oracle.kv_write(k, 2), oracle.kv_write(v, 2)
    rng = np.random.default_rng(width)
    idx = np.full((n_kvh, width), -1, np.int32)
    for kh in range(n_kvh):
        m = rng.integers(0, width + 1)
        slots = rng.choice(width, m, replace=False)
        idx[kh, slots] = rng.choice(ctx, m, replace=False)
    if width == 33:
        idx[1, :] = -1          # one kv head with nothing selected
    gate = oracle.normal(1, width, n_head * hd)
    st = q4gpu.KVStore(1, n_kvh, hd, ctx, 2)
    st.append(0, dev(k), dev(v), 0, ctx)
    dout = torch.full((n_head * hd,), 7.0, device="cuda")
    st.decode(0, dev(q), dout, n_head, 0.09, gate=dev(gate), idx=dev(idx), width=width, idx_kvh_stride=width, n_kv=ctx)
    ref = oracle.attn(q, kc, vc, gate, n_head, n_kvh, hd, 1, 0, ctx, 0.09, 2, idx=idx, width=width, idx_kvh_stride=width)[0]
    got = host(dout).reshape(n_head, hd)
    assert_close(got, ref, "width %d" % width)
    if width == 33:
        assert not got[8:].any()
    # shared list through the reference ABI
    dkc, dvc, dg = dev_bytes(kc), dev_bytes(vc), dev(gate)
    assert L.q4_hip_qsa_decode_idx(dev(q).data_ptr(), dkc.data_ptr(), dvc.data_ptr(), dg.data_ptr(), dout.data_ptr(),
                                   dev(idx[0]).data_ptr(), width, n_head, n_kvh, hd, 1, ctx, 0.09, 2)
    ref2 = oracle.attn(q, kc, vc, gate, n_head, n_kvh, hd, 1, 0, ctx, 0.09, 2, idx=idx[0], width=width)[0]
    assert_close(host(dout).reshape(n_head, hd), ref2, "shared list width %d" % width)
    # positions beyond max_kv are skipped, not dereferenced, and reported
    L.q4_gpu_last_error()
    bad = idx.copy()
    bad[0, 0] = ctx + 5
    st.decode(0, dev(q), dout, n_head, 0.09, gate=dev(gate), idx=dev(bad), width=width, idx_kvh_stride=width, n_kv=ctx)
    torch.cuda.synchronize()
    assert L.q4_gpu_last_error() & 4
    bad[0, 0] = -1
    ref3 = oracle.attn(q, kc, vc, gate, n_head, n_kvh, hd, 1, 0, ctx, 0.09, 2, idx=bad, width=width, idx_kvh_stride=width)[0]
    assert_close(host(dout).reshape(n_head, hd), ref3, "out-of-range skipped")
    st.close()


def test_causal_batch_through_reference_abi(oracle):
    """n_tok > 1: token t attends [0, kv_base + t + 1), capped at max_kv (src/q4_rocm.cu:7032-7033);
    indexed form with one list per token"""
    L = lib()
    n_head, n_kvh, hd, n_tok, kv_base, max_kv = 16, 2, 128, 9, 50, 56
    kvw = n_kvh * hd
    k = oracle.normal(77, 0, max_kv * kvw)
    v = oracle.normal(77, 1, max_kv * kvw)
    q = oracle.normal(77, 2, n_tok * n_head * hd)
    gate = oracle.normal(77, 3, n_tok * n_head * hd)
    for kind in (2, 1, 0):
        kc, vc = oracle.kv_write(k, kind), oracle.kv_write(v, kind)
        ref = oracle.attn(q, kc, vc, gate, n_head, n_kvh, hd, n_tok, kv_base, max_kv, 0.0884, kind)
        dout = torch.empty(n_tok * n_head * hd, device="cuda")
        assert L.q4_hip_qsa_decode_n(dev(q).data_ptr(), dev_bytes(kc).data_ptr(), dev_bytes(vc).data_ptr(),
                                     dev(gate).data_ptr(), dout.data_ptr(), n_head, n_kvh, hd, n_tok, kv_base,
                                     max_kv, 0.0884, kind)
        assert_close(host(dout).reshape(n_tok, n_head, hd), ref, "causal kind %d" % kind)
    width = 20
    rng = np.random.default_rng(5)
    idx = np.stack([np.sort(rng.choice(max_kv, width, replace=False)) for _ in range(n_tok)]).astype(np.int32)
    idx[3, 10:] = -1
    kc, vc = oracle.kv_write(k, 2), oracle.kv_write(v, 2)
    ref = oracle.attn(q, kc, vc, gate, n_head, n_kvh, hd, n_tok, 0, max_kv, 0.0884, 2, idx=idx, width=width)
    assert L.q4_hip_qsa_decode_idx(dev(q).data_ptr(), dev_bytes(kc).data_ptr(), dev_bytes(vc).data_ptr(),
                                   dev(gate).data_ptr(), dout.data_ptr(), dev(idx).data_ptr(), width, n_head, n_kvh,
                                   hd, n_tok, max_kv, 0.0884, 2)
    assert_close(host(dout).reshape(n_tok, n_head, hd), ref, "indexed batch")


@pytest.mark.parametrize("kind", [2, 1, 0])
@pytest.mark.parametrize("per_kvh", [True, False])
def test_sparse_prefill_on_the_store(oracle, kind, per_kvh):
    """n_tok queries, each over its own list (one per kv head, or one shared by the kv heads as in the
    reference), padding inside the lists, one launch on the library-owned store"""
    lib()
    n_head, n_kvh, hd, ctx, n_tok, width = 16, 2, 128, 3000, 37, 301
    k, v, _ = make_case(oracle, 4100 + kind, ctx, n_head, n_kvh, hd, rope=False)
    q = oracle.normal(4100, 7, n_tok * n_head * hd)
    gate = oracle.normal(4100, 8, n_tok * n_head * hd)
    rng = np.random.default_rng(41 + kind)
    lists = n_kvh if per_kvh else 1
    idx = np.full((n_tok, lists, width), -1, np.int32)
    for t in range(n_tok):
        for l in range(lists):
            m = int(rng.integers(1, width + 1))
            idx[t, l, np.sort(rng.choice(width, m, replace=False))] = np.sort(rng.choice(ctx, m, replace=False))
    idx[5] = -1                                  # a token that selects nothing -> zeros
    kc, vc = oracle.kv_write(k, kind), oracle.kv_write(v, kind)
    ref = oracle.attn(q, kc, vc, gate, n_head, n_kvh, hd, n_tok, 0, ctx, 0.0884, kind, idx=idx, width=width,
                      idx_kvh_stride=width if per_kvh else 0)
    st = q4gpu.KVStore(1, n_kvh, hd, ctx, kind)
    st.append(0, dev(k), dev(v), 0, ctx)
    dout = torch.full((n_tok * n_head * hd,), 3.0, device="cuda")
    st.decode_idx_n(0, dev(q), dout, n_head, 0.0884, dev(idx), width, n_tok, idx_tok_stride=lists * width,
                    idx_kvh_stride=width if per_kvh else 0, gate=dev(gate))
    got = host(dout).reshape(n_tok, n_head, hd)
    assert_close(got, ref, "sparse prefill kind %d" % kind)
    assert not got[5].any()
    # bf16 queries: same call, the oracle sees the rounded values
    qb = dev(q).to(torch.bfloat16)
    ref_b = oracle.attn(host(qb.float()), kc, vc, None, n_head, n_kvh, hd, n_tok, 0, ctx, 0.0884, kind, idx=idx,
                        width=width, idx_kvh_stride=width if per_kvh else 0)
    st.decode_idx_n(0, qb, dout, n_head, 0.0884, dev(idx), width, n_tok, idx_tok_stride=lists * width,
                    idx_kvh_stride=width if per_kvh else 0, q_bf16=True)
    assert_close(host(dout).reshape(n_tok, n_head, hd), ref_b, "sparse prefill bf16 q kind %d" % kind)
    st.close()


@pytest.mark.parametrize("kind", [2, 1, 0])
def test_sequence_shards_partial_and_merge(oracle, kind):
    """One sequence split by position over G stores: each computes (m, l, acc), the records are merged
    (the exchange payload of the sequence-sharded decode) == attention over the whole sequence; records
    also match the oracle's records."""
    L = lib()
    n_head, n_kvh, hd, ctx, G = 16, 2, 128, 4096, 4
    k, v, q = make_case(oracle, 4242 + kind, ctx, n_head, n_kvh, hd)
    scale = 1.0 / np.sqrt(hd)
    kc, vc = oracle.kv_write(k, kind), oracle.kv_write(v, kind)
    gate = oracle.normal(4242, 9, n_head * hd)
    full = oracle.attn(q, kc, vc, gate, n_head, n_kvh, hd, 1, ctx - 1, ctx, scale, kind)[0]
    parts = torch.empty(G, n_head, hd + 2, device="cuda")
    per = ctx // G
    stores = []
    for r in range(G):
        st = q4gpu.KVStore(1, n_kvh, hd, per, kind)
        st.append(0, dev(k[r * per:(r + 1) * per]), dev(v[r * per:(r + 1) * per]), 0, per)
        st.decode_partial(0, dev(q), parts[r], n_head, scale, n_kv=per)
        stores.append(st)
    dout = torch.empty(n_head * hd, device="cuda")
    assert L.q4_gpu_lse_merge(parts.data_ptr(), G, n_head, hd, dev(gate).data_ptr(), dout.data_ptr())
    assert_close(host(dout).reshape(n_head, hd), full, "merged shards kind %d" % kind)
    got = host(parts)
    for r in range(G):
        want = oracle.attn_partial(q, kc, vc, n_head, n_kvh, hd, scale, kind, r * per, (r + 1) * per)
        # records are equal up to the common factor exp(m_got - m_want): compare normalised
        assert np.allclose(got[r, :, 0], want[:, 0], atol=2e-3)
        assert_close(got[r, :, 2:] / got[r, :, 1:2], want[:, 2:] / want[:, 1:2], "record %d" % r)
    # an empty shard contributes nothing
    empty = torch.zeros(1, n_head, hd + 2, device="cuda")
    both = torch.cat([parts, empty])
    assert L.q4_gpu_lse_merge(both.data_ptr(), G + 1, n_head, hd, dev(gate).data_ptr(), dout.data_ptr())
    assert_close(host(dout).reshape(n_head, hd), full, "merge with empty shard")
    assert_close(host(dout).reshape(n_head, hd), oracle.lse_merge(host(both), n_head, hd, gate), "merge kernel vs oracle merge")
    for st in stores:
        st.close()


def test_batched_sessions_match_single_session(oracle):
    """Sessions of different lengths decoded by one launch per layer: same numbers as one at a time;
    dense and sparse; append through the batch at each session's own position."""
    lib()
    n_head, n_kvh, hd, n_layers, width = 16, 2, 128, 2, 64
    lens = [1, 17, 300, 64, 1000, 33, 128, 2]
    kvw = n_kvh * hd
    stores, data = [], []
    for s, n in enumerate(lens):
        st = q4gpu.KVStore(n_layers, n_kvh, hd, 1024, 2)
        k = oracle.normal(500 + s, 0, n * kvw).reshape(n, kvw)
        v = oracle.normal(500 + s, 1, n * kvw).reshape(n, kvw)
        if n > 1:
            st.append(1, dev(k[:-1]), dev(v[:-1]), 0, n - 1)
        stores.append(st)
        data.append((k, v))
    b = q4gpu.Batch(stores)
    b.set_pos([n - 1 for n in lens])
    last_k = np.stack([d[0][-1] for d in data])
    last_v = np.stack([d[1][-1] for d in data])
    b.append(1, dev(last_k), dev(last_v))          # row s -> slot lens[s]-1 of session s
    q = oracle.normal(600, 0, len(lens) * n_head * hd).reshape(len(lens), n_head, hd)
    gate = oracle.normal(600, 1, len(lens) * n_head * hd).reshape(len(lens), n_head, hd)
    dout = torch.empty(len(lens) * n_head * hd, device="cuda")
    b.decode(1, dev(q), dout, n_head, 0.0884, gate=dev(gate))
    got = host(dout).reshape(len(lens), n_head, hd)
    for s, n in enumerate(lens):
        kc, vc = oracle.kv_write(data[s][0], 2), oracle.kv_write(data[s][1], 2)
        ref = oracle.attn(q[s], kc, vc, gate[s], n_head, n_kvh, hd, 1, n - 1, n, 0.0884, 2)[0]
        assert_close(got[s], ref, "dense session %d" % s)
    idx = np.full((len(lens), n_kvh, width), -1, np.int32)
    for s, n in enumerate(lens):
        for kh in range(n_kvh):
            sel = oracle.select(700 + s, kh, n, width, sink=2, recent=30, nrand=32)
            idx[s, kh] = sel
    b.decode(1, dev(q), dout, n_head, 0.0884, idx=dev(idx), width=width, idx_kvh_stride=width,
             idx_sess_stride=n_kvh * width)
    got = host(dout).reshape(len(lens), n_head, hd)
    for s, n in enumerate(lens):
        kc, vc = oracle.kv_write(data[s][0], 2), oracle.kv_write(data[s][1], 2)
        ref = oracle.attn(q[s], kc, vc, None, n_head, n_kvh, hd, 1, 0, n, 0.0884, 2, idx=idx[s], width=width,
                          idx_kvh_stride=width)[0]
        assert_close(got[s], ref, "sparse session %d" % s)
    b.close()
    for st in stores:
        st.close()


def test_graph_captured_decode_follows_the_position_word(oracle):
    """append + dense decode captured once, replayed for successive tokens: rows attended = position
    word + 1 (the reference's graphed decode layer, src/q4_fwd.c:838-928)."""
    L = lib()
    L.q4_gpu_set_stream(None)
    n_head, n_kvh, hd, max_kv = 16, 2, 128, 64
    kvw = n_kvh * hd
    st = q4gpu.KVStore(1, n_kvh, hd, max_kv, 2)
    kbuf, vbuf = torch.zeros(kvw, device="cuda"), torch.zeros(kvw, device="cuda")
    qbuf, obuf = torch.zeros(n_head * hd, device="cuda"), torch.zeros(n_head * hd, device="cuda")
    torch.cuda.synchronize()
    assert L.q4_hip_qsa_topk_alloc()
    assert L.q4_hip_graph_begin() == 1
    assert L.q4_gpu_kv_append_d(st.h, 0, kbuf.data_ptr(), vbuf.data_ptr())
    assert L.q4_gpu_kv_decode(st.h, 0, qbuf.data_ptr(), 0, None, obuf.data_ptr(), n_head, None, 0, 0, 0, 0.0884)
    g = L.q4_hip_graph_end()
    assert g
    ks, vs = [], []
    for pos in range(40):
        k, v, q = oracle.normal(800, pos, kvw), oracle.normal(801, pos, kvw), oracle.normal(802, pos, n_head * hd)
        ks.append(k)
        vs.append(v)
        for d, h in ((kbuf, k), (vbuf, v), (qbuf, q)):
            assert L.q4_hip_h2d(d.data_ptr(), h.ctypes.data, h.nbytes)
        L.q4_hip_pos_push(pos)
        assert L.q4_hip_graph_launch(g)
        out = np.empty(n_head * hd, np.float32)
        assert L.q4_hip_d2h(out.ctypes.data, obuf.data_ptr(), out.nbytes)
        if pos in (0, 1, 15, 16, 17, 39):
            kc, vc = oracle.kv_write(np.stack(ks), 2), oracle.kv_write(np.stack(vs), 2)
            ref = oracle.attn(q, kc, vc, None, n_head, n_kvh, hd, 1, pos, pos + 1, 0.0884, 2)[0]
            assert_close(out.reshape(n_head, hd), ref, "replay pos %d" % pos)
    L.q4_hip_graph_free(g)
    q4gpu.use_torch_stream()
    st.close()


def test_graph_captured_batch_step_advances_its_positions_on_the_device(oracle):
    """position advance + fused append + dense decode of three sessions captured once and replayed for
    successive tokens with no position upload in between: after set_pos(p - 1) the k-th replay appends at
    slot p + k - 1 of every session and attends p + k rows."""
    L = lib()
    L.q4_gpu_set_stream(None)
    n_head, n_kvh, hd, max_kv = 16, 2, 128, 96
    kvw = n_kvh * hd
    starts = [5, 31, 48]
    stores, rows = [], []
    for s, p in enumerate(starts):
        k = oracle.normal(820 + s, 0, p * kvw).reshape(p, kvw)
        st = q4gpu.KVStore(1, n_kvh, hd, max_kv, 2)
        st.append(0, dev(k), dev(k), 0, p)
        stores.append(st)
        rows.append(list(k))
    b = q4gpu.Batch(stores)
    n = len(starts)
    kbuf, qbuf = torch.zeros(n, kvw, device="cuda"), torch.zeros(n, n_head * hd, device="cuda")
    obuf = torch.zeros(n, n_head * hd, device="cuda")
    torch.cuda.synchronize()
    b.set_pos([p - 1 for p in starts])
    assert L.q4_hip_graph_begin() == 1
    b.advance(1)
    b.append_decode(0, kbuf, kbuf, qbuf, obuf, n_head, 0.0884)
    g = L.q4_hip_graph_end()
    assert g
    for step in range(20):
        k = oracle.normal(830, step, n * kvw).reshape(n, kvw)
        q = oracle.normal(831, step, n * n_head * hd).reshape(n, n_head * hd)
        for d, h in ((kbuf, k), (qbuf, q)):
            assert L.q4_hip_h2d(d.data_ptr(), h.ctypes.data, h.nbytes)
        assert L.q4_hip_graph_launch(g)
        out = np.empty((n, n_head * hd), np.float32)
        assert L.q4_hip_d2h(out.ctypes.data, obuf.data_ptr(), out.nbytes)
        for s in range(n):
            rows[s].append(k[s])
        if step in (0, 1, 10, 19):
            for s in range(n):
                kc = oracle.kv_write(np.stack(rows[s]), 2)
                n_kv = starts[s] + step + 1
                ref = oracle.attn(q[s], kc, kc, None, n_head, n_kvh, hd, 1, n_kv - 1, n_kv, 0.0884, 2)[0]
                assert_close(out[s].reshape(n_head, hd), ref, "replay %d session %d" % (step, s))
    # outside a capture the advance is an ordinary launch; a negative step takes positions back
    b.advance(-20)
    b.advance(1)
    assert L.q4_hip_graph_launch(g)                       # advances once more: slot p + 1 again, rewritten
    out = np.empty((n, n_head * hd), np.float32)
    assert L.q4_hip_d2h(out.ctypes.data, obuf.data_ptr(), out.nbytes)
    for s in range(n):
        kc = oracle.kv_write(np.stack(rows[s][:starts[s] + 1] + [k[s]]), 2)
        ref = oracle.attn(q[s], kc, kc, None, n_head, n_kvh, hd, 1, starts[s] + 1, starts[s] + 2, 0.0884, 2)[0]
        assert_close(out[s].reshape(n_head, hd), ref, "after rewind, session %d" % s)
    assert L.q4_gpu_last_error() == 0
    L.q4_hip_graph_free(g)
    q4gpu.use_torch_stream()
    b.close()
    for st in stores:
        st.close()


@pytest.mark.parametrize("q_bf16", [False, True])
@pytest.mark.parametrize("mode", ["sigma8", "head_x50"])
def test_large_magnitude_queries(oracle, mode, q_bf16):
    """Queries far larger than N(0,1) -- every element ~ N(0, 8^2), or one head of each kv group scaled by
    50 -- through the sparse and the dense decode of the q8_0 store.  The K side of the kernel enters the
    codes as 1152 + code and removes 1152 * sum(q) through the accumulator, so the cancellation error
    grows with sum |q|; the outputs must stay within the stated tolerance of the fp32 oracle."""
    lib()
    n_head, n_kvh, hd, ctx, width = 16, 2, 128, 6000, 2051
    k, v, q = make_case(oracle, 4100, ctx, n_head, n_kvh, hd, rope=False)
    q = q.copy()
    if mode == "sigma8":
        q *= 8.0
    else:
        q[3] *= 50.0
        q[12] *= 50.0
    if q_bf16:
        qb = oracle.f32_to_bf16(q)
        q = oracle.bf16_to_f32(qb)
        dq = torch.from_numpy(qb.view(np.int16).reshape(-1)).cuda()
    else:
        dq = dev(q)
    gate = oracle.normal(4101, 0, n_head * hd)
    kc, vc = oracle.kv_write(k, 2), oracle.kv_write(v, 2)
    st = q4gpu.KVStore(1, n_kvh, hd, ctx, 2)
    st.append(0, dev(k), dev(v), 0, ctx)
    scale = 1.0 / np.sqrt(hd)
    idx = selection(oracle, 4102, ctx, n_kvh)
    out = torch.empty(n_head * hd, device="cuda")
    st.decode(0, dq, out, n_head, scale, gate=dev(gate), idx=dev(idx), width=width, idx_kvh_stride=width, n_kv=ctx,
              q_bf16=q_bf16)
    ref = oracle.attn(q, kc, vc, gate, n_head, n_kvh, hd, 1, 0, ctx, scale, 2, idx=idx, width=width, idx_kvh_stride=width)[0]
    assert_close(host(out).reshape(n_head, hd), ref, "sparse, %s" % mode)
    st.decode(0, dq, out, n_head, scale, gate=dev(gate), n_kv=ctx, q_bf16=q_bf16)
    ref = oracle.attn(q, kc, vc, gate, n_head, n_kvh, hd, 1, ctx - 1, ctx, scale, 2)[0]
    assert_close(host(out).reshape(n_head, hd), ref, "dense, %s" % mode)
    st.close()
