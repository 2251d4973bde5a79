"""The CPU oracle against what the reference itself pins for this path: its one hot-path fixture
(src/q4_test.c:134-238), its dequantiser compiled in place, and the quantiser's source contract."""
import numpy as np
import pytest


def ref_fixture():
    """Inputs of src/q4_test.c:136-153 (formulas evaluated in fp32 like the C source)."""
    n_head, n_kvh, hd, n_tok, npos = 2, 1, 32, 2, 4
    i = np.arange(npos * hd)
    k = (((i * 17) % 11).astype(np.float32) * np.float32(0.05) - np.float32(0.2)).astype(np.float32)
    v = (((i * 13) % 9).astype(np.float32) * np.float32(0.07)).astype(np.float32)
    j = np.arange(n_tok * n_head * hd)
    q = (((j * 3) % 7).astype(np.float32) * np.float32(0.1)).astype(np.float32)
    gate = (((j % 5) - 2).astype(np.float32) * np.float32(0.3)).astype(np.float32)
    return dict(n_head=n_head, n_kvh=n_kvh, hd=hd, n_tok=n_tok, npos=npos, k=k, v=v, q=q,
                gate=gate, scale=np.float32(1.0) / np.sqrt(np.float32(hd)))


def dense_ref64(fx):
    """The fixture's inline reference (src/q4_test.c:155-182) in float64."""
    nh, hd, nt = fx["n_head"], fx["hd"], fx["n_tok"]
    q = fx["q"].astype(np.float64).reshape(nt, nh, hd)
    k = fx["k"].astype(np.float64).reshape(-1, hd)
    v = fx["v"].astype(np.float64).reshape(-1, hd)
    g = fx["gate"].astype(np.float64).reshape(nt, nh, hd)
    out = np.zeros((nt, nh, hd))
    for t in range(nt):
        n_kv = t + 1
        for h in range(nh):
            s = k[:n_kv] @ q[t, h] * float(fx["scale"])
            w = np.exp(s - s.max())
            out[t, h] = (w @ v[:n_kv]) / w.sum() / (1 + np.exp(-g[t, h]))
    return out


def test_reference_fixture_all_kinds(oracle):
    fx = ref_fixture()
    ref = dense_ref64(fx)
    # tolerances the reference asserts against the UNquantised result: :201, :213, :228
    for kind, tol in ((0, 1e-3), (1, 2e-2), (2, 8e-2)):
        kc, vc = oracle.kv_write(fx["k"], kind), oracle.kv_write(fx["v"], kind)
        got = oracle.attn(fx["q"], kc, vc, fx["gate"], fx["n_head"], fx["n_kvh"], fx["hd"],
                          fx["n_tok"], 0, fx["npos"], float(fx["scale"]), kind)
        assert np.abs(got - ref).max() <= tol, kind
    # f32 KV is the same arithmetic: agree to fp32 rounding
    kc, vc = oracle.kv_write(fx["k"], 0), oracle.kv_write(fx["v"], 0)
    got = oracle.attn(fx["q"], kc, vc, fx["gate"], 2, 1, 32, 2, 0, 4, float(fx["scale"]), 0)
    assert np.abs(got - ref).max() < 1e-6


def test_f16_decode_matches_reference_all_patterns(oracle):
    R = oracle.ref_lib()
    if R is None:
        pytest.skip("oracle/_ref not built")
    L = oracle.lib()
    a = np.array([L.q4o_f16_to_f32(h) for h in range(65536)], np.float32)
    b = np.array([R.q4_f16_to_f32(h) for h in range(65536)], np.float32)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    c = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)
    fin = ~np.isnan(c)          # numpy quiets signalling-NaN payloads; everything else is bitwise
    assert np.array_equal(a.view(np.uint32)[fin], c.view(np.uint32)[fin])


def test_f16_encode_rne(oracle):
    rng = np.random.default_rng(7)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32),
        (rng.standard_normal(50000) * 1e-6).astype(np.float32),
        (rng.standard_normal(50000) * 3e4).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25,
                  1.5 * 2.0 ** -25, 2.0 ** -14, np.inf, -np.inf], np.float32),
        np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)[:31744],
    ])
    got = oracle.f32_to_f16(x)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)


def test_dequant_matches_reference_dequantiser(oracle):
    if oracle.ref_lib() is None:
        pytest.skip("oracle/_ref not built")
    rng = np.random.default_rng(3)
    nb = 4096
    blk = rng.integers(0, 256, (nb, 34), dtype=np.uint8)
    # finite scales only (an Inf/NaN scale is outside the contract)
    sc = rng.integers(0, 0x7C00, nb).astype(np.uint16) | (rng.integers(0, 2, nb).astype(np.uint16) << 15)
    blk[:, 0:2] = sc.view(np.uint8).reshape(nb, 2)
    a = oracle.dequant_q8_0(blk, nb * 32)
    b = oracle.ref_dequant_q8_0(blk, nb * 32)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_quantiser_contract(oracle):
    """Source contract of f32_to_q8_k (src/q4_rocm.cu:7221-7238) and its edge cases."""
    x = oracle.normal(11, 0, 32 * 4096)
    x[:32] = 0.0                                  # all-zero block -> scale 0, codes 0
    x[32:64] = np.float32(1e-9) * np.arange(32)   # d underflows fp16, codes still from fp32 d
    x[64:96] = 0.0
    x[64] = -3.0                                  # -amax -> -127, never -128
    b = oracle.quant_q8_0(x).reshape(-1, 34)
    sc = b[:, :2].copy().view(np.uint16).reshape(-1)
    codes = b[:, 2:].view(np.int8)
    assert sc[0] == 0 and not codes[0].any()
    assert sc[1] == 0 and codes[1].max() == 127
    assert codes[2][0] == -127 and codes.min() >= -127
    xb = x.reshape(-1, 32)
    amax = np.abs(xb).max(1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        idv = np.where(d > 0, np.float32(1.0) / d, np.float32(0)).astype(np.float32)
    want = np.clip(np.rint((xb * idv[:, None]).astype(np.float32)), -127, 127).astype(np.int8)
    assert np.array_equal(codes, want)
    assert np.array_equal(sc, d.astype(np.float16).view(np.uint16))
    # round trip through the reference's own dequantiser: |x - dq| <= d/2 + fp16 rounding of d
    if oracle.ref_lib() is not None:
        dq = oracle.ref_dequant_q8_0(b, x.size).reshape(-1, 32)
        dh = sc.view(np.float16).astype(np.float32)
        ok = np.abs(xb - dq) <= (0.5 * d + 127 * np.abs(dh - d) + 1e-12)[:, None]
        assert ok[2:].all()


def test_quantiser_matches_the_reference_source_compiled_in_place(oracle):
    """q4o_quant_q8_0 against the reference's own quantiser -- the body of f32_to_q8_k cut out of
    src/q4_rocm.cu:7221-7238 at build time and compiled for the host (oracle/Makefile, ref_quant_shim.c) --
    bit for bit on 2 Mi blocks of N(0,1) values at several magnitudes and on the edge cases: all-zero blocks,
    scales below the fp16 range, +-amax, ties of rint at .5, fp16 scale overflow to infinity."""
    if oracle.ref_quant_lib() is None:
        pytest.skip("oracle/_ref/libq4refquant.so not built (no reference tree)")
    rng = np.random.default_rng(2026)
    n_blocks = 1 << 21
    x = rng.standard_normal(n_blocks * 32, dtype=np.float32)
    x.reshape(-1, 32)[1::4] *= np.float32(1e-3)
    x.reshape(-1, 32)[2::4] *= np.float32(37.0)
    x.reshape(-1, 32)[3::4] *= rng.uniform(0, 50, (n_blocks // 4, 1)).astype(np.float32)
    e = x[:32 * 16].reshape(16, 32)
    e[0] = 0.0
    e[1] = np.float32(1e-9) * np.arange(32)
    e[2] = 0.0; e[2, 5] = -3.0
    e[3] = np.float32(1e-40)                                   # denormal inputs
    e[4] = np.arange(32, dtype=np.float32) - 15.5              # x * id lands on .5 ties
    e[5] = 127.0; e[5, 1:] = np.arange(31, dtype=np.float32) + 0.5
    e[6] = np.float32(9e6)                                     # d = 70866 > fp16 max: scale rounds to infinity
    e[7] = np.float32(-65504.0 * 127.0)
    e[8] = np.float32(2.0 ** -24 * 127.0)                      # d is the smallest fp16 denormal
    e[9] = np.float32(2.0 ** -25 * 127.0)                      # d halfway to it: ties to even -> 0
    got = oracle.quant_q8_0(x)
    want = oracle.ref_quant_q8_0(x)
    assert got.shape == want.shape
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, "first differing byte %d (block %d)" % (bad[0], bad[0] // 34)


def test_rope_and_prep(oracle):
    hd, n_rot, base = 128, 128, 1e7
    x = oracle.normal(5, 1, hd)
    y = oracle.rope(x, n_rot, 4095, base)
    p = np.arange(hd // 2)
    ang = np.float32(4095) * np.power(np.float32(base), -(p.astype(np.float32)) / np.float32(hd // 2)).astype(np.float32)
    c, s = np.cos(ang.astype(np.float64)), np.sin(ang.astype(np.float64))
    want = np.empty(hd)
    want[0::2] = x[0::2] * c - x[1::2] * s
    want[1::2] = x[0::2] * s + x[1::2] * c
    assert np.abs(y - want).max() < 2e-3   # fp32 angle of ~4e3 rad carries ~2e-4 of rounding
    # rotation preserves pair norms; partial rotary leaves the tail untouched
    y2 = oracle.rope(x, 64, 17, base)
    assert np.array_equal(y2[64:], x[64:])
    assert np.allclose(y2[0:64:2] ** 2 + y2[1:64:2] ** 2, x[0:64:2] ** 2 + x[1:64:2] ** 2, rtol=1e-5)
    qg = oracle.normal(5, 2, 2 * 4 * 2 * hd)
    wn = (1 + 0.1 * oracle.normal(5, 3, hd)).astype(np.float32)
    q, g = oracle.q_prep(qg, wn, 4, hd, 64, 9, base, 1e-6)
    src = qg.reshape(2, 4, 2, hd)
    assert np.array_equal(g, src[:, :, 1])
    nrm = src[0, 1, 0] / np.sqrt((src[0, 1, 0].astype(np.float64) ** 2).mean() + 1e-6) * wn
    assert np.allclose(q[0, 1, 64:], nrm[64:], rtol=1e-5, atol=1e-6)


def test_select_recipe(oracle):
    s = oracle.select(2, 0, 262144)
    assert s.shape == (2051,) and (np.diff(s) > 0).all()
    assert list(s[:4]) == [0, 1, 2, 3] and s[-1] == 262143 and s[-1024] == 262144 - 1024
    assert ((s[4:1027] >= 4) & (s[4:1027] < 262144 - 1024)).all()
    assert not np.array_equal(s, oracle.select(2, 1, 262144))
    t = oracle.select(2, 0, 1500)
    assert (t[:1500] == np.arange(1500)).all() and (t[1500:] == -1).all()
    u = oracle.select(2, 0, 2051)
    assert (u == np.arange(2051)).all()
    w = oracle.select(2, 0, 2052)   # smallest ctx with a real draw: 1023 of 1024 middle positions
    assert len(set(w.tolist())) == 2051 and w.min() == 0 and w.max() == 2051


def test_partials_merge_equals_full(oracle):
    n_head, n_kvh, hd, n = 16, 2, 128, 700
    k = oracle.normal(9, 0, n * n_kvh * hd)
    v = oracle.normal(9, 1, n * n_kvh * hd)
    q = oracle.normal(9, 2, n_head * hd)
    scale = 1 / np.sqrt(hd)
    for kind in (0, 1, 2):
        kc, vc = oracle.kv_write(k, kind), oracle.kv_write(v, kind)
        full = oracle.attn(q, kc, vc, None, n_head, n_kvh, hd, 1, n - 1, n, scale, kind)[0]
        cuts = [0, 1, 130, 130, 512, 700]     # includes an empty slice
        parts = np.stack([oracle.attn_partial(q, kc, vc, n_head, n_kvh, hd, scale, kind, a, b)
                          for a, b in zip(cuts[:-1], cuts[1:])])
        got = oracle.lse_merge(parts, n_head, hd)
        assert np.abs(got - full).max() < 2e-6
        f64 = oracle.attn(q, kc, vc, None, n_head, n_kvh, hd, 1, n - 1, n, scale, kind, acc64=True)[0]
        assert np.abs(f64 - full).max() < 5e-6


def test_indexed_padding_and_all_masked(oracle):
    n_head, n_kvh, hd, n = 4, 2, 64, 90
    k = oracle.normal(4, 0, n * n_kvh * hd)
    v = oracle.normal(4, 1, n * n_kvh * hd)
    q = oracle.normal(4, 2, n_head * hd)
    kc, vc = oracle.kv_write(k, 2), oracle.kv_write(v, 2)
    idx = np.full((2, 40), -1, np.int32)
    idx[0, :33] = np.arange(0, 66, 2)
    idx[1, 5:12] = [3, 9, 27, 81, 82, 83, 89]
    out = oracle.attn(q, kc, vc, None, n_head, n_kvh, hd, 1, 0, n, 0.125, 2, idx=idx, width=40,
                      idx_kvh_stride=40)[0]
    # same thing via dense attention over compacted caches
    for kh in range(2):
        sel = idx[kh][idx[kh] >= 0]
        kk = k.reshape(n, n_kvh, hd)[sel][:, kh:kh + 1]
        vv = v.reshape(n, n_kvh, hd)[sel][:, kh:kh + 1]
        o = oracle.attn(q.reshape(n_head, hd)[2 * kh:2 * kh + 2], oracle.kv_write(kk, 2),
                        oracle.kv_write(vv, 2), None, 2, 1, hd, 1, len(sel) - 1, len(sel), 0.125, 2)[0]
        assert np.array_equal(o, out[2 * kh:2 * kh + 2])
    shared = oracle.attn(q, kc, vc, None, n_head, n_kvh, hd, 1, 0, n, 0.125, 2, idx=idx[0], width=40)[0]
    assert np.array_equal(shared[:2], out[:2])
    dead = np.full(40, -1, np.int32)
    z = oracle.attn(q, kc, vc, None, n_head, n_kvh, hd, 1, 0, n, 0.125, 2, idx=dead, width=40)[0]
    assert not z.any()


# ------------------------------------------------------------------------------ QSA indexer
def _ix_case(oracle, seed, n_tok, n_head=4, ratio=4):
    raw = oracle.f32_to_f16(oracle.normal(seed, 0, n_tok * 128).reshape(n_tok, 128))
    wn = 1.0 + 0.1 * oracle.normal(seed, 1, 128)
    q = oracle.normal(seed, 2, n_head * 128).reshape(1, n_head, 128)
    return raw, wn.astype(np.float32), q


def test_indexer_pool_and_score_match_float64(oracle):
    """qsa_pool_k / qsa_score_k restatements against a float64 evaluation of the same formulas"""
    n_tok, ratio, n_rot, base, eps = 1027, 4, 64, 1e7, 1e-6
    raw, wn, q = _ix_case(oracle, 41, n_tok)
    nb = n_tok // ratio
    pool = oracle.ix_pool(raw, wn, ratio, 0, nb, n_rot, base, eps)
    x = raw[:nb * ratio].view(np.float16).reshape(nb, ratio, 128).astype(np.float64)
    v = x.mean(axis=1)
    v = v / np.sqrt((v * v).mean(axis=1, keepdims=True) + eps) * wn
    ref = v.copy()
    p = np.arange(n_rot // 2)
    freq = base ** (-p / (n_rot // 2))
    ang = (np.arange(nb) * ratio)[:, None].astype(np.float64) * freq[None, :]
    ref[:, 0:n_rot:2] = v[:, 0:n_rot:2] * np.cos(ang) - v[:, 1:n_rot:2] * np.sin(ang)
    ref[:, 1:n_rot:2] = v[:, 0:n_rot:2] * np.sin(ang) + v[:, 1:n_rot:2] * np.cos(ang)
    assert np.abs(pool - ref).max() < 2e-3          # fp32 angles at positions ~1e3
    assert np.abs(pool[:8] - ref[:8]).max() < 1e-5
    pos = n_tok - 1
    score = oracle.ix_score(q, pool, 1, nb + 3, nb + 8, 4, pos, ratio)
    want = np.maximum(pool.astype(np.float64) @ q[0].astype(np.float64).T, 0).sum(axis=1)
    n_vis = (pos + 1) // ratio
    assert np.allclose(score[0, :n_vis], want[:n_vis], rtol=1e-5, atol=1e-4)
    assert (score[0, n_vis:nb + 3] == np.float32(-1e30)).all()


def _topk_reference(row, n_vis, need, ratio, pos, width):
    """independent statement of the selection: sort by (score desc, index asc), keep `need`, emit above-threshold
    blocks in index order, then threshold ties in index order"""
    order = sorted(range(n_vis), key=lambda b: (-float(row[b]), b))[:need]
    thr = row[order[-1]]
    above = sorted(b for b in order if row[b] > thr)
    ties = sorted(b for b in order if row[b] == thr)
    sel = [b * ratio + j for b in above + ties for j in range(ratio)]
    sel += list(range(n_vis * ratio, pos + 1))
    sel = sel[:width] + [-1] * max(0, width - len(sel))
    return np.array(sel, np.int32)


@pytest.mark.parametrize("n_tok,k_blk,width", [(4099, 512, 2051), (1500, 512, 2051), (2051, 512, 2051), (2052, 512, 2051),
                                                (300, 16, 67), (70, 16, 67)])
def test_indexer_topk_order_and_ties(oracle, n_tok, k_blk, width):
    """qsa_topk_k restatement: exact set, the reference's emit order, ties at the threshold broken by index
    (relu makes exact zeros, and quantised scores make plenty of ties), dense prefix when every block fits"""
    ratio, pos = 4, n_tok - 1
    n_vis = (pos + 1) // ratio
    rng = np.random.default_rng(n_tok)
    for trial in range(3):
        row = np.maximum(rng.standard_normal(n_vis + 5), 0).astype(np.float32)        # many exact zeros
        if trial == 1:
            row = np.round(row * 4) / 4                                                # heavy ties everywhere
        if trial == 2:
            row[:] = 1.0                                                               # all equal
        sel = oracle.ix_topk(row[None, :], 1, n_vis + 5, k_blk, ratio, pos, width)[0]
        need = min(n_vis, k_blk)
        if need == n_vis:
            want = np.array([w if w <= pos else -1 for w in range(width)], np.int32)
        else:
            want = _topk_reference(row, n_vis, need, ratio, pos, width)
        assert np.array_equal(sel, want)
