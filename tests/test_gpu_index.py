"""QSA indexer through the reference's entry points (q4_hip_qsa_pool / score / topk and their
device-position forms) against the oracle: pooled keys within fp32 libm tolerance (rsqrt, cos, sin
differ in the last bits between libm and the device), scores bit-exact on the same pool bytes, the
selection lists exactly equal -- including ties at the threshold, all-equal rows, the dense-prefix
case, a 65 536-block row (ctx 262 144) and several tokens per call."""
import numpy as np
import pytest
import torch

from gpu_util import dev, host, lib

pytestmark = pytest.mark.gpu

RATIO, N_ROT, BASE, EPS = 4, 64, 1e7, 1e-6


def make(oracle, seed, n_tok, n_head=4):
    raw = oracle.f32_to_f16(oracle.normal(seed, 0, n_tok * 128).reshape(n_tok, 128))
    wn = (1.0 + 0.1 * oracle.normal(seed, 1, 128)).astype(np.float32)
    return raw, wn


@pytest.mark.parametrize("n_tok", [4, 37, 4099])
def test_pool_matches_oracle(oracle, n_tok):
    L = lib()
    raw, wn = make(oracle, 50 + n_tok, n_tok)
    nb = n_tok // RATIO
    want = oracle.ix_pool(raw, wn, RATIO, 0, nb, N_ROT, BASE, EPS)
    d_raw = torch.from_numpy(raw.view(np.int16)).cuda()
    d_pool = torch.zeros(nb + 1, 128, device="cuda")
    # in two pieces, as a chunked prefill would
    mid = nb // 2
    if mid:
        assert L.q4_hip_qsa_pool(d_raw.data_ptr(), d_pool.data_ptr(), dev(wn).data_ptr(), 128, RATIO, 0, mid, N_ROT, BASE, EPS)
    assert L.q4_hip_qsa_pool(d_raw.data_ptr(), d_pool.data_ptr(), dev(wn).data_ptr(), 128, RATIO, mid, nb, N_ROT, BASE, EPS)
    got = host(d_pool)
    assert np.abs(got[:nb] - want).max() < 2e-3
    assert np.abs(got[:min(nb, 8)] - want[:min(nb, 8)]).max() < 2e-6
    assert (got[nb] == 0).all()
    # no weight: plain RMSNorm
    assert L.q4_hip_qsa_pool(d_raw.data_ptr(), d_pool.data_ptr(), None, 128, RATIO, 0, nb, N_ROT, BASE, EPS)
    assert np.abs(host(d_pool)[:nb] - oracle.ix_pool(raw, None, RATIO, 0, nb, N_ROT, BASE, EPS)).max() < 2e-3
    assert not L.q4_hip_qsa_pool(d_raw.data_ptr(), d_pool.data_ptr(), None, 64, RATIO, 0, nb, N_ROT, BASE, EPS)


def test_pool_d_completes_a_block_only_on_its_last_token(oracle):
    L = lib()
    n_tok = 23
    raw, wn = make(oracle, 61, n_tok)
    d_raw = torch.from_numpy(raw.view(np.int16)).cuda()
    d_pool = torch.zeros(n_tok // RATIO + 1, 128, device="cuda")
    want = oracle.ix_pool(raw, wn, RATIO, 0, n_tok // RATIO, N_ROT, BASE, EPS)
    for pos in range(n_tok):
        L.q4_hip_pos_push(pos)
        assert L.q4_hip_qsa_pool_d(d_raw.data_ptr(), d_pool.data_ptr(), dev(wn).data_ptr(), 128, RATIO, N_ROT, BASE, EPS)
        got = host(d_pool)
        done = (pos + 1) // RATIO
        assert np.abs(got[:done] - want[:done]).max() < 1e-5 if done else True
        assert (got[done:] == 0).all()


@pytest.mark.parametrize("n_head,n_tok,pos0", [(4, 1, 4098), (1, 1, 99), (3, 5, 700), (4, 3, 262141)])
def test_score_bit_exact_and_topk_exact(oracle, n_head, n_tok, pos0):
    """same pool bytes in, identical scores out (the dot product is one fused multiply-add per dim, in
    dim order); identical lists out"""
    L = lib()
    n_all = pos0 + n_tok
    nb = n_all // RATIO
    stride = nb + 7
    rng = np.random.default_rng(pos0)
    pool = rng.standard_normal((nb, 128)).astype(np.float32)
    q = rng.standard_normal((n_tok, n_head, 128)).astype(np.float32)
    want = oracle.ix_score(q, pool, n_tok, nb, stride, n_head, pos0, RATIO)
    d_score = torch.full((n_tok, stride), 7.0, device="cuda")
    assert L.q4_hip_qsa_score(dev(q).data_ptr(), dev(pool).data_ptr(), d_score.data_ptr(), n_tok, nb, stride, n_head, 128, pos0, RATIO)
    got = host(d_score)
    assert np.array_equal(got[:, :nb].view(np.uint32), want[:, :nb].view(np.uint32))
    assert (got[:, nb:] == 7.0).all()
    width, k_blk = 2051, 512
    d_sel = torch.zeros(n_tok, width, dtype=torch.int32, device="cuda")
    assert L.q4_hip_qsa_topk(d_score.data_ptr(), d_sel.data_ptr(), n_tok, nb, stride, k_blk, RATIO, pos0, width)
    want_sel = oracle.ix_topk(want, n_tok, stride, k_blk, RATIO, pos0, width)
    assert np.array_equal(host(d_sel), want_sel)


@pytest.mark.parametrize("n_tok,k_blk,width", [(4099, 512, 2051), (2051, 512, 2051), (2052, 512, 2051), (300, 16, 67),
                                                (70, 16, 67), (262144, 512, 2051)])
def test_topk_ties_and_degenerate_rows(oracle, n_tok, k_blk, width):
    L = lib()
    pos = n_tok - 1
    n_vis = (pos + 1) // RATIO
    stride = n_vis + 5
    rng = np.random.default_rng(n_tok)
    rows = [np.maximum(rng.standard_normal(stride), 0), np.round(np.maximum(rng.standard_normal(stride), 0) * 4) / 4,
            np.ones(stride), -np.abs(rng.standard_normal(stride)), np.where(np.arange(stride) % 3 == 0, 2.0, -1e30)]
    for i, row in enumerate(rows):
        row = row.astype(np.float32)[None, :]
        d_sel = torch.zeros(1, width, dtype=torch.int32, device="cuda")
        assert L.q4_hip_qsa_topk(dev(row).data_ptr(), d_sel.data_ptr(), 1, n_vis, stride, k_blk, RATIO, pos, width)
        want = oracle.ix_topk(row, 1, stride, k_blk, RATIO, pos, width)
        assert np.array_equal(host(d_sel), want), "row kind %d" % i


def test_device_position_forms_feed_the_sparse_decode(oracle):
    """score_d + topk_d at the position word == the host-position forms; the list is a valid input of the
    decode kernel (all entries <= pos or -1, no duplicates)"""
    L = lib()
    pos, n_head = 9001, 4
    nb = (pos + 1) // RATIO
    max_blocks = 4096
    rng = np.random.default_rng(7)
    pool = rng.standard_normal((max_blocks, 128)).astype(np.float32)
    q = rng.standard_normal((1, n_head, 128)).astype(np.float32)
    d_pool, d_q = dev(pool), dev(q)
    a_score, b_score = torch.zeros(1, max_blocks, device="cuda"), torch.zeros(1, max_blocks, device="cuda")
    a_sel = torch.zeros(2051, dtype=torch.int32, device="cuda")
    b_sel = torch.zeros_like(a_sel)
    assert L.q4_hip_qsa_score(d_q.data_ptr(), d_pool.data_ptr(), a_score.data_ptr(), 1, nb, max_blocks, n_head, 128, pos, RATIO)
    assert L.q4_hip_qsa_topk(a_score.data_ptr(), a_sel.data_ptr(), 1, nb, max_blocks, 512, RATIO, pos, 2051)
    L.q4_hip_pos_push(pos)
    assert L.q4_hip_qsa_score_d(d_q.data_ptr(), d_pool.data_ptr(), b_score.data_ptr(), max_blocks, n_head, 128, RATIO)
    assert L.q4_hip_qsa_topk_d(b_score.data_ptr(), b_sel.data_ptr(), max_blocks, 512, RATIO, 2051)
    assert np.array_equal(host(a_score)[0, :nb], host(b_score)[0, :nb])
    sel = host(b_sel)
    assert np.array_equal(sel, host(a_sel))
    live = sel[sel >= 0]
    assert live.max() <= pos and len(np.unique(live)) == len(live) == 2048 + (pos + 1) % RATIO
    assert L.q4_gpu_last_error() == 0


def test_batched_sessions_select_like_single_sessions(oracle):
    """q4_gpu_qsa_select_batch: every session has its own pool and position; scores bit-equal and lists
    equal to the oracle's per-session result (short rows, the dense-prefix case and a long row together)"""
    L = lib()
    n_head, width, k_blk = 4, 2051, 512
    positions = [4098, 99, 70001, 2050, 20000]          # 99 and 2050: every block fits (dense prefix)
    stride = max(p + 1 for p in positions) // RATIO + 3
    rng = np.random.default_rng(77)
    pools, d_pools, want_sc, want_sel = [], [], [], []
    q = rng.standard_normal((len(positions), n_head, 128)).astype(np.float32)
    for s_i, pos in enumerate(positions):
        nb = (pos + 1) // RATIO
        pool = rng.standard_normal((max(nb, 1), 128)).astype(np.float32)
        d_pools.append(dev(pool))
        sc = oracle.ix_score(q[s_i:s_i + 1], pool, 1, nb, stride, n_head, pos, RATIO)
        want_sc.append(sc)
        want_sel.append(oracle.ix_topk(sc, 1, stride, k_blk, RATIO, pos, width))
    ptrs = torch.tensor([t.data_ptr() for t in d_pools], dtype=torch.int64, device="cuda")
    d_pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    d_score = torch.zeros(len(positions), stride, device="cuda")
    d_sel = torch.zeros(len(positions), width, dtype=torch.int32, device="cuda")
    assert L.q4_gpu_qsa_select_batch(ptrs.data_ptr(), d_pos.data_ptr(), dev(q).data_ptr(), d_score.data_ptr(),
                                     d_sel.data_ptr(), len(positions), stride, n_head, 128, k_blk, RATIO, width)
    got_sc, got_sel = host(d_score), host(d_sel)
    for s_i, pos in enumerate(positions):
        nb = (pos + 1) // RATIO
        assert np.array_equal(got_sc[s_i, :nb].view(np.uint32), want_sc[s_i][0, :nb].view(np.uint32)), s_i
        assert np.array_equal(got_sel[s_i], want_sel[s_i][0]), s_i
    assert not L.q4_gpu_qsa_select_batch(None, d_pos.data_ptr(), dev(q).data_ptr(), d_score.data_ptr(), d_sel.data_ptr(),
                                         len(positions), stride, n_head, 128, k_blk, RATIO, width)
    L.q4_gpu_last_error()


def test_argument_checks():
    L = lib()
    z = torch.zeros(256, device="cuda")
    s = torch.zeros(64, dtype=torch.int32, device="cuda")
    assert not L.q4_hip_qsa_score(z.data_ptr(), z.data_ptr(), z.data_ptr(), 1, 1, 1, 5, 128, 3, 4)     # > 4 heads
    assert not L.q4_hip_qsa_score(z.data_ptr(), z.data_ptr(), z.data_ptr(), 1, 1, 1, 4, 64, 3, 4)      # hd != 128
    assert not L.q4_hip_qsa_topk(z.data_ptr(), s.data_ptr(), 1, 1, 1, 513, 4, 3, 64)                   # k_blk > 512
    assert not L.q4_hip_qsa_topk(None, s.data_ptr(), 1, 1, 1, 16, 4, 3, 64)
