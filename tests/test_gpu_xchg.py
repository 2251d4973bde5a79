"""Sequence-sharded decode with the exchange inside the kernel (q4_gpu_xchg_*), on one GPU.

Kernels that wait on one another are never run as separate launches on one GPU, so the ranks of a
node are emulated in one process without any wait that a later launch would have to satisfy: every
rank first runs the push-only phase (attend + store the record into all windows), then every rank
runs the wait-and-merge phase, which finds all records already published.  The fused single-launch
phase is exercised where it cannot block: world size 1, and a peer that never publishes, where the
bounded wait runs out and reports it."""
import numpy as np
import pytest
import torch

import q4gpu
from gpu_util import assert_close, dev, host, lib
from test_gpu_decode import make_case

pytestmark = pytest.mark.gpu


def make_ranks(world, n_head, n_kvh, hd):
    xs = [q4gpu.Exchange(r, world, n_head, n_kvh, hd) for r in range(world)]
    for a in xs:
        for b in xs:
            if a is not b:
                a.attach_ptr(b.rank, b.window())
    return xs


@pytest.mark.parametrize("kind,world,n_head,n_kvh,hd", [(2, 2, 16, 2, 128), (2, 4, 16, 2, 128), (1, 3, 8, 2, 64),
                                                        (0, 2, 32, 2, 128), (2, 8, 4, 4, 32), (1, 2, 4, 1, 256)])
def test_emulated_ranks_match_whole_sequence(oracle, kind, world, n_head, n_kvh, hd):
    """world stores hold uneven slices of one sequence; push on every rank, then merge on every rank:
    each rank's output == attention over the whole sequence (oracle), for several calls in a row
    (both parities of the double-buffered slots, changing queries)."""
    L = lib()
    ctx = 3000 + 7 * world
    k, v, q0 = make_case(oracle, 9100 + kind + world, ctx, n_head, n_kvh, hd)
    scale = 1.0 / np.sqrt(hd)
    kc, vc = oracle.kv_write(k, kind), oracle.kv_write(v, kind)
    cuts = [0] + sorted(int(x) for x in np.random.default_rng(world).choice(np.arange(1, ctx), world - 1, replace=False)) + [ctx]
    stores = []
    for r in range(world):
        n = cuts[r + 1] - cuts[r]
        st = q4gpu.KVStore(1, n_kvh, hd, n, kind)
        st.append(0, dev(k[cuts[r]:cuts[r + 1]]), dev(v[cuts[r]:cuts[r + 1]]), 0, n)
        stores.append(st)
    xs = make_ranks(world, n_head, n_kvh, hd)
    outs = [torch.zeros(n_head * hd, device="cuda") for _ in range(world)]
    for call in range(5):
        q = (q0 * (1.0 + 0.25 * call)).astype(np.float32)
        gate = oracle.normal(77 + call, 3, n_head * hd) if call % 2 == 0 else None
        full = oracle.attn(q, kc, vc, gate, n_head, n_kvh, hd, 1, ctx - 1, ctx, scale, kind)[0]
        dq, dg = dev(q), (dev(gate) if gate is not None else None)
        for r in range(world):
            xs[r].decode(stores[r], 0, dq, outs[r], scale, cuts[r + 1] - cuts[r], gate=dg, phase=q4gpu.Exchange.PUSH)
        for r in range(world):
            xs[r].decode(None, 0, None, outs[r], scale, 0, gate=dg, phase=q4gpu.Exchange.MERGE)
        for r in range(world):
            assert_close(host(outs[r]).reshape(n_head, hd), full, "call %d rank %d" % (call, r))
    assert L.q4_gpu_last_error() == 0
    for o in xs + stores:
        o.close()


def test_world_of_one_is_plain_decode(oracle):
    """fused phase with no peers: nothing to wait for; equals q4_gpu_kv_decode"""
    L = lib()
    n_head, n_kvh, hd, ctx = 16, 2, 128, 5000
    k, v, q = make_case(oracle, 31, ctx, n_head, n_kvh, hd)
    st = q4gpu.KVStore(1, n_kvh, hd, ctx, 2)
    st.append(0, dev(k), dev(v), 0, ctx)
    x = q4gpu.Exchange(0, 1, n_head, n_kvh, hd)
    a, b = torch.zeros(n_head * hd, device="cuda"), torch.zeros(n_head * hd, device="cuda")
    for _ in range(3):
        x.decode(st, 0, dev(q), a, 0.1, ctx)
    st.decode(0, dev(q), b, n_head, 0.1, n_kv=ctx)
    assert_close(host(a), host(b), "world 1")
    assert L.q4_gpu_last_error() == 0
    x.close()
    st.close()


def test_missing_peer_times_out_and_reports(oracle):
    """A peer that never publishes: the bounded wait runs out (20 ms here), status bit 32 is set, the
    output is this rank's own part, and the library keeps working afterwards."""
    L = lib()
    n_head, n_kvh, hd, ctx = 16, 2, 128, 2048
    k, v, q = make_case(oracle, 32, ctx, n_head, n_kvh, hd)
    st = q4gpu.KVStore(1, n_kvh, hd, ctx, 2)
    st.append(0, dev(k), dev(v), 0, ctx)
    xs = make_ranks(2, n_head, n_kvh, hd)
    xs[0].set_timeout_ms(20)
    out, own = torch.zeros(n_head * hd, device="cuda"), torch.zeros(n_head * hd, device="cuda")
    xs[0].decode(st, 0, dev(q), out, 0.1, ctx)        # rank 1 never runs
    st.decode(0, dev(q), own, n_head, 0.1, n_kv=ctx)
    torch.cuda.synchronize()
    assert L.q4_gpu_last_error() == 32
    assert_close(host(out), host(own), "own part after the time limit")
    assert L.q4_gpu_last_error() == 0
    st.decode(0, dev(q), own, n_head, 0.1, n_kv=ctx)
    assert L.q4_gpu_last_error() == 0
    for o in xs + [st]:
        o.close()


def test_argument_checks():
    L = lib()
    assert not L.q4_gpu_xchg_create(0, 17, 16, 2, 128)
    assert not L.q4_gpu_xchg_create(2, 2, 16, 2, 128)
    assert not L.q4_gpu_xchg_create(0, 2, 16, 2, 96)
    assert L.q4_gpu_last_error() & 1
    x = q4gpu.Exchange(0, 2, 16, 2, 128)
    out = torch.zeros(16 * 128, device="cuda")
    # peer not attached yet
    assert not L.q4_gpu_kv_decode_xchg(None, x.h, 0, None, 0, None, out.data_ptr(), 0, 0.1, 2)
    assert L.q4_gpu_last_error() & 1
    x.close()


def test_library_communicator_on_one_rank(oracle):
    """q4_gpu_comm_* with a world of one (what a one-GPU box can run): unique id, communicator, all-gather of
    the single record + merge == the decode's own output; the multi-rank form runs in test_gpu_xchg_multi.py"""
    L = lib()
    n_head, n_kvh, hd, ctx = 16, 2, 128, 700
    k = oracle.normal(61, 0, ctx * n_kvh * hd).reshape(ctx, n_kvh * hd)
    v = oracle.normal(61, 1, ctx * n_kvh * hd).reshape(ctx, n_kvh * hd)
    q = oracle.normal(61, 2, n_head * hd)
    gate = oracle.normal(61, 3, n_head * hd)
    st = q4gpu.KVStore(1, n_kvh, hd, ctx, 2)
    st.append(0, dev(k), dev(v), 0, ctx)
    comm = q4gpu.Comm(0, 1)
    part = torch.empty(n_head, hd + 2, device="cuda")
    parts = torch.empty(1, n_head, hd + 2, device="cuda")
    out = torch.empty(n_head * hd, device="cuda")
    st.decode_partial(0, dev(q), part, n_head, 0.0884, n_kv=ctx)
    comm.allgather_merge(part, parts, n_head, hd, out, gate=dev(gate))
    ref = oracle.attn(q, oracle.kv_write(k, 2), oracle.kv_write(v, 2), gate, n_head, n_kvh, hd, 1, ctx - 1, ctx, 0.0884, 2)[0]
    assert_close(host(out).reshape(n_head, hd), ref, "collective form, world 1")
    assert torch.equal(parts[0], part)
    comm.close()
    assert not L.q4_gpu_comm_create(None, 0, 1) and L.q4_gpu_last_error() & 1
    st.close()
