"""Worker of tests/test_gpu_xchg_multi.py: one rank of a sequence-sharded decode with the exchange inside
the kernel, on its own GPU.  Launched by torch.distributed.run; prints one line per check and exits
non-zero on the first failure.  The processes exchange only the 64-byte window handles (gloo)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "suzuqu-engine-4exp_b200"))
sys.path.insert(0, HERE)

import q4gpu                                    # noqa: E402
from oracle import q4_oracle as oracle          # noqa: E402
from q4gpu import shard                         # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    L = q4gpu.init()
    q4gpu.use_torch_stream()
    n_head, n_kvh, hd, ctx, kind = 16, 2, 128, 6000 + 13 * world, 2
    kvw = n_kvh * hd
    k = oracle.normal(777, 0, ctx * kvw).reshape(ctx, kvw)
    v = oracle.normal(777, 1, ctx * kvw).reshape(ctx, kvw)
    kc, vc = oracle.kv_write(k, kind), oracle.kv_write(v, kind)
    b, e = shard.rows_for_rank(ctx, rank, world)
    st = q4gpu.KVStore(1, n_kvh, hd, e - b, kind)
    st.append(0, torch.from_numpy(k[b:e]).cuda(), torch.from_numpy(v[b:e]).cuda(), 0, e - b)
    x = q4gpu.Exchange(rank, world, n_head, n_kvh, hd)
    x.attach_all(dist)
    out = torch.zeros(n_head * hd, device="cuda")
    scale = 1.0 / np.sqrt(hd)
    for call in range(6):
        q = oracle.normal(778, call, n_head * hd).reshape(n_head, hd)
        gate = oracle.normal(779, call, n_head * hd) if call % 2 else None
        x.decode(st, 0, torch.from_numpy(q).cuda(), out, scale, e - b,
                 gate=None if gate is None else torch.from_numpy(gate).cuda())
        torch.cuda.synchronize()
        ref = oracle.attn(q, kc, vc, gate, n_head, n_kvh, hd, 1, ctx - 1, ctx, scale, kind)[0].reshape(-1)
        err = np.abs(out.cpu().numpy() - ref)
        ok = bool((err <= 2e-3 + 1e-3 * np.abs(ref)).all())
        print("rank %d call %d max err %.2e %s" % (rank, call, err.max(), "ok" if ok else "FAIL"), flush=True)
        if not ok:
            sys.exit(1)
    assert L.q4_gpu_last_error() == 0
    # ---- the collective form: the library's own NCCL communicator from a unique id handed over by the host
    # (here: broadcast over the gloo group), all-gather of the ranks' records + merge, against the oracle
    comm = q4gpu.Comm(rank, world, dist)
    part = torch.empty(n_head, hd + 2, device="cuda")
    parts = torch.empty(world, n_head, hd + 2, device="cuda")
    for call in range(2):
        q = oracle.normal(780, call, n_head * hd).reshape(n_head, hd)
        gate = oracle.normal(781, call, n_head * hd) if call else None
        st.decode_partial(0, torch.from_numpy(q).cuda(), part, n_head, scale, n_kv=e - b)
        comm.allgather_merge(part, parts, n_head, hd, out, gate=None if gate is None else torch.from_numpy(gate).cuda())
        torch.cuda.synchronize()
        ref = oracle.attn(q, kc, vc, gate, n_head, n_kvh, hd, 1, ctx - 1, ctx, scale, kind)[0].reshape(-1)
        err = np.abs(out.cpu().numpy() - ref)
        ok = bool((err <= 2e-3 + 1e-3 * np.abs(ref)).all())
        print("rank %d comm call %d max err %.2e %s" % (rank, call, err.max(), "ok" if ok else "FAIL"), flush=True)
        if not ok:
            sys.exit(1)
    comm.close()
    assert L.q4_gpu_last_error() == 0
    # ---- a peer that stops calling (between steps, nothing in flight): the others' bounded wait runs
    # out, they get status bit 32 and their own part, and keep working
    dist.barrier()
    if os.environ.get("Q4_XCHG_TEST_DROPOUT") == "1":
        x.set_timeout_ms(100)
        if rank != world - 1:
            q = oracle.normal(778, 99, n_head * hd).reshape(n_head, hd)
            x.decode(st, 0, torch.from_numpy(q).cuda(), out, scale, e - b)
            torch.cuda.synchronize()
            status = L.q4_gpu_last_error()
            own = torch.zeros_like(out)
            st.decode(0, torch.from_numpy(q).cuda(), own, n_head, scale, n_kv=e - b)
            torch.cuda.synchronize()
            same = bool(torch.allclose(out, own, atol=2e-3, rtol=1e-3))
            print("rank %d dropout: status %#x own-part %s" % (rank, status, "ok" if same else "FAIL"), flush=True)
            if status != 32 or not same or L.q4_gpu_last_error() != 0:
                sys.exit(1)
        dist.barrier()
    x.close()
    st.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
