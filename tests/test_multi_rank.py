"""The N > 1 host path on CPU: two gloo ranks shard one sequence by rows, build their records,
exchange them with the package's all-gather and merge -- equal to attention over the whole sequence;
and the session / row partitioning helpers."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from q4gpu import shard

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_partition_helpers():
    for world in (1, 2, 4, 8):
        seen = []
        for r in range(world):
            seen += shard.sessions_for_rank(64, r, world)
        assert sorted(seen) == list(range(64))
        for ctx in (262144, 1000, 7, 8, 9):
            edges = [shard.rows_for_rank(ctx, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == ctx
            assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
            sizes = [e - b for b, e in edges]
            assert max(sizes) - min(sizes) <= 1
            for pos in {0, ctx // 2, ctx - 1} | {b for b, _ in edges if b < ctx}:
                r = shard.owner_of_row(pos, ctx, world)
                assert edges[r][0] <= pos < edges[r][1]


def _rank_main(rank, world, port, q_out):
    sys.path.insert(0, ROOT)
    from oracle import q4_oracle as oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n_head, n_kvh, hd, ctx = 16, 2, 128, 1001
    kvw = n_kvh * hd
    k = oracle.normal(77, 0, ctx * kvw)
    v = oracle.normal(77, 1, ctx * kvw)
    q = oracle.normal(77, 2, n_head * hd)
    gate = oracle.normal(77, 3, n_head * hd)
    scale = 1.0 / np.sqrt(hd)
    kc, vc = oracle.kv_write(k, 2), oracle.kv_write(v, 2)
    b, e = shard.rows_for_rank(ctx, rank, world)
    part = oracle.attn_partial(q, kc, vc, n_head, n_kvh, hd, scale, 2, b, e)
    allp = shard.exchange_records(torch.from_numpy(part))
    out = oracle.lse_merge(allp.numpy(), n_head, hd, gate)
    full = oracle.attn(q, kc, vc, gate, n_head, n_kvh, hd, 1, ctx - 1, ctx, scale, 2)[0]
    q_out.put((rank, float(np.abs(out - full).max()), tuple(allp.shape)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sequence_shard_exchange_gloo():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q_out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, shape in res:
        assert shape == (2, 16, 130)
        assert err < 2e-6, (rank, err)
