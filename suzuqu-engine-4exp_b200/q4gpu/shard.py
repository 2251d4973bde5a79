"""Host-side partitioning for one 8-GPU box (one process per GPU).

Two modes, as the engine would use them:
 * concurrent sessions: whole sessions are assigned to ranks, no data-path collective;
 * one long sequence: contiguous, even row ranges per rank; each rank produces per-head
   (m, l, acc) records over its rows and the records are all-gathered (8 320 bytes per rank at
   16 heads x hd 128) before the merge (the multi-GPU form of the split-KV merge,
   src/q4_rocm.cu:6968-7012).
The transport is torch.distributed (NCCL over NVLink for CUDA tensors, gloo for CPU tensors in
tests); the arithmetic on either side of it is the library's.
"""


def sessions_for_rank(n_sessions, rank, world):
    """round-robin: session i lives on rank i % world (compute per session is constant at 2051
    positions, so round-robin balances the step; memory balance is within one session)"""
    return [i for i in range(n_sessions) if i % world == rank]


def rows_for_rank(ctx, rank, world):
    """[begin, end) of the rows rank owns: even contiguous split, the remainder spread over the first ranks"""
    base, rem = divmod(ctx, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def owner_of_row(pos, ctx, world):
    """rank whose shard holds row pos (the rank an append at pos goes to)"""
    base, rem = divmod(ctx, world)
    edge = rem * (base + 1)
    return pos // (base + 1) if pos < edge else rem + (pos - edge) // max(base, 1)


def exchange_records(part, group=None):
    """all-gather one [n_head][hd+2] record tensor per rank -> [world][n_head][hd+2] on every rank"""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    part = part.contiguous()
    flat = torch.empty((world * part.shape[0],) + tuple(part.shape[1:]), dtype=part.dtype, device=part.device)
    dist.all_gather_into_tensor(flat, part, group=group)
    return flat.view((world,) + tuple(part.shape))
