"""Data-parallel sharding of the WKV7 path over the GPUs of one node.

Every (sequence, head) pair is independent in all operators of this package, so work is split with no collective
on the data path: rank `i` of `n` owns a contiguous block of sequences (or of heads, when there are fewer
sequences than ranks) together with the matching slice of the state pool.  A collective (all-gather over
NCCL/NVLink) runs only when the caller asks for the outputs or final states of all shards on every rank.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(total: int, world_size: int, rank: int) -> tuple[int, int]:
    """Contiguous [begin, end) block of `total` items owned by `rank` (earlier ranks take the remainder)."""
    if not 0 <= rank < world_size:
        raise ValueError("rank must be in [0, world_size)")
    base, extra = divmod(total, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_plan(num_sequences: int, num_heads: int, world_size: int, rank: int) -> dict:
    """Which sequences and heads this rank computes: sequences are split first, heads when B < world_size."""
    if num_sequences >= world_size:
        s0, s1 = shard_range(num_sequences, world_size, rank)
        return {"sequences": (s0, s1), "heads": (0, num_heads), "axis": "sequence"}
    if num_heads % world_size and num_heads < world_size:
        raise ValueError("fewer (sequence, head) blocks than ranks")
    h0, h1 = shard_range(num_heads, world_size, rank)
    return {"sequences": (0, num_sequences), "heads": (h0, h1), "axis": "head"}


def shard_packed(tokens: torch.Tensor, cu_seqlens: torch.Tensor, plan: dict):
    """Slice packed `[N,H,D]` tokens and their offsets for a plan; returns (tokens, cu_seqlens) of the shard."""
    s0, s1 = plan["sequences"]
    h0, h1 = plan["heads"]
    cu = cu_seqlens.tolist()
    part = tokens[cu[s0]:cu[s1], h0:h1].contiguous()
    local_cu = (cu_seqlens[s0:s1 + 1] - cu_seqlens[s0]).to(torch.int32).contiguous()
    return part, local_cu


def gather_shards(local: torch.Tensor, plan: dict, group=None, total: int | None = None) -> torch.Tensor:
    """All-gather per-rank results (outputs `[n_local,H_local,D]` or states `[B_local,H_local,D,D]`) so that every
    rank holds the full tensor.  Shards may have different sizes along the split axis.

    `total` is the size of the split axis before sharding (sequences, or packed tokens of equal-length sequences,
    or heads).  When it is given the shard sizes follow from `shard_range` on every rank and equal shards go
    through one `all_gather_into_tensor`; without it the sizes are exchanged first, which costs a second
    collective and a host synchronisation."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    dim = 0 if plan["axis"] == "sequence" else 1
    if total is not None:
        sizes = [shard_range(total, world, r)[1] - shard_range(total, world, r)[0] for r in range(world)]
        if sizes[dist.get_rank(group)] != local.shape[dim]:
            raise ValueError("local shard does not match shard_range(total, world_size, rank)")
        if dim == 0 and len(set(sizes)) == 1:
            out = local.new_empty((total, *local.shape[1:]))
            dist.all_gather_into_tensor(out, local.contiguous(), group=group)
            return out
    else:
        sizes = [torch.zeros(1, dtype=torch.int64, device=local.device) for _ in range(world)]
        dist.all_gather(sizes, torch.tensor([local.shape[dim]], dtype=torch.int64, device=local.device), group=group)
        sizes = [int(s.item()) for s in sizes]
    biggest = max(sizes)
    pad_shape = list(local.shape)
    pad_shape[dim] = biggest
    padded = local.new_zeros(pad_shape)
    padded.narrow(dim, 0, local.shape[dim]).copy_(local)
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p.narrow(dim, 0, n) for p, n in zip(parts, sizes)], dim=dim)
