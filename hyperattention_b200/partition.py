"""Partition of the (batch x heads) axis over the GPUs of one node.

Every stage of the path (hash, sort, attention, merge, the causal recursion) treats (batch, head) pairs independently
(the reference's recursion only folds more independent pseudo-heads, hyper_attention.py:67-69), so the multi-GPU
form of a call is: each rank owns a contiguous slice of the flattened batch*heads axis and no data-path collective
is needed.  torch.distributed is only used by callers for barriers / gathering results.
"""
import torch


def head_slice(n_units: int, rank: int, world: int) -> slice:
    """Contiguous slice of `n_units` (batch*heads) owned by `rank`; the first n_units % world ranks get one extra."""
    assert 0 <= rank < world and n_units >= 0
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def shard_heads(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """[B, H, n, d] -> this rank's [1, units, n, d] slice of the flattened (B*H) axis."""
    B, H = t.shape[:2]
    flat = t.reshape(1, B * H, *t.shape[2:])
    return flat[:, head_slice(B * H, rank, world)]


def gather_heads(local: torch.Tensor, shape, group=None) -> torch.Tensor:
    """Inverse of shard_heads across the process group (all ranks get the full tensor)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    B, H = shape[:2]
    sizes = [head_slice(B * H, r, world) for r in range(world)]
    parts = [torch.empty(1, s.stop - s.start, *local.shape[2:], dtype=local.dtype, device=local.device) for s in sizes]
    dist.all_gather(parts, local.contiguous(), group=group) if len({p.shape for p in parts}) == 1 else _uneven_gather(parts, local, group)
    return torch.cat(parts, dim=1).reshape(B, H, *local.shape[2:])


def _uneven_gather(parts, local, group):
    import torch.distributed as dist
    for r, buf in enumerate(parts):
        if r == dist.get_rank(group):
            buf.copy_(local)
        dist.broadcast(buf, src=r, group=group)
