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


# ------------------------------------------------------------------------------------------------
# Optional ingress for sequence-sharded inputs
# ------------------------------------------------------------------------------------------------
def seq_to_head_shards(x_local: torch.Tensor, group=None) -> torch.Tensor:
    """x_local [B, H, n/G, d] (this rank's contiguous slice of the sequence, all heads) -> [B, H/G, n, d] (this rank's
    heads, the whole sequence).  One all-to-all over the process group (NCCL over NVLink on GPUs, gloo on CPU); the data
    lands in this rank's own memory, the attention kernels never touch a peer's memory.  H must be divisible by the
    group size.  Preferred over gathering K/V whenever there are at least as many heads as ranks."""
    import torch.distributed as dist
    G = dist.get_world_size(group)
    B, H, m, d = x_local.shape
    assert H % G == 0, 'heads must be divisible by the number of ranks'
    send = x_local.reshape(B, G, H // G, m, d).permute(1, 0, 2, 3, 4).contiguous()      # [G, B, H/G, m, d]: block g -> rank g
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)                                      # recv[g] = rank g's sequence slice
    return recv.permute(1, 2, 0, 3, 4).reshape(B, H // G, G * m, d)


def head_to_seq_shards(o_local: torch.Tensor, group=None) -> torch.Tensor:
    """Inverse of seq_to_head_shards for outputs: [B, H/G, n, d] -> [B, H, n/G, d]."""
    import torch.distributed as dist
    G = dist.get_world_size(group)
    B, hl, n, d = o_local.shape
    assert n % G == 0
    send = o_local.reshape(B, hl, G, n // G, d).permute(2, 0, 1, 3, 4).contiguous()     # [G, B, H/G, n/G, d]
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)                                      # recv[g] = heads of rank g
    return recv.permute(1, 0, 2, 3, 4).reshape(B, G * hl, n // G, d)


def all_gather_sequence(x_local: torch.Tensor, group=None) -> torch.Tensor:
    """x_local [B, H, n/G, d] -> [B, H, n, d] on every rank (all-gather along the sequence): the fallback when there are
    fewer heads than ranks, e.g. for K and V of a multi-query layer."""
    import torch.distributed as dist
    G = dist.get_world_size(group)
    parts = [torch.empty_like(x_local) for _ in range(G)]
    dist.all_gather(parts, x_local.contiguous(), group=group)
    return torch.cat(parts, dim=2)
