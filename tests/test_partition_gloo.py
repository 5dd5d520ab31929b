"""The multi-GPU form of the path on CPU ranks (gloo, world_size 2): heads are partitioned, every rank runs the
oracle on its shard with no data-path collective, and the gathered result equals the single-process result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hyperattention_b200.partition import head_slice


def test_head_slice_covers_everything():
    for n, w in [(32, 8), (32, 4), (7, 3), (2, 4), (0, 2)]:
        seen = []
        for r in range(w):
            s = head_slice(n, r, w)
            seen += list(range(s.start, s.stop))
        assert seen == list(range(n))
    assert head_slice(32, 3, 8) == slice(12, 16)


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, causal, out_q):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from hyperattention_b200.partition import gather_heads, shard_heads
        from oracle import hyper_oracle as O
        torch.manual_seed(0)                          # same data on every rank, as bench.py generates it
        B, H, n, d = 1, 3, 512, 32                    # 3 heads over 2 ranks: uneven split
        q, k, v = [torch.randn(B, H, n, d) for _ in range(3)]
        proj = torch.randn(1, 1, d, 8)
        orc = O.HyperAttentionOracle(proj, 128, 128, 256, False)
        ql, kl, vl = [shard_heads(t, rank, world) for t in (q, k, v)]
        o_local, lse_local = orc(ql, kl, vl, causal=causal, return_lse=True)
        o = gather_heads(o_local, (B, H))
        lse = gather_heads(lse_local, (B, H))
        if rank == 0:
            o_ref, lse_ref = orc(q, k, v, causal=causal, return_lse=True)
            out_q.put((torch.equal(o, o_ref), torch.equal(lse, lse_ref), tuple(o.shape)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('causal', [False, True])
def test_sharded_equals_unsharded_on_two_gloo_ranks(causal):
    ctx = mp.get_context('spawn')
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, causal, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    same_o, same_lse, shape = out_q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert same_o and same_lse and shape == (1, 3, 512, 32)


def _seq_worker(rank, world, port, out_q):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from hyperattention_b200.partition import all_gather_sequence, head_to_seq_shards, seq_to_head_shards
        torch.manual_seed(0)
        B, H, n, d = 2, 4, 64, 8
        x = torch.randn(B, H, n, d)
        m = n // world
        x_local = x[:, :, rank * m:(rank + 1) * m].contiguous()                # sequence shard, all heads
        xh = seq_to_head_shards(x_local)                                       # head shard, whole sequence
        hl = H // world
        ok1 = torch.equal(xh, x[:, rank * hl:(rank + 1) * hl])
        back = head_to_seq_shards(xh)
        ok2 = torch.equal(back, x_local)
        ok3 = torch.equal(all_gather_sequence(x_local), x)
        res = torch.tensor([int(ok1), int(ok2), int(ok3)])
        dist.all_reduce(res, op=dist.ReduceOp.MIN)
        if rank == 0:
            out_q.put(res.tolist())
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_sequence_shard_ingress_on_two_gloo_ranks():
    ctx = mp.get_context('spawn')
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_seq_worker, args=(r, 2, port, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    res = out_q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res == [1, 1, 1]
