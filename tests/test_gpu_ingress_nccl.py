"""Sequence-sharded ingress on real GPUs: two ranks (one process per GPU, NCCL) each hold half of the sequence of every
head; an all-to-all turns that into whole sequences of half of the heads in the rank's OWN memory, the local kernels run,
and a second all-to-all returns sequence shards of the output.  Compared bit for bit with the single-GPU result.
Skipped where fewer than two GPUs are visible.  (NVLS is switched off for this test's process group: nothing here needs
it, and a rank that ends early must not leave a multicast binding behind.)"""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, causal, out_q):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    try:
        import hyperattention_b200 as ha
        from hyperattention_b200.partition import head_to_seq_shards, seq_to_head_shards
        B, H, n, d = 1, 4, 4096, 64
        g = torch.Generator().manual_seed(11)
        q, k, v = [torch.randn(B, H, n, d, generator=g).bfloat16() for _ in range(3)]
        mod = ha.HyperAttention(input_dim=d, min_seq_len=1024, rng=torch.Generator().manual_seed(12)).to(device=dev, dtype=torch.bfloat16)
        m = n // world
        local = [t[:, :, rank * m:(rank + 1) * m].contiguous().to(dev) for t in (q, k, v)]    # sequence shard, all heads
        ql, kl, vl = [seq_to_head_shards(t) for t in local]                                   # my heads, whole sequence
        o_heads, lse_heads = mod(ql, kl, vl, causal=causal, return_lse=True)
        o_seq = head_to_seq_shards(o_heads.contiguous())                                      # back to sequence shards
        ha.check_device_status(dev)
        # reference: the whole call on this rank's GPU alone
        o_full = mod(q.to(dev), k.to(dev), v.to(dev), causal=causal)
        ok = torch.tensor([int(torch.equal(o_seq, o_full[:, :, rank * m:(rank + 1) * m]))], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if rank == 0:
            out_q.put(int(ok.item()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('causal', [False, True])
def test_sequence_shard_ingress_on_two_gpus(causal):
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    ctx = mp.get_context('spawn')
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, causal, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    res = out_q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert res == 1
