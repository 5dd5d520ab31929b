"""Host-buffer entry point: chunks of heads streamed through the GPU give the same results as one call on the device."""
import pytest
import torch


def rel(a, b):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()


def test_host_stream_rejects_a_cpu_module():
    import hyperattention_b200 as ha
    from hyperattention_b200.host import HostStream
    with pytest.raises(AssertionError):
        HostStream(ha.HyperAttention(), device='cpu')


@pytest.mark.gpu
@pytest.mark.parametrize('causal', [False, True])
def test_host_stream_matches_device_call(causal):
    import hyperattention_b200 as ha
    from hyperattention_b200.host import HostStream, check_after
    torch.manual_seed(40)
    B, H, n, d = 1, 6, 1024, 64
    host = [torch.randn(B, H, n, d).bfloat16().pin_memory() for _ in range(4)]
    mod = ha.HyperAttention(input_dim=d, block_size=128, sample_size=128, min_seq_len=256,
                            rng=torch.Generator().manual_seed(3)).cuda().to(dtype=torch.bfloat16)
    qd, kd, vd, dod = [t.cuda() for t in host]
    qd, kd, vd = [t.requires_grad_() for t in (qd, kd, vd)]
    o_ref = mod(qd, kd, vd, causal=causal)
    g_ref = torch.autograd.grad(o_ref, (qd, kd, vd), dod)
    for hpc in (1, 4, None):                 # 6 chunks; 2 chunks, the last one ragged; a single chunk
        hs = HostStream(mod, heads_per_chunk=hpc)
        o = hs.forward(*host[:3], causal=causal)
        check_after()
        assert o.is_pinned() and torch.equal(o, o_ref.detach().cpu())      # the forward is deterministic: bit-exact
        o2, dq, dk, dv = hs.forward_backward(*host, causal=causal)
        check_after()
        assert torch.equal(o2, o_ref.detach().cpu())
        for g, w in zip((dq, dk, dv), g_ref):                              # fp32 atomics: order-dependent rounding
            assert rel(g, w) < 2e-3
    # batch of two: a chunk of heads is not contiguous in host memory then (copied per batch index)
    host2 = [torch.randn(2, 4, n, d).bfloat16().pin_memory() for _ in range(4)]
    q2, k2, v2, do2 = [t.cuda() for t in host2]
    q2, k2, v2 = [t.requires_grad_() for t in (q2, k2, v2)]
    o2_ref = mod(q2, k2, v2, causal=causal)
    g2_ref = torch.autograd.grad(o2_ref, (q2, k2, v2), do2)
    res2 = HostStream(mod, heads_per_chunk=3).forward_backward(*host2, causal=causal)
    check_after()
    assert torch.equal(res2[0], o2_ref.detach().cpu())
    for g, w in zip(res2[1:], g2_ref):
        assert rel(g, w) < 2e-3
    # caller-supplied output buffers, called twice in a row (buffers and streams are reused)
    outs = tuple(torch.empty(B, H, n, d, dtype=torch.bfloat16).pin_memory() for _ in range(4))
    hs = HostStream(mod, heads_per_chunk=2)
    for _ in range(2):
        res = hs.forward_backward(*host, causal=causal, out=outs)
        check_after()
        assert res[0] is outs[0] and torch.equal(outs[0], o_ref.detach().cpu())
