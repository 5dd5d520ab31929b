"""GPU tests at the headline benchmark sizes (batch 1, 32 heads, head_dim 64, 131072 tokens, bf16; configs 1 and 2).

The CPU oracle is too slow for all 32 heads at this length, so full-size runs are checked through size-independent
properties (permutation validity and stability, softmax rows summing to one, linearity in V, causality, determinism)
plus a direct comparison of a single head with the oracle (heads are independent in every stage, so a one-head oracle
run is an exact reference for that head of the 32-head run).  Tolerances: bf16 outputs/LSE 2e-2, gradients 3e-2
(relative Frobenius norm); integer results bit-exact.
"""
import pytest
import torch

from oracle import hyper_oracle as O

pytestmark = pytest.mark.gpu

H, N, D = 32, 131072, 64


def rel(a, b):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()


@pytest.fixture(scope='module')
def data():
    import hyperattention_b200 as ha
    from bench import clustered_inputs
    q, k, v, do = clustered_inputs(H, N, D, seed=1)
    g = torch.Generator().manual_seed(1234)
    mod = ha.HyperAttention(input_dim=D, rng=g).to(device='cuda', dtype=torch.bfloat16)
    return ha, mod, [t.cuda() for t in (q, k, v, do)]


def test_hash_and_sort_full_size(data):
    ha, mod, (q, k, v, do) = data
    codes = mod.lsh.hash_triton(q)
    assert codes.shape == (1, H, N) and int(codes.min()) >= 0 and int(codes.max()) < 256
    assert torch.equal(codes, mod.lsh.hash_triton(q))                      # deterministic
    # bit-exact against the oracle on a sample of rows
    sel = torch.randint(0, N, (4096,), generator=torch.Generator().manual_seed(0))
    qs = q[0, :, sel].cpu()
    want = O.lsh_hash(qs, mod.lsh.proj_dir.cpu())
    ties = O.lsh_tie_mask(qs, mod.lsh.proj_dir.cpu())
    got = codes[0][:, sel.cuda()].cpu()
    assert not ((got != want) & ~ties).any() and ties.float().mean() < 2e-3
    # the sort output is a stable ascending permutation of every head
    idx = ha.seg_sort(codes, 8).view(H, N).long()
    c = codes.view(H, N)
    assert torch.equal(torch.sort(idx, dim=1)[0], torch.arange(N, device='cuda').expand(H, N))
    sc = torch.gather(c, 1, idx)
    assert bool((sc[:, 1:] >= sc[:, :-1]).all())
    same = sc[:, 1:] == sc[:, :-1]
    assert bool((idx[:, 1:][same] > idx[:, :-1][same]).all())               # ties keep the original order


def test_noncausal_forward_properties(data):
    ha, mod, (q, k, v, do) = data
    o, lse = mod(q, k, v, return_lse=True)
    assert o.shape == (1, H, N, D) and lse.shape == (1, H, N, 1) and torch.isfinite(o).all() and torch.isfinite(lse).all()
    # rows of the attention matrix sum to one
    ones = mod(q, k, torch.ones_like(v))
    assert (ones.float() - 1).abs().max().item() < 2e-2
    # linear in V
    v2 = torch.randn_like(v)
    o2 = mod(q, k, v2)
    o12 = mod(q, k, (v.float() + v2.float()).to(v.dtype))
    assert rel(o12, o.float() + o2.float()) < 2e-2
    # one head against the oracle, forward and backward: the backward launch here is the one the benchmark times (whole
    # 256-row blocks with the sampled tiles fused in, gradients written directly in bf16)
    h = 5
    qg, kg, vg = [t.clone().requires_grad_() for t in (q, k, v)]
    og = mod(qg, kg, vg)
    dq, dk, dv = torch.autograd.grad(og, (qg, kg, vg), do)
    assert torch.equal(og.detach(), o)
    for t in (dq, dk, dv):
        assert torch.isfinite(t).all()
    orc = O.HyperAttentionOracle(mod.lsh.proj_dir.float().cpu(), 256, 256, 2048, False)
    qc, kc, vc = [x[:, h:h + 1].float().cpu().requires_grad_() for x in (q, k, v)]
    ow, lw = orc(qc, kc, vc, return_lse=True)
    ow.backward(do[:, h:h + 1].float().cpu())
    assert rel(o[:, h:h + 1], ow) < 2e-2 and rel(lse[:, h:h + 1], lw) < 2e-2
    assert rel(dq[:, h:h + 1], qc.grad) < 3e-2
    assert rel(dk[:, h:h + 1], kc.grad) < 3e-2
    assert rel(dv[:, h:h + 1], vc.grad) < 3e-2


def test_causal_forward_backward_full_size(data):
    ha, mod, (q, k, v, do) = data
    qg, kg, vg = [t.clone().requires_grad_() for t in (q, k, v)]
    o, lse = mod(qg, kg, vg, causal=True, return_lse=True)
    dq, dk, dv = torch.autograd.grad(o, (qg, kg, vg), do)
    for t in (o, lse, dq, dk, dv):
        assert torch.isfinite(t).all()
    # causality: changing keys / values from position t on leaves every earlier output row bit-identical
    t = 70000
    k2, v2 = k.clone(), v.clone()
    k2[:, :, t:] = torch.randn_like(k2[:, :, t:])
    v2[:, :, t:] = torch.randn_like(v2[:, :, t:])
    o2, lse2 = mod(q, k2, v2, causal=True, return_lse=True)
    assert torch.equal(o2[:, :, :t], o.detach()[:, :, :t]) and torch.equal(lse2[:, :, :t], lse.detach()[:, :, :t])
    assert not torch.equal(o2[:, :, t:], o.detach()[:, :, t:])
    # the first row attends to itself only
    assert rel(o[:, :, 0], v[:, :, 0]) < 1e-2
    # one head against the oracle, forward and backward (reference gradient conventions)
    h = 17
    orc = O.HyperAttentionOracle(mod.lsh.proj_dir.float().cpu(), 256, 256, 2048, False)
    qc, kc, vc = [x[:, h:h + 1].float().cpu().requires_grad_() for x in (q, k, v)]
    ow, lw = orc(qc, kc, vc, causal=True, return_lse=True)
    ow.backward(do[:, h:h + 1].float().cpu())
    assert rel(o[:, h:h + 1], ow) < 2e-2 and rel(lse[:, h:h + 1], lw) < 2e-2
    assert rel(dq[:, h:h + 1], qc.grad) < 3e-2
    assert rel(dk[:, h:h + 1], kc.grad) < 3e-2
    assert rel(dv[:, h:h + 1], vc.grad) < 3e-2


def test_tensor_core_and_cuda_core_paths_agree(data):
    """the fp32 CUDA-core kernels (HA_FLAG_FORCE_SIMT) on the same bf16 inputs, two heads, 16384 tokens"""
    ha, mod, (q, k, v, do) = data
    from hyperattention_b200 import _lib as L
    n = 16384
    qs, ks, vs, dos = [t[:, :2, :n].contiguous() for t in (q, k, v, do)]
    outs = []
    for flags in (0, L.FLAG_FORCE_SIMT):
        m2 = ha.HyperAttention(input_dim=D, kernel_flags=flags).to(device='cuda', dtype=torch.bfloat16)
        m2.lsh.proj_dir.copy_(mod.lsh.proj_dir)
        qg, kg, vg = [t.clone().requires_grad_() for t in (qs, ks, vs)]
        o = m2(qg, kg, vg, causal=True)
        outs.append((o,) + torch.autograd.grad(o, (qg, kg, vg), dos))
    for a, b in zip(*outs):
        assert rel(a, b) < 2e-2
