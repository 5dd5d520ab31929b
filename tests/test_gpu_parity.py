"""GPU parity tests: every kernel is called through the C ABI (hyperattention_b200.ops / .module) and compared with
the CPU oracle on the same seeded inputs, and with the golden fixtures produced by the reference.

Tolerances (relative error in Frobenius norm, the quantity the reference's own tests print):
  float32 inputs : 1e-4 for outputs / LSE, 2e-4 for gradients
  bf16 / fp16    : 2e-2 for outputs / LSE, 3e-2 for gradients
Integer results (bucket codes, sort permutations) must be bit-exact.
"""
import math
import os

import pytest
import torch

from oracle import hyper_oracle as O

pytestmark = pytest.mark.gpu

T = lambda t: t.transpose(1, 2)
TOL = {torch.float32: (1e-4, 2e-4), torch.bfloat16: (2e-2, 3e-2), torch.float16: (2e-2, 3e-2)}


@pytest.fixture(scope='module')
def ha():
    import hyperattention_b200 as ha
    assert torch.cuda.is_available()
    return ha


def rel(a, b):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()


def dev(t):
    return t.cuda()


# ------------------------------------------------------------------------------------------------ LSH
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('shape,r', [((2, 3, 1000, 64), 8), ((1, 2, 513, 128), 8), ((1, 1, 300, 64), 16), ((1, 2, 257, 96), 5),
                                     ((1, 1, 64, 32), 8), ((1, 1, 0, 64), 8)])
def test_lsh_codes_bit_exact(ha, dtype, shape, r):
    torch.manual_seed(0)
    x = torch.randn(*shape).to(dtype)
    proj = torch.randn(1, 1, shape[-1], r).to(dtype)
    codes = ha.lsh_hash(dev(x), dev(proj.float().view(shape[-1], r).contiguous())).cpu()
    want = O.lsh_hash(x, proj)
    ties = O.lsh_tie_mask(x, proj, rel=2.0 ** -18)
    assert codes.dtype == torch.int32 and codes.shape == x.shape[:-1]
    assert not ((codes != want) & ~ties).any()
    assert x.numel() == 0 or ties.float().mean() < 2e-3


def test_lsh_strided_input_and_module_buffers(ha):
    torch.manual_seed(1)
    lsh = ha.AngularLSH(8, (1, 1, 64)).to(device='cuda', dtype=torch.bfloat16)
    assert set(dict(lsh.named_buffers())) == {'perm', 'proj_dir', 'enc_vec'} and len(lsh.state_dict()) == 0
    x = torch.randn(2, 200, 3, 64, device='cuda').to(torch.bfloat16).transpose(1, 2)   # [B,H,n,d] view, strided
    codes = lsh.hash_triton(x)
    want = O.lsh_hash(x.cpu(), lsh.proj_dir.cpu())
    ties = O.lsh_tie_mask(x.cpu(), lsh.proj_dir.cpu(), rel=2.0 ** -18)
    assert not ((codes.cpu() != want) & ~ties).any()
    assert torch.equal(lsh.perm.cpu(), O.gray_table(8))


@pytest.mark.parametrize('tag', ['a', 'b', 'c'])
def test_lsh_golden_reference_kernel(ha, golden_dir, tag):
    r = torch.load(os.path.join(golden_dir, f'kernel_lsh_{tag}.pt'))
    d, nb = r['proj_dir'].shape[-2:]
    codes = ha.lsh_hash(dev(r['x']), dev(r['proj_dir'].float().view(d, nb).contiguous())).cpu()
    ties = O.lsh_tie_mask(r['x'], r['proj_dir'], rel=2.0 ** -18)
    assert not ((codes != r['codes_kernel']) & ~ties).any()


# ------------------------------------------------------------------------------------------------ sort
@pytest.mark.parametrize('rows,n,bits', [(3, 5000, 8), (2, 128, 8), (1, 131072, 8), (4, 1000, 16), (2, 4096, 3), (1, 1, 8)])
def test_seg_sort_matches_stable_torch_sort(ha, rows, n, bits):
    torch.manual_seed(2)
    codes = torch.randint(0, 2 ** bits, (rows, n), dtype=torch.int32)
    idx = ha.seg_sort(dev(codes), bits).cpu()
    want = torch.sort(codes, dim=-1, stable=True)[1].to(torch.int32)
    assert torch.equal(idx, want)


def test_seg_sort_segments(ha):
    """spans cut into halves, as the causal schedule sorts them"""
    torch.manual_seed(3)
    rows, n, span = 3, 2048, 512
    codes = torch.randint(0, 256, (rows, n), dtype=torch.int32)
    for seg_off in (0, span // 2):
        idx = ha.seg_sort(dev(codes), 8, span=span, seg_off=seg_off, seg_len=span // 2).cpu()
        c = codes.view(rows, n // span, span)[:, :, seg_off:seg_off + span // 2].reshape(-1, span // 2)
        assert torch.equal(idx, torch.sort(c, dim=-1, stable=True)[1].to(torch.int32))


def test_indexing(ha):
    torch.manual_seed(4)
    x = torch.randn(2, 3, 100, 64).to(torch.bfloat16)
    idx = torch.randint(0, 100, (2, 3, 77))
    out = ha.indexing(dev(x), dev(idx)).cpu()
    assert torch.equal(out, x.gather(2, idx.unsqueeze(-1).expand(-1, -1, -1, 64)))
    out = ha.indexing(dev(x), dev(idx), chunk_size=32).cpu()
    assert out.shape[2] == 96 and torch.equal(out[:, :, 77:], torch.zeros(2, 3, 19, 64, dtype=torch.bfloat16))
    x32 = torch.randn(1, 2, 50, 33)
    idx = torch.randint(0, 50, (1, 2, 10))
    assert torch.equal(ha.indexing(dev(x32), dev(idx)).cpu(), x32.gather(2, idx.unsqueeze(-1).expand(-1, -1, -1, 33)))


def test_lse_merge_kernel(ha):
    torch.manual_seed(5)
    for dtype in (torch.float32, torch.bfloat16):
        a1, a2 = torch.randn(4, 300, 64).to(dtype), torch.randn(4, 300, 64).to(dtype)
        l1, l2 = torch.randn(4, 300), torch.randn(4, 300) * 3
        for exact in (False, True):
            o, l = ha.lse_merge_(dev(a1.clone()), dev(l1.clone()), dev(a2), dev(l2), exact=exact)
            fn = O.merge_exact if exact else O.add_self_attentions
            ow, lw = fn(a1, l1.unsqueeze(-1), a2, l2.unsqueeze(-1))
            assert rel(o, ow) < (1e-5 if dtype == torch.float32 else 1e-2)
            assert rel(l, lw.squeeze(-1)) < (1e-5 if dtype == torch.float32 else 5e-3)


# ------------------------------------------------------------------------------------------------ hyper attention op
def _hyper_case(B, H, n, d, dv, dtype, seed, buckets=16):
    torch.manual_seed(seed)
    q = torch.randn(B, H, n, d).to(dtype)
    k = torch.randn(B, H, n, d).to(dtype)
    v = torch.randn(B, H, n, dv).to(dtype)
    do = torch.randn(B, H, n, dv).to(dtype)
    qi = torch.sort(torch.randint(0, buckets, (B, H, n)), dim=2, stable=True)[1]
    ki = torch.sort(torch.randint(0, buckets, (B, H, n)), dim=2, stable=True)[1]
    return q, k, v, do, qi, ki


def _run_hyper_both(ha, q, k, v, do, qi, ki, block, sample, smooth, sample_idx=None, flags=0, exact_pattern=False):
    qg, kg, vg = [dev(t).requires_grad_() for t in (q, k, v)]
    o, lse = ha.hyper_attn_func(T(qg), T(kg), T(vg), T(dev(qi)), T(dev(ki)), block, sample, None, smooth,
                                None if sample_idx is None else dev(sample_idx), flags)
    T(o).backward(dev(do))
    qc, kc, vc = [t.float().requires_grad_() for t in (q, k, v)]
    ow, lw = O.hyper_attn_func(T(qc), T(kc), T(vc), T(qi), T(ki), block, sample, None, smooth, sample_idx, exact_pattern)
    T(ow).backward(do.float())
    return (T(o), lse, qg.grad, kg.grad, vg.grad), (T(ow), lw, qc.grad, kc.grad, vc.grad)


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize('cfg', [
    # B, H, n, d, dv, block, sample, smooth
    (1, 2, 512, 64, 64, 256, 128, False),
    (2, 1, 384, 64, 64, 256, 128, False),      # last block is partial
    (1, 2, 512, 64, 32, 128, 0, False),        # no sampled part, dv != d
    (1, 1, 768, 128, 128, 256, 256, False),
    (1, 2, 512, 64, 64, 256, 128, True),       # smooth windows
    (1, 1, 640, 32, 32, 384, 128, True),
    (1, 1, 256, 64, 64, 200, 128, False),      # block size rounded up to 256
])
def test_hyper_attn_fwd_bwd_vs_oracle(ha, dtype, cfg):
    B, H, n, d, dv, block, sample, smooth = cfg
    q, k, v, do, qi, ki = _hyper_case(B, H, n, d, dv, dtype, seed=10)
    from hyperattention_b200 import _lib as L
    flags = L.FLAG_BWD_REF_SMOOTH if smooth else 0
    got, want = _run_hyper_both(ha, q, k, v, do, qi, ki, block, sample, smooth, flags=flags)
    t_out, t_grad = TOL[dtype]
    assert got[0].shape == (B, H, n, dv) and got[1].shape == (B, H, n) and got[1].dtype == torch.float32
    assert rel(got[0], want[0]) < t_out
    assert rel(got[1], want[1]) < t_out
    for g, w in zip(got[2:], want[2:]):
        assert rel(g, w) < t_grad


def test_hyper_attn_exact_smooth_gradient(ha):
    """without HA_FLAG_BWD_REF_SMOOTH the backward enumerates the forward's own pair set (true gradient)"""
    q, k, v, do, qi, ki = _hyper_case(1, 2, 640, 64, 64, torch.float32, seed=11)
    got, want = _run_hyper_both(ha, q, k, v, do, qi, ki, 256, 128, True, exact_pattern=True)
    for g, w in zip(got[2:], want[2:]):
        assert rel(g, w) < 2e-4


def test_hyper_attn_explicit_sample_idx(ha):
    q, k, v, do, qi, ki = _hyper_case(1, 2, 512, 64, 64, torch.float32, seed=12)
    sidx = torch.stack([torch.randperm(512)[:128] for _ in range(2)]).view(1, 2, 128)
    got, want = _run_hyper_both(ha, q, k, v, do, qi, ki, 128, 128, False, sample_idx=sidx)
    assert rel(got[0], want[0]) < 1e-4 and rel(got[1], want[1]) < 1e-4
    for g, w in zip(got[2:], want[2:]):
        assert rel(g, w) < 2e-4


# ------------------------------------------------------------------------- weighted (uniformly sampled) key columns
def test_sample_weights_kernel(ha):
    """dropped-slot masks bit-exact, log weights to fp32 rounding, against the oracle's restatement"""
    torch.manual_seed(30)
    for n, block, S, smooth in [(512, 256, 128, False), (640, 384, 256, True), (384, 256, 128, False), (1024, 128, 384, True)]:
        segs = 3
        ki = torch.stack([torch.randperm(n) for _ in range(segs)])
        sidx = torch.stack([torch.randperm(n)[:S] for _ in range(segs)])
        logw, mask = ha.sample_weights(dev(ki).int(), dev(sidx).int(), n, block, S, smooth)
        for sg in range(segs):
            m_want, l_want = O.sample_tile_weights(n, ki[sg], block, sidx[sg], smooth)
            bits = ((mask[sg].cpu().long()[:, :, None] >> torch.arange(32)) & 1).bool().view(n // 128, S)
            assert torch.equal(bits, m_want)
            assert torch.allclose(logw[sg].cpu(), l_want, rtol=1e-6, atol=1e-6)
    # default rows 0..S-1 when no sample_idx is given
    logw, mask = ha.sample_weights(dev(ki).int(), None, 1024, 128, 384, True)
    m_want, _ = O.sample_tile_weights(1024, ki[0], 128, torch.arange(384), True)
    assert torch.equal(((mask[0].cpu().long()[:, :, None] >> torch.arange(32)) & 1).bool().view(8, 384), m_want)


@pytest.mark.parametrize('cfg', [
    # B, H, n, d, dv, block, sample, smooth, dtype
    (1, 2, 512, 64, 64, 256, 128, False, torch.float32),     # CUDA-core kernels
    (1, 2, 512, 64, 64, 256, 128, False, torch.bfloat16),    # tensor-core kernels, pipelined backward
    (2, 1, 640, 64, 64, 256, 256, True, torch.bfloat16),
    (1, 1, 768, 128, 128, 256, 256, False, torch.float16),   # tensor-core kernels, serial backward
    (1, 2, 384, 64, 32, 128, 128, False, torch.bfloat16),    # dv != d -> CUDA-core backward
])
def test_hyper_attn_weighted_sampling_vs_oracle(ha, cfg):
    """uniformly sampled key rows, own block excluded, importance-weighted: forward and backward.  With n this small
    about half of the sampled slots fall inside the query tile's window, so the dropped-slot path is exercised."""
    B, H, n, d, dv, block, sample, smooth, dtype = cfg
    q, k, v, do, qi, ki = _hyper_case(B, H, n, d, dv, dtype, seed=31)
    sidx = torch.stack([torch.randperm(n)[:sample] for _ in range(B * H)]).view(B, H, sample)
    from hyperattention_b200 import _lib as L
    flags = L.FLAG_BWD_REF_SMOOTH if smooth else 0
    qg, kg, vg = [dev(t).requires_grad_() for t in (q, k, v)]
    o, lse = ha.hyper_attn_func(T(qg), T(kg), T(vg), T(dev(qi)), T(dev(ki)), block, sample, None, smooth, dev(sidx), flags, True)
    T(o).backward(dev(do))
    qc, kc, vc = [t.float().requires_grad_() for t in (q, k, v)]
    ow, lw = O.hyper_attn_func(T(qc), T(kc), T(vc), T(qi), T(ki), block, sample, None, smooth, sidx, False, True)
    T(ow).backward(do.float())
    t_out, t_grad = TOL[dtype]
    assert rel(T(o), T(ow)) < t_out and rel(lse, lw) < t_out
    for g, w in zip((qg.grad, kg.grad, vg.grad), (qc.grad, kc.grad, vc.grad)):
        assert rel(g, w) < t_grad


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_weighted_sampling_of_every_key_is_exact_attention(ha, dtype):
    """property: when the sample is ALL keys, every key is counted once (in the block or as a kept sample of weight 1),
    so the estimator equals exact attention whatever the permutations are"""
    B, H, n, d = 1, 2, 512, 64
    q, k, v, do, qi, ki = _hyper_case(B, H, n, d, d, dtype, seed=32)
    sidx = torch.stack([torch.randperm(n) for _ in range(B * H)]).view(B, H, n)
    qg, kg, vg = [dev(t).requires_grad_() for t in (q, k, v)]
    o, lse = ha.hyper_attn_func(T(qg), T(kg), T(vg), T(dev(qi)), T(dev(ki)), 256, n, None, False, dev(sidx), 0, True)
    T(o).backward(dev(do))
    qc, kc, vc = [t.float().requires_grad_() for t in (q, k, v)]
    s = (qc @ kc.transpose(-1, -2)) * d ** -0.5
    ow = torch.softmax(s, -1) @ vc
    ow.backward(do.float())
    t_out, t_grad = TOL[dtype]
    assert rel(T(o), ow) < t_out and rel(lse, torch.logsumexp(s, -1)) < t_out
    for g, w in zip((qg.grad, kg.grad, vg.grad), (qc.grad, kc.grad, vc.grad)):
        assert rel(g, w) < t_grad


def test_module_uniform_sampling_mode(ha):
    """HyperAttention(sampling='uniform'): seeded draws are reproducible, distinct and in range; the output matches the
    oracle fed with the same draws; the causal recursion runs with it"""
    import hyperattention_b200 as hb
    torch.manual_seed(33)
    B, H, n, d = 1, 2, 1024, 64
    q, k, v = [torch.randn(B, H, n, d).bfloat16() for _ in range(3)]
    gen = torch.Generator(device='cuda')
    gen.manual_seed(7)
    mod = hb.HyperAttention(input_dim=d, block_size=128, sample_size=128, min_seq_len=256, sampling='uniform',
                            sample_generator=gen, rng=torch.Generator().manual_seed(1)).cuda().to(dtype=torch.bfloat16)
    o1, lse1 = mod(dev(q), dev(k), dev(v), return_lse=True)
    sidx = mod.last_sample_idx.cpu().long()
    assert sidx.shape == (B, H, 128) and sidx.min() >= 0 and sidx.max() < n
    assert all(len(set(sidx[0, h].tolist())) == 128 for h in range(H))
    gen.manual_seed(7)
    o2, _ = mod(dev(q), dev(k), dev(v), return_lse=True)
    assert torch.equal(o1, o2) and torch.equal(mod.last_sample_idx.cpu().long(), sidx)
    proj = mod.lsh.proj_dir.detach().cpu()
    qi = O.stable_argsort(O.lsh_hash(q, proj))
    ki = O.stable_argsort(O.lsh_hash(k, proj))
    ow, lw = O.hyper_attn_func(T(q.float()), T(k.float()), T(v.float()), T(qi), T(ki), 128, 128, None, False, sidx, False, True)
    if not (O.lsh_tie_mask(q, proj).any() or O.lsh_tie_mask(k, proj).any()):
        assert rel(o1, T(ow)) < TOL[torch.bfloat16][0] and rel(lse1.squeeze(-1), lw) < TOL[torch.bfloat16][0]
    oc = mod(dev(q), dev(k), dev(v), causal=True)
    assert oc.shape == (B, H, n, d) and torch.isfinite(oc.float()).all()
    # without a generator: counter-based draws, which the oracle computes on the host bit for bit (seed, call number)
    mod2 = hb.HyperAttention(input_dim=d, block_size=128, sample_size=128, min_seq_len=256, sampling='uniform', sample_seed=11,
                             rng=torch.Generator().manual_seed(1)).cuda().to(dtype=torch.bfloat16)
    for call in range(2):
        o3, lse3 = mod2(dev(q), dev(k), dev(v), return_lse=True)
        want = O.uniform_sample_idx(11, call, B * H, 128, n).view(B, H, 128)
        assert torch.equal(mod2.last_sample_idx.cpu().long(), want)
        ow, lw = O.hyper_attn_func(T(q.float()), T(k.float()), T(v.float()), T(qi), T(ki), 128, 128, None, False, want, False, True)
        if not (O.lsh_tie_mask(q, proj).any() or O.lsh_tie_mask(k, proj).any()):
            assert rel(o3, T(ow)) < TOL[torch.bfloat16][0] and rel(lse3.squeeze(-1), lw) < TOL[torch.bfloat16][0]


@pytest.mark.parametrize('cfg', [
    # n, d, block, sample, smooth, weighted, dtype
    (1024, 64, 256, 256, False, False, torch.bfloat16),
    (640, 64, 256, 128, True, False, torch.float16),
    (768, 128, 256, 256, False, False, torch.bfloat16),
    (512, 64, 128, 0, False, False, torch.bfloat16),          # no sampled part: no slot buffers
    (512, 64, 256, 0, False, False, torch.bfloat16),          # direct dq without a sampled launch
    (1152, 64, 256, 256, False, False, torch.float16),        # 9 query tiles: a last chunk of one tile; odd block count -> level 1
    (2304, 64, 256, 256, False, False, torch.bfloat16),       # 18 query tiles: chunks of 8, 8, 2
    (768, 64, 256, 128, False, False, torch.bfloat16),        # one sampled tile: slot buffers of a single 128-row tile
    (768, 64, 256, 384, False, False, torch.bfloat16),        # three sampled tiles
    (1024, 64, 256, 256, False, True, torch.bfloat16),
])
def test_direct_dk_dv_matches_fp32_accumulators(ha, cfg):
    """the backward with dK/dV stored directly (+ slot buffers and the finish kernel) against the same kernel reducing
    into fp32 accumulators: dq identical up to atomic order, dk/dv within one extra rounding of the storage dtype"""
    from hyperattention_b200 import ops, _lib as L
    n, d, block, sample, smooth, weighted, dtype = cfg
    B, H = 1, 3
    q, k, v, do, qi, ki = _hyper_case(B, H, n, d, d, dtype, seed=41)
    sidx = torch.stack([torch.randperm(n)[:sample] for _ in range(B * H)]).view(B, H, sample) if weighted else None
    flags = (L.FLAG_SMOOTH | L.FLAG_BWD_REF_SMOOTH) if smooth else 0
    qd, kd, vd, dod = [T(dev(t)) for t in (q, k, v, do)]
    o, lse = ha.hyper_attn_func(qd, kd, vd, T(dev(qi)), T(dev(ki)), block, sample, None, smooth,
                                None if sidx is None else dev(sidx), flags & ~L.FLAG_SMOOTH, weighted)
    qi32, ki32 = dev(qi).int().view(B * H, n), dev(ki).int().view(B * H, n)
    si32 = None if sidx is None else dev(sidx).int().view(B * H, sample)
    wts = ops.sample_weights(ki32, si32, n, block, sample, smooth) if weighted else None
    delta = (o.float() * dod.float()).sum(-1).transpose(1, 2).contiguous()
    args = (qd, kd, vd, qi32, ki32, si32, o, lse, dod, delta, block, sample, d ** -0.5, flags, wts)
    direct = ops.hyper_bwd(*args, direct=True)
    legacy = ops.hyper_bwd(*args, direct=False)
    assert rel(direct[0], legacy[0]) < 1e-3
    for g, w in zip(direct[1:], legacy[1:]):
        assert g.dtype == dtype and rel(g, w) < 6e-3


@pytest.mark.parametrize('shape', [(1, 2, 1024, 256), (2, 3, 2048, 256), (1, 2, 1024, 0), (1, 1, 512, 128), (1, 40, 2048, 256), (1, 3, 768, 384)])
@pytest.mark.parametrize('direct', [True, False])
def test_warp_specialised_backward_matches_earlier_kernel(ha, shape, direct):
    """attn_tc_bwd_ws_kernel (rows leave transposed through a staging tile; sampled rows as whole-tile bulk additions into
    slot buffers of its own layout) against the earlier backward kernel (HA_FLAG_NO_WS) on the same inputs, with typed
    outputs and with fp32 accumulators: the same sums in a different order and with one rounding of the partials"""
    from hyperattention_b200 import ops, _lib as L
    B, H, n, S = shape
    g = torch.Generator(device='cuda').manual_seed(7)
    q, k, v, do = [torch.randn(B, H, n, 64, device='cuda', generator=g).bfloat16() for _ in range(4)]
    proj = torch.randn(64, 8, device='cuda', generator=g)
    codes = torch.empty(2, B, H, n, dtype=torch.int32, device='cuda')
    ops.lsh_hash(q, proj, codes[0])
    ops.lsh_hash(k, proj, codes[1])
    idx = ops.seg_sort(codes.view(2 * B * H, n), 8)
    qi, ki = idx[:B * H].view(B, H, n), idx[B * H:].view(B, H, n)
    o, lse = ops.hyper_attn_func(T(q), T(k), T(v), T(qi), T(ki), 256, S)
    delta = (o.float() * T(do).float()).sum(-1).transpose(1, 2).contiguous()
    outs = []
    for flags in (L.FLAG_NO_WS, 0):
        r = ops.hyper_bwd(T(q), T(k), T(v), qi.view(B * H, n), ki.view(B * H, n), None, o, lse, T(do), delta, 256, S, 0.125, flags, None, direct)
        torch.cuda.synchronize()
        outs.append([t.clone() for t in r])
    for a_, b_ in zip(outs[1], outs[0]):
        assert rel(a_, b_) < 4e-3


@pytest.mark.parametrize('tag', ['plain', 'smooth', 'nosamp', 'd128', 'd128bwd', 's256bwd'])
def test_hyper_attn_golden_reference_kernels(ha, golden_dir, tag):
    """outputs of the reference's Triton kernels (fp16, interpreter) on their own inputs"""
    from hyperattention_b200 import _lib as L
    r = torch.load(os.path.join(golden_dir, f'kernel_hyper_{tag}.pt'))
    q, k, v = [dev(r[x]).requires_grad_() for x in 'qkv']
    flags = L.FLAG_BWD_REF_SMOOTH if r['smooth_block'] else 0
    o, lse = ha.hyper_attn_func(T(q), T(k), T(v), T(dev(r['q_sort_idx'])), T(dev(r['k_sort_idx'])), r['block_size'],
                                r['sample_size'], r['scale'], r['smooth_block'], None, flags)
    assert rel(T(o), r['o']) < 2e-3 and rel(lse, r['lse']) < 1e-3
    if 'do' in r:
        T(o).backward(dev(r['do']))
        assert rel(q.grad, r['dq']) < 5e-3 and rel(k.grad, r['dk']) < 5e-3 and rel(v.grad, r['dv']) < 5e-3


def test_hyper_attn_rejects_bad_shapes(ha):
    q, k, v, do, qi, ki = _hyper_case(1, 1, 200, 64, 64, torch.bfloat16, seed=13)
    with pytest.raises(AssertionError):
        ha.hyper_attn_func(T(dev(q)), T(dev(k)), T(dev(v)), T(dev(qi)), T(dev(ki)), 128, 128)   # n % 128 != 0
    q, k, v, do, qi, ki = _hyper_case(1, 1, 256, 64, 64, torch.bfloat16, seed=13)
    with pytest.raises(AssertionError):
        ha.hyper_attn_func(T(dev(q)), T(dev(k)), T(dev(v)), T(dev(qi)), T(dev(ki)), 128, 100)   # sample % 128 != 0
    with pytest.raises(AssertionError):
        ha.hyper_attn_func(T(q), T(k), T(v), T(qi), T(ki), 128, 128)                            # CPU tensors


# ------------------------------------------------------------------------------------------------ exact attention op
@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('cfg', [(1, 2, 256, 64, True), (2, 2, 200, 64, True), (1, 1, 384, 128, False), (1, 3, 77, 32, False),
                                 (1, 2, 1024, 64, True),
                                 (1, 1, 4608, 64, True),      # 36 query tiles: three chunks per key tile, some of them empty
                                 (1, 1, 2304, 64, False)])
def test_flash_fwd_bwd_vs_oracle(ha, dtype, cfg):
    B, H, n, d, causal = cfg
    torch.manual_seed(20)
    q, k, v, do = [torch.randn(B, n, H, d).to(dtype) for _ in range(4)]
    qg, kg, vg = [dev(t).requires_grad_() for t in (q, k, v)]
    o, lse = ha.flash_attn_func(qg, kg, vg, None, causal, None)
    o.backward(dev(do))
    qc, kc, vc = [t.float().requires_grad_() for t in (q, k, v)]
    ow, lw = O.flash_attn_func(qc, kc, vc, None, causal, None)
    ow.backward(do.float())
    t_out, t_grad = TOL[dtype]
    assert lse.shape == lw.shape
    assert rel(o, ow) < t_out and rel(lse[:, :, :n], lw[:, :, :n]) < t_out
    for g, w in zip((qg.grad, kg.grad, vg.grad), (qc.grad, kc.grad, vc.grad)):
        assert rel(g, w) < t_grad


def test_flash_fewer_keys_than_queries(ha):
    """the reference's unit test attends all queries to the first sample_size keys (unit_tests/test_hyper_attention.py:65-67)"""
    torch.manual_seed(21)
    q = torch.randn(1, 512, 2, 64)
    k, v = torch.randn(1, 128, 2, 64), torch.randn(1, 128, 2, 64)
    o, lse = ha.flash_attn_func(dev(q), dev(k), dev(v))
    ow, lw = O.flash_attn_func(q, k, v)
    assert rel(o, ow) < 1e-4 and rel(lse, lw) < 1e-4


@pytest.mark.parametrize('tag', ['causal', 'full'])
def test_flash_backward_golden_reference_kernels(ha, golden_dir, tag):
    """forward and backward of the reference's exact-attention Triton kernels (fp16, interpreter) on their own inputs"""
    r = torch.load(os.path.join(golden_dir, f'kernel_flash_bwd_{tag}.pt'))
    n = r['q'].shape[1]
    q, k, v = [dev(r[x]).requires_grad_() for x in 'qkv']
    o, lse = ha.flash_attn_func(q, k, v, None, r['causal'], r['scale'])
    assert rel(o, r['o']) < 2e-3 and rel(lse[:, :, :n], r['lse']) < 1e-3
    o.backward(dev(r['do']))
    assert rel(q.grad, r['dq']) < 5e-3 and rel(k.grad, r['dk']) < 5e-3 and rel(v.grad, r['dv']) < 5e-3


@pytest.mark.parametrize('tag', ['causal', 'full'])
def test_flash_golden_reference_kernel(ha, golden_dir, tag):
    r = torch.load(os.path.join(golden_dir, f'kernel_flash_{tag}.pt'))
    n = r['q'].shape[1]
    o, lse = ha.flash_attn_func(dev(r['q']), dev(r['k']), dev(r['v']), None, r['causal'], r['scale'])
    assert rel(o, r['o']) < 2e-3 and rel(lse[:, :, :n], r['lse']) < 1e-3


# ------------------------------------------------------------------------------------------------ module
def _module_pair(ha, r_or_cfg, dtype=torch.float32, **kw):
    cfg = r_or_cfg
    mod = ha.HyperAttention(input_dim=cfg['d'], lsh_num_projs=8, block_size=cfg['block_size'], sample_size=cfg['sample_size'],
                            min_seq_len=cfg['min_seq_len'], smooth_block=cfg['smooth_block'], **kw)
    mod.lsh.proj_dir.copy_(cfg['proj_dir'])
    return mod.to(device='cuda', dtype=dtype)


def _golden_module(golden_dir, tag):
    r = torch.load(os.path.join(golden_dir, f'module_{tag}.pt'))
    if 'q' not in r:
        torch.manual_seed(r['seed'])
        r['q'], r['k'], r['v'] = [torch.randn(1, 4, 4096, 64) for _ in range(3)]
        assert torch.equal(torch.randn(1, 1, 64, 8), r['proj_dir'])
        r['do'] = torch.randn(1, 4, 4096, 64)
    r['d'] = r['q'].shape[-1]
    return r


@pytest.mark.parametrize('tag', ['c0_noncausal', 'causal_2lvl', 'causal_odd', 'short_flash', 'causal_leaf', 'smooth'])
@pytest.mark.parametrize('fused', [True, False])
def test_module_matches_reference_golden(ha, golden_dir, tag, fused):
    """float32, the reference's own HyperAttention.forward output and gradients (benchmark configuration 0 is 'c0_noncausal')"""
    r = _golden_module(golden_dir, tag)
    mod = _module_pair(ha, r, fused_causal=fused)
    q, k, v = [dev(r[x]).requires_grad_() for x in 'qkv']
    o, lse = mod(q, k, v, causal=r['causal'], return_lse=True)
    o.backward(dev(r['do']))
    st = r.get('row_stride', 1)
    n = q.shape[2]
    assert tuple(lse.shape) == tuple(r['lse'].shape)
    assert rel(o[:, :, ::st], r['o']) < 1e-4
    assert rel(lse[:, :, :n], r['lse'][:, :, :n]) < 1e-4
    assert rel(q.grad[:, :, ::st], r['dq']) < 2e-4
    assert rel(k.grad[:, :, ::st], r['dk']) < 2e-4
    assert rel(v.grad[:, :, ::st], r['dv']) < 2e-4
    if 'q_codes' in r:   # bit-exact integer stages of benchmark configuration 0
        qc = mod.lsh.hash_triton(q.detach())
        kc = mod.lsh.hash_triton(k.detach())
        assert torch.equal(qc.cpu(), r['q_codes'].int()) and torch.equal(kc.cpu(), r['k_codes'].int())
        assert torch.equal(ha.seg_sort(qc, 8).view(1, 4, 4096).cpu(), r['q_sort_idx'].int() & 0xFFFF)
        assert torch.equal(ha.seg_sort(kc, 8).view(1, 4, 4096).cpu(), r['k_sort_idx'].int() & 0xFFFF)


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('causal', [False, True])
def test_module_half_precision_vs_oracle(ha, dtype, causal):
    torch.manual_seed(30)
    B, H, n, d = 1, 2, 2048, 64
    cfg = dict(d=d, block_size=256, sample_size=256, min_seq_len=512, smooth_block=False,
               proj_dir=torch.randn(1, 1, d, 8).to(dtype).float())
    q, k, v, do = [torch.randn(B, H, n, d).to(dtype) for _ in range(4)]
    mod = _module_pair(ha, cfg, dtype)
    qg, kg, vg = [dev(t).requires_grad_() for t in (q, k, v)]
    o, lse = mod(qg, kg, vg, causal=causal, return_lse=True)
    o.backward(dev(do))
    orc = O.HyperAttentionOracle(cfg['proj_dir'], 256, 256, 512, False)
    qc, kc, vc = [t.float().requires_grad_() for t in (q, k, v)]
    ow, lw = orc(qc, kc, vc, causal=causal, return_lse=True)
    ow.backward(do.float())
    assert o.dtype == dtype and lse.dtype == torch.float32
    assert rel(o, ow) < 2e-2 and rel(lse, lw) < 2e-2
    for g, w in zip((qg.grad, kg.grad, vg.grad), (qc.grad, kc.grad, vc.grad)):
        assert rel(g, w) < 3e-2


def test_module_exact_modes(ha):
    """grad_mode='exact' + merge_mode='exact': the gradient of the returned output (autograd through the oracle with
    the un-rounded merge and d(lse) kept)."""
    torch.manual_seed(31)
    B, H, n, d = 1, 2, 1024, 32
    proj = torch.randn(1, 1, d, 8)
    q, k, v, do = [torch.randn(B, H, n, d) for _ in range(4)]
    cfg = dict(d=d, block_size=128, sample_size=128, min_seq_len=256, smooth_block=False, proj_dir=proj)
    mod = _module_pair(ha, cfg, grad_mode='exact', merge_mode='exact')
    qg, kg, vg = [dev(t).requires_grad_() for t in (q, k, v)]
    o = mod(qg, kg, vg, causal=True)
    o.backward(dev(do))
    # differentiable dense restatement: same key sets, true softmax gradient
    import oracle.dense_check as D
    ow, grads = D.causal_exact_gradient(q, k, v, do, proj, 128, 128, 256)
    assert rel(o, ow) < 1e-4
    for g, w in zip((qg.grad, kg.grad, vg.grad), grads):
        assert rel(g, w) < 2e-4


def test_module_rejects_like_the_reference(ha):
    mod = ha.HyperAttention(input_dim=64).to(device='cuda', dtype=torch.bfloat16)
    q = torch.randn(1, 2, 4096, 64, device='cuda', dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        mod(q, q[:, :, :2048], q[:, :, :2048])            # n_query != n_key (hyper_attention.py:45)
    with pytest.raises(AssertionError):
        mod(q[:, :, :2100], q[:, :, :2100], q[:, :, :2100])   # not a multiple of 128 (src/hyper_attn_triton.py:695)
    with pytest.raises(ValueError):
        ha.AngularLSH(0, (1, 1, 64))


def test_launch_counter_moves(ha):
    before = ha.launch_count()
    ha.lsh_hash(torch.randn(1, 1, 128, 64, device='cuda'), torch.randn(64, 8, device='cuda'))
    assert ha.launch_count() == before + 1


@pytest.mark.parametrize('cfg', [(2, 3, 1024, 256, 256, torch.bfloat16), (1, 2, 512, 200, 128, torch.float16), (1, 40, 2048, 256, 0, torch.bfloat16)])
def test_persistent_forward_matches_one_tile_forward(ha, cfg):
    """the persistent warp-specialised forward (block size 256, head dim 64) against the one-tile-per-CTA kernel on the
    same inputs: same arithmetic in the same order per row, so outputs and lse are bit-identical.  The last case has
    more work items (320) than SMs, so every CTA walks several items and the copy ring wraps."""
    from hyperattention_b200 import _lib as L
    B, H, n, block, sample, dtype = cfg
    q, k, v, do, qi, ki = _hyper_case(B, H, n, 64, 64, dtype, seed=50)
    args = (T(dev(q)), T(dev(k)), T(dev(v)), T(dev(qi)), T(dev(ki)), block, sample, None, False, None)
    o1, l1 = ha.hyper_attn_func(*args, 0)
    o2, l2 = ha.hyper_attn_func(*args, L.FLAG_NO_WS)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)


def test_persistent_forward_in_the_causal_schedule_matches_one_tile_forward(ha):
    """the merging rectangle launches of the causal schedule through the persistent forward (default) and through the
    one-tile kernel (HA_FLAG_NO_WS): identical outputs, lse and -- reference gradient convention, which reads the
    un-merged part outputs -- gradients up to the order of fp32 atomic additions"""
    import hyperattention_b200 as hb
    from hyperattention_b200 import _lib as L
    torch.manual_seed(51)
    B, H, n, d = 1, 3, 4096, 64
    q, k, v, do = [torch.randn(B, H, n, d).bfloat16() for _ in range(4)]
    outs = []
    for flags in (0, L.FLAG_NO_WS):
        mod = hb.HyperAttention(input_dim=d, block_size=256, sample_size=256, min_seq_len=512, kernel_flags=flags,
                                rng=torch.Generator().manual_seed(2)).cuda().to(dtype=torch.bfloat16)
        qg, kg, vg = [dev(t).requires_grad_() for t in (q, k, v)]
        o, lse = mod(qg, kg, vg, causal=True, return_lse=True)
        o.backward(dev(do))
        outs.append((o.detach(), lse.detach(), qg.grad, kg.grad, vg.grad))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    for a, b in zip(outs[0][2:], outs[1][2:]):
        assert rel(a, b) < 1e-2      # (the two backward kernels round their per-item partial sums differently)
