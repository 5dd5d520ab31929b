"""Parity at the sizes and flag combinations that the benchmark configurations time.

The CPU oracle is O(n) per head on the hyper pattern, so one head of a full-size run can be checked against it even at
524288 tokens; heads are independent in every stage, so a one-head oracle run is an exact reference for that head of a
32-head GPU run.  Tolerances are the ones the task states: outputs / LSE 2e-2 (bf16), gradients 3e-2 (relative
Frobenius norm), fp32 1e-4 / 2e-4.  What is compared is what the reference's own test compares
(unit_tests/test_hyper_attention.py:135-256): output, LSE and the three gradients.
"""
import ctypes as C

import pytest
import torch

from oracle import hyper_oracle as O

pytestmark = pytest.mark.gpu


def rel(a, b):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()


def _one_head_vs_oracle(mod, q, k, v, do, h, causal, block, sample, msl, smooth=False, tol_o=2e-2, tol_g=3e-2):
    """Runs the module on all heads, the oracle on head h; compares o, lse, dq, dk, dv of that head."""
    qg, kg, vg = [t.detach().requires_grad_() for t in (q, k, v)]
    o, lse = mod(qg, kg, vg, causal=causal, return_lse=True)
    dq, dk, dv = torch.autograd.grad(o, (qg, kg, vg), do)
    for t in (o, lse, dq, dk, dv):
        assert torch.isfinite(t).all()
    orc = O.HyperAttentionOracle(mod.lsh.proj_dir.float().cpu(), block, sample, msl, smooth)
    qc, kc, vc = [x[:, h:h + 1].float().cpu().requires_grad_() for x in (q, k, v)]
    ow, lw = orc(qc, kc, vc, causal=causal, return_lse=True)
    ow.backward(do[:, h:h + 1].float().cpu())
    n = q.shape[2]
    errs = {'o': rel(o[:, h:h + 1], ow), 'lse': rel(lse[:, h:h + 1, :n], lw[:, :, :n]), 'dq': rel(dq[:, h:h + 1], qc.grad),
            'dk': rel(dk[:, h:h + 1], kc.grad), 'dv': rel(dv[:, h:h + 1], vc.grad)}
    assert errs['o'] < tol_o and errs['lse'] < tol_o and max(errs['dq'], errs['dk'], errs['dv']) < tol_g, errs
    return errs


def _randn_heads(H, n, d, seed, count=4, dtype=torch.bfloat16):
    g = torch.Generator(device='cuda').manual_seed(seed)
    return [torch.randn(1, H, n, d, device='cuda', generator=g).to(dtype) for _ in range(count)]


@pytest.mark.parametrize('causal', [False, True])
def test_sweep_longest_length_one_head_vs_oracle(causal):
    """Sequence-length sweep, longest point: 32 heads x 524288 x 64, bf16, i.i.d. N(0,1) (byte offsets beyond 2^31,
    4096 sort sub-chunks per head, eight half-splits in the causal case)."""
    import hyperattention_b200 as ha
    H, n, d = 32, 524288, 64
    q, k, v, do = _randn_heads(H, n, d, seed=3)
    mod = ha.HyperAttention(input_dim=d, rng=torch.Generator().manual_seed(1234)).to(device='cuda', dtype=torch.bfloat16)
    _one_head_vs_oracle(mod, q, k, v, do, 29, causal, 256, 256, 2048)
    del q, k, v, do
    torch.cuda.empty_cache()


@pytest.mark.parametrize('grad_mode', ['reference', 'exact'])
def test_causal_smooth_block_both_gradient_modes(grad_mode):
    """causal=True with smooth_block=True through the single-call schedule, n = 8192 (two half-splits), float32 kernels so
    that the comparison is tight.  'reference' reproduces the reference's gradient conventions (the oracle's autograd);
    'exact' is the gradient of the returned output (dense differentiable restatement)."""
    import hyperattention_b200 as ha
    import oracle.dense_check as D
    torch.manual_seed(61)
    B, H, n, d = 1, 2, 8192, 64
    proj = torch.randn(1, 1, d, 8)
    q, k, v, do = [torch.randn(B, H, n, d) for _ in range(4)]
    kw = dict(grad_mode='exact', merge_mode='exact') if grad_mode == 'exact' else {}
    mod = ha.HyperAttention(input_dim=d, block_size=256, sample_size=256, min_seq_len=2048, smooth_block=True, **kw)
    mod.lsh.proj_dir.copy_(proj)
    mod = mod.cuda()
    assert mod._regular_causal(n)
    qg, kg, vg = [t.cuda().requires_grad_() for t in (q, k, v)]
    o = mod(qg, kg, vg, causal=True)
    o.backward(do.cuda())
    if grad_mode == 'exact':
        ow, grads = D.causal_exact_gradient(q, k, v, do, proj, 256, 256, 2048, smooth=True)
    else:
        orc = O.HyperAttentionOracle(proj, 256, 256, 2048, True)
        qc, kc, vc = [t.clone().requires_grad_() for t in (q, k, v)]
        ow = orc(qc, kc, vc, causal=True)
        ow.backward(do)
        grads = (qc.grad, kc.grad, vc.grad)
    assert rel(o, ow) < 1e-4
    for g, w in zip((qg.grad, kg.grad, vg.grad), grads):
        assert rel(g, w) < 2e-4
    # and in bf16 on the tensor-core kernels
    modh = ha.HyperAttention(input_dim=d, block_size=256, sample_size=256, min_seq_len=2048, smooth_block=True, **kw)
    modh.lsh.proj_dir.copy_(proj.bfloat16().float())
    modh = modh.to(device='cuda', dtype=torch.bfloat16)
    qh, kh, vh, doh = [t.bfloat16() for t in (q, k, v, do)]
    qg, kg, vg = [t.cuda().requires_grad_() for t in (qh, kh, vh)]
    o = modh(qg, kg, vg, causal=True)
    o.backward(doh.cuda())
    if grad_mode == 'exact':
        ow, grads = D.causal_exact_gradient(qh.float(), kh.float(), vh.float(), doh.float(), proj.bfloat16().float(), 256, 256, 2048, smooth=True)
    else:
        orc = O.HyperAttentionOracle(proj.bfloat16().float(), 256, 256, 2048, True)
        qc, kc, vc = [t.float().requires_grad_() for t in (qh, kh, vh)]
        ow = orc(qc, kc, vc, causal=True)
        ow.backward(doh.float())
        grads = (qc.grad, kc.grad, vc.grad)
    assert rel(o, ow) < 2e-2
    for g, w in zip((qg.grad, kg.grad, vg.grad), grads):
        assert rel(g, w) < 3e-2


def test_decoder_attention_shape_one_head_vs_oracle():
    """The attention call of the ChatGLM2-6B-shaped prefill: 32 heads x 32768 x head_dim 128, causal, bf16
    (four half-splits, 16 leaves of 2048 rows per head)."""
    import hyperattention_b200 as ha
    H, n, d = 32, 32768, 128
    q, k, v, do = _randn_heads(H, n, d, seed=4)
    mod = ha.HyperAttention(input_dim=d, rng=torch.Generator().manual_seed(77)).to(device='cuda', dtype=torch.bfloat16)
    _one_head_vs_oracle(mod, q, k, v, do, 11, True, 256, 256, 2048)


@pytest.mark.parametrize('fused', [True, False])
@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_causal_deepest_rectangle_below_min_seq_len_is_exact(fused, dtype):
    """n = 3 * 512 with min_seq_len = 512: two half-splits, leaves of 384 rows.  The deepest rectangles (384 x 384) are
    shorter than min_seq_len, so the reference computes them exactly (hyper_attention.py:109-113); the single-call
    schedule and the per-level path must both do that."""
    import hyperattention_b200 as ha
    torch.manual_seed(62)
    B, H, n, d = 1, 3, 1536, 64
    proj = torch.randn(1, 1, d, 8).to(dtype).float()
    q, k, v, do = [torch.randn(B, H, n, d).to(dtype) for _ in range(4)]
    mod = ha.HyperAttention(input_dim=d, block_size=256, sample_size=256, min_seq_len=512, fused_causal=fused)
    mod.lsh.proj_dir.copy_(proj)
    mod = mod.to(device='cuda', dtype=dtype)
    assert mod._regular_causal(n) and mod._causal_levels(n) == 2
    qg, kg, vg = [t.cuda().requires_grad_() for t in (q, k, v)]
    o, lse = mod(qg, kg, vg, causal=True, return_lse=True)
    o.backward(do.cuda())
    orc = O.HyperAttentionOracle(proj, 256, 256, 512, False)
    qc, kc, vc = [t.float().requires_grad_() for t in (q, k, v)]
    ow, lw = orc(qc, kc, vc, causal=True, return_lse=True)
    ow.backward(do.float())
    assert ('flash', (1, 4 * H, 384, d), True) in orc.trace          # the leaves
    assert ('flash', (1, 2 * H, 384, d), False) in orc.trace         # the deepest rectangles: exact, no mask
    assert ('hyper', (1, H, 768, d), False) in orc.trace             # the top rectangle: hyper pattern
    to, tg = (1e-4, 2e-4) if dtype == torch.float32 else (2e-2, 3e-2)
    assert rel(o, ow) < to and rel(lse, lw) < to
    for g, w in zip((qg.grad, kg.grad, vg.grad), (qc.grad, kc.grad, vc.grad)):
        assert rel(g, w) < tg


def test_strided_inputs_need_no_copy():
    """[B, n, H, d]-resident q, k, v passed as transposed [B, H, n, d] views: same kernels, same launch count and
    bit-identical results as the contiguous call (the reference copies them, hyper_attention.py:38-40)."""
    import hyperattention_b200 as ha
    torch.manual_seed(63)
    B, H, n, d = 2, 4, 2048, 64
    mod = ha.HyperAttention(input_dim=d, min_seq_len=512, rng=torch.Generator().manual_seed(5)).to(device='cuda', dtype=torch.bfloat16)
    base = [torch.randn(B, n, H, d, device='cuda').bfloat16() for _ in range(3)]
    views = [t.transpose(1, 2) for t in base]
    assert not views[0].is_contiguous()
    c0 = ha.launch_count()
    o1, l1 = mod(*views, return_lse=True)
    c1 = ha.launch_count()
    o2, l2 = mod(*[t.contiguous() for t in views], return_lse=True)
    c2 = ha.launch_count()
    assert c1 - c0 == c2 - c1                    # no extra kernel for the strided call
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    # gradients flow to the strided leaves
    qg, kg, vg = [t.clone().requires_grad_() for t in base]
    o = mod(qg.transpose(1, 2), kg.transpose(1, 2), vg.transpose(1, 2))
    o.sum().backward()
    assert qg.grad.shape == qg.shape and torch.isfinite(qg.grad).all()


def test_device_timeout_reaches_the_host_as_an_exception():
    """A bounded device-side wait that runs out (a probe kernel polling a barrier nobody arrives at -- nothing else in
    flight) sets the status words; the next call into the library raises RuntimeError without anybody having to ask, and
    the library is usable again afterwards."""
    import hyperattention_b200 as ha
    from hyperattention_b200 import _lib as L
    from hyperattention_b200 import ops
    dev_w, host_w = ops._status_words(torch.cuda.current_device())
    assert int(host_w[0]) == 0
    x = torch.randn(1, 1, 256, 64, device='cuda')
    proj = torch.randn(64, 8, device='cuda')
    q = torch.randn(1, 256, 1, 64, device='cuda').bfloat16()
    rc = L.load().ha_wait_probe(C.c_void_p(dev_w.data_ptr()), C.c_void_p(host_w.data_ptr()), 300,
                                C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(dev_w.item()) == 1 and int(host_w[0]) == 1
    with pytest.raises(RuntimeError, match='timed out'):
        ha.flash_attn_func(q, q, q)                 # the next attention call notices, before launching anything
    assert int(host_w[0]) == 0
    torch.cuda.synchronize()
    assert int(dev_w.item()) == 0
    o, _ = ha.flash_attn_func(q, q, q)              # healthy again
    assert torch.isfinite(o).all()
    ha.check_device_status()
    assert ha.lsh_hash(x, proj).shape == (1, 1, 256)


@pytest.mark.parametrize('dtype,smooth', [(torch.bfloat16, False), (torch.float16, True), (torch.float32, False)])
def test_single_call_noncausal_path_matches_per_operator_path(dtype, smooth):
    """ha_noncausal_fwd / ha_noncausal_bwd (hash, sort, attention; delta, backward, finishing pass in one library call
    each way) against the same module calling one operator at a time: identical forward, gradients equal up to the order
    of fp32 additions; and far fewer calls into the library."""
    import hyperattention_b200 as ha
    torch.manual_seed(64)
    B, H, n, d = 2, 3, 2048, 64
    q, k, v, do = [torch.randn(B, H, n, d, device='cuda').to(dtype) for _ in range(4)]
    outs = []
    for fused in (True, False):
        mod = ha.HyperAttention(input_dim=d, block_size=256, sample_size=256, min_seq_len=512, smooth_block=smooth, fused_calls=fused,
                                rng=torch.Generator().manual_seed(6)).to(device='cuda', dtype=dtype)
        qg, kg, vg = [t.clone().requires_grad_() for t in (q, k, v)]
        o, lse = mod(qg, kg, vg, return_lse=True)
        assert o.shape == (B, H, n, d) and lse.shape == (B, H, n, 1)
        o.backward(do)
        outs.append((o.detach(), lse.detach(), qg.grad, kg.grad, vg.grad))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    for a, b in zip(outs[0][2:], outs[1][2:]):
        assert rel(a, b) < 1e-3


@pytest.mark.parametrize('causal', [False, True])
@pytest.mark.parametrize('dtype,d', [(torch.bfloat16, 128), (torch.bfloat16, 64), (torch.float32, 64)])
def test_grouped_query_heads_match_expanded_heads(causal, dtype, d):
    """Grouped-query attention: K/V with 2 heads serving 8 (bf16: 16) query heads, hashed and sorted once per K/V head,
    against the same call with K/V expanded to every query head (what the reference is given,
    chatglm_fast_attention.py:53-58): identical forward; dK/dV of a K/V head equal the sum over its group's expanded
    heads; and one head group against the oracle."""
    import hyperattention_b200 as ha
    torch.manual_seed(65)
    B, Hkv, rep, n = 1, 2, (8 if dtype == torch.bfloat16 else 4), 4096
    H = Hkv * rep
    q = torch.randn(B, H, n, d, device='cuda').to(dtype)
    k, v = [torch.randn(B, Hkv, n, d, device='cuda').to(dtype) for _ in range(2)]
    do = torch.randn(B, H, n, d, device='cuda').to(dtype)
    mod = ha.HyperAttention(input_dim=d, min_seq_len=1024, rng=torch.Generator().manual_seed(7)).to(device='cuda', dtype=dtype)
    qg, kg, vg = [t.clone().requires_grad_() for t in (q, k, v)]
    o, lse = mod(qg, kg, vg, causal=causal, return_lse=True)
    o.backward(do)
    ke, ve = [t.repeat_interleave(rep, dim=1).clone().requires_grad_() for t in (k, v)]
    qe = q.clone().requires_grad_()
    oe, lse_e = mod(qe, ke, ve, causal=causal, return_lse=True)
    oe.backward(do)
    assert o.shape == (B, H, n, d) and kg.grad.shape == k.shape
    assert torch.equal(o, oe) and torch.equal(lse, lse_e)
    tol = 2e-4 if dtype == torch.float32 else 1e-2
    assert rel(qg.grad, qe.grad) < tol
    assert rel(kg.grad, ke.grad.float().view(B, Hkv, rep, n, d).sum(2)) < tol
    assert rel(vg.grad, ve.grad.float().view(B, Hkv, rep, n, d).sum(2)) < tol
    # the first K/V head and one of its query heads against the oracle
    orc = O.HyperAttentionOracle(mod.lsh.proj_dir.float().cpu(), 256, 256, 1024, False)
    ow, lw = orc(q[:, 1:2].float().cpu(), k[:, 0:1].float().cpu(), v[:, 0:1].float().cpu(), causal=causal, return_lse=True)
    to = 1e-4 if dtype == torch.float32 else 2e-2
    assert rel(o[:, 1:2], ow) < to and rel(lse[:, 1:2], lw) < to


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_index_check_turns_a_bad_permutation_into_a_status(dtype):
    """HA_FLAG_CHECK_INDICES: a hand-made permutation with a row outside the sequence does not make the kernels read a row
    that does not exist (the checking kernel sets the status word, the attention kernel returns at once); the next call
    into the library raises.  With valid indices the flag changes nothing."""
    import hyperattention_b200 as ha
    from hyperattention_b200 import _lib as L
    torch.manual_seed(66)
    B, H, n, d = 1, 2, 1024, 64
    q, k, v = [torch.randn(B, n, H, d, device='cuda').to(dtype) for _ in range(3)]
    qi = torch.stack([torch.randperm(n) for _ in range(B * H)]).view(B, H, n).transpose(1, 2).cuda()
    ki = torch.stack([torch.randperm(n) for _ in range(B * H)]).view(B, H, n).transpose(1, 2).cuda()
    o0, l0 = ha.hyper_attn_func(q, k, v, qi, ki, 256, 256)
    o1, l1 = ha.hyper_attn_func(q, k, v, qi, ki, 256, 256, None, False, None, L.FLAG_CHECK_INDICES)
    assert torch.equal(o0, o1) and torch.equal(l0, l1)
    ha.check_device_status()
    bad = ki.clone()
    bad[0, 17, 1] = n + 5                       # one key position of head 1 points past the sequence
    ha.hyper_attn_func(q, k, v, qi, bad, 256, 256, None, False, None, L.FLAG_CHECK_INDICES)     # no fault, no exception yet
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match='index'):
        ha.hyper_attn_func(q, k, v, qi, ki, 256, 256)
    o2, _ = ha.hyper_attn_func(q, k, v, qi, ki, 256, 256)            # healthy again
    assert torch.equal(o2, o0)
    ha.check_device_status()
