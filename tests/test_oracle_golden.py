"""The CPU oracle against the fixtures produced by running the reference (tests/golden/make_golden.py)."""
import glob
import os

import pytest
import torch

from oracle import hyper_oracle as O

T = lambda t: t.transpose(1, 2)


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)).item()


def _load(golden_dir, name):
    return torch.load(os.path.join(golden_dir, name))


@pytest.mark.parametrize('tag', ['a', 'b', 'c'])
def test_lsh_matches_reference_kernel_and_hash_torch(golden_dir, tag):
    r = _load(golden_dir, f'kernel_lsh_{tag}.pt')
    codes = O.lsh_hash(r['x'], r['proj_dir'])
    ties = O.lsh_tie_mask(r['x'], r['proj_dir'])
    assert codes.dtype == torch.int32
    # bit-exact outside ties (sign of a projection within fp rounding of zero)
    assert not ((codes != r['codes_kernel']) & ~ties).any()
    assert not ((codes != r['codes_hash_torch']) & ~ties).any()
    assert torch.equal(O.gray_table(r['proj_dir'].shape[-1]), r['perm'])


@pytest.mark.parametrize('tag', ['plain', 'smooth', 'nosamp', 'd128', 'd128bwd', 's256bwd'])
def test_hyper_attn_matches_reference_kernels(golden_dir, tag):
    """fp16 Triton-interpreter output of _fwd_hyper_kernel and the three backward kernels; tolerance is fp16
    rounding of inputs/outputs (1e-3 relative in norm).  's256bwd': sample_size = 256, where only the reference's backward
    is usable (its forward reads other rows there); the fixture's (o, lse) are those of rows 0..255, which is what the
    backward kernels were given."""
    r = _load(golden_dir, f'kernel_hyper_{tag}.pt')
    q, k, v = [r[x].float().requires_grad_() for x in 'qkv']
    o, lse = O.hyper_attn_func(T(q), T(k), T(v), T(r['q_sort_idx']), T(r['k_sort_idx']), r['block_size'],
                               r['sample_size'], r['scale'], r['smooth_block'])
    assert rel(T(o), r['o']) < 1e-3
    assert rel(lse, r['lse']) < 1e-5
    if 'do' in r:
        T(o).backward(r['do'].float())
        assert rel(q.grad, r['dq']) < 2e-3
        assert rel(k.grad, r['dk']) < 2e-3
        assert rel(v.grad, r['dv']) < 2e-3


def test_smooth_block_reference_backward_is_not_the_forward_gradient(golden_dir):
    """The reference's smooth_block backward enumerates a different pair set than its forward; the oracle's
    exact_pattern=True switch gives the true gradient, which must differ visibly from the reference's."""
    r = _load(golden_dir, 'kernel_hyper_smooth.pt')
    q, k, v = [r[x].float().requires_grad_() for x in 'qkv']
    o, _ = O.hyper_attn_func(T(q), T(k), T(v), T(r['q_sort_idx']), T(r['k_sort_idx']), r['block_size'],
                             r['sample_size'], r['scale'], True, None, True)
    T(o).backward(r['do'].float())
    assert rel(k.grad, r['dk']) > 0.1


@pytest.mark.parametrize('tag', ['causal', 'full'])
def test_flash_backward_matches_reference_kernels(golden_dir, tag):
    """_bwd_preprocess_do_o_dot + _bwd_kernel of the exact attention under the interpreter (fp16)"""
    r = _load(golden_dir, f'kernel_flash_bwd_{tag}.pt')
    n = r['q'].shape[1]
    q, k, v = [r[x].float().requires_grad_() for x in 'qkv']
    o, lse = O.flash_attn_func(q, k, v, None, r['causal'], r['scale'])
    assert rel(o, r['o']) < 1e-3 and rel(lse[:, :, :n], r['lse']) < 1e-5
    o.backward(r['do'].float())
    assert rel(q.grad, r['dq']) < 2e-3 and rel(k.grad, r['dk']) < 2e-3 and rel(v.grad, r['dv']) < 2e-3


@pytest.mark.parametrize('tag', ['causal', 'full'])
def test_flash_matches_reference_kernel(golden_dir, tag):
    r = _load(golden_dir, f'kernel_flash_{tag}.pt')
    n = r['q'].shape[1]
    o, lse = O.flash_attn_func(r['q'].float(), r['k'].float(), r['v'].float(), None, r['causal'], r['scale'])
    assert rel(o, r['o']) < 1e-3
    assert rel(lse[:, :, :n], r['lse']) < 1e-5
    assert lse.shape[-1] % 128 == 0


def _module_inputs(r):
    if 'q' in r:
        return r['q'], r['k'], r['v'], r['do']
    # benchmark configuration 0: regenerate from the seed in the order the fixture script drew them
    torch.manual_seed(r['seed'])
    q = torch.randn(1, 4, 4096, 64)
    k = torch.randn(1, 4, 4096, 64)
    v = torch.randn(1, 4, 4096, 64)
    proj = torch.randn(1, 1, 64, 8)
    assert torch.equal(proj, r['proj_dir'])
    do = torch.randn(1, 4, 4096, 64)
    return q, k, v, do


@pytest.mark.parametrize('tag', ['c0_noncausal', 'causal_2lvl', 'causal_odd', 'short_flash', 'causal_leaf', 'smooth'])
def test_module_restatement_matches_reference_glue(golden_dir, tag):
    """HyperAttentionOracle against the reference's own HyperAttention.forward run on CPU (float32)."""
    r = _load(golden_dir, f'module_{tag}.pt')
    q, k, v, do = _module_inputs(r)
    q, k, v = [t.clone().requires_grad_() for t in (q, k, v)]
    mod = O.HyperAttentionOracle(r['proj_dir'], r['block_size'], r['sample_size'], r['min_seq_len'], r['smooth_block'])
    o, lse = mod(q, k, v, causal=r['causal'], return_lse=True)
    o.backward(do)
    st = r.get('row_stride', 1)
    n = q.shape[2]
    assert lse.shape == r['lse'].shape          # includes the reference's rank-3 / padded cases
    sel = lambda t: t[:, :, ::st]
    assert rel(sel(o), r['o']) < 1e-5
    if lse.dim() == 4:
        assert rel(lse[:, :, :n], r['lse'][:, :, :n]) < 1e-6
    else:
        assert rel(lse[:, :, :n], r['lse'][:, :, :n]) < 1e-6
    assert rel(sel(q.grad), r['dq']) < 1e-4
    assert rel(sel(k.grad), r['dk']) < 1e-4
    assert rel(sel(v.grad), r['dv']) < 1e-4
    if 'q_codes' in r:
        qc = O.lsh_hash(q.detach(), r['proj_dir'])
        kc = O.lsh_hash(k.detach(), r['proj_dir'])
        tq = O.lsh_tie_mask(q.detach(), r['proj_dir'])
        assert not ((qc != r['q_codes'].int()) & ~tq).any()
        assert torch.equal(qc, r['q_codes'].int()) and torch.equal(kc, r['k_codes'].int())
        assert torch.equal(O.stable_argsort(qc), r['q_sort_idx'].long() & 0xFFFF)
        assert torch.equal(O.stable_argsort(kc), r['k_sort_idx'].long() & 0xFFFF)


def test_causal_schedule_trace():
    """hyper_attention.py:51-96: n=1024, min_seq_len=256 -> rectangles of 512 and 256 rows, one causal leaf call
    on 4x the heads with 256 rows."""
    torch.manual_seed(0)
    proj = torch.randn(1, 1, 16, 4)
    mod = O.HyperAttentionOracle(proj, 128, 128, 256, False)
    q, k, v = [torch.randn(1, 2, 1024, 16) for _ in range(3)]
    mod(q, k, v, causal=True)
    kinds = [(t[0], t[1][1], t[1][2], t[2]) for t in mod.trace]
    assert kinds == [('flash', 8, 256, True), ('hyper', 4, 256, False), ('hyper', 2, 512, False)]


def test_merge_formulas_agree_up_to_rounding():
    torch.manual_seed(1)
    a1, a2 = torch.randn(2, 3, 8, 4), torch.randn(2, 3, 8, 4)
    l1, l2 = torch.randn(2, 3, 8, 1), torch.randn(2, 3, 8, 1)
    o_r, l_r = O.add_self_attentions(a1, l1, a2, l2)
    o_e, l_e = O.merge_exact(a1, l1, a2, l2)
    assert rel(o_r, o_e) < 1e-5 and rel(l_r, l_e) < 1e-5
