"""True-gradient companion of the oracle.  TEST INFRASTRUCTURE ONLY.

hyper_oracle.py reproduces the reference's gradient conventions (both attention Functions drop the gradient that
flows into their log-sum-exp output, src/hyper_attn_triton.py:923 and src/flash_attn_triton.py:1015).  This file
computes, with plain differentiable PyTorch ops, the same forward values and lets autograd differentiate them in
full (merge without rounding), which is what the module's grad_mode='exact' + merge_mode='exact' promises.
Parity of this mode is not pinned by the reference (it has no such mode).
"""
import torch

from . import hyper_oracle as O


def _dense_causal(q, k, v, scale):
    n = q.shape[2]
    s = torch.einsum('bhmd,bhnd->bhmn', q, k) * scale
    mask = torch.ones(n, n, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float('-inf'))
    lse = torch.logsumexp(s, dim=-1, keepdim=True)
    return torch.exp(s - lse) @ v, lse


def _hyper_rect(q, k, v, proj, block, sample, scale, smooth):
    B, H, n, _ = q.shape
    qi = O.stable_argsort(O.lsh_hash(q.detach(), proj))
    ki = O.stable_argsort(O.lsh_hash(k.detach(), proj))
    sidx = O._default_sample_idx(sample) if sample > 0 else None
    outs, lses = [], []
    for b in range(B):
        for h in range(H):
            o, l = O._hyper_fwd_head(q[b, h], k[b, h], v[b, h], qi[b, h], ki[b, h], block, sidx, scale, smooth)
            outs.append(o)
            lses.append(l)
    return torch.stack(outs).view(B, H, n, -1), torch.stack(lses).view(B, H, n, 1)


def _rec(q, k, v, proj, block, sample, msl, scale, smooth):
    B, H, n, d = q.shape
    if n <= msl:
        return _dense_causal(q, k, v, scale)
    m = n // 2
    fold = lambda t: t.reshape(B, 2 * H, m, t.shape[-1])
    o_d, l_d = _rec(fold(q), fold(k), fold(v), proj, block, sample, msl, scale, smooth)
    o_d, l_d = o_d.reshape(B, H, n, -1), l_d.reshape(B, H, n, 1)
    o_r, l_r = _hyper_rect(q[:, :, m:], k[:, :, :m], v[:, :, :m], proj, block, sample, scale, smooth)
    o_low, l_low = O.merge_exact(o_d[:, :, m:], l_d[:, :, m:], o_r, l_r)
    return torch.cat([o_d[:, :, :m], o_low], 2), torch.cat([l_d[:, :, :m], l_low], 2)


def causal_exact_gradient(q, k, v, do, proj, block, sample, msl, smooth=False):
    q, k, v = [t.detach().float().clone().requires_grad_() for t in (q, k, v)]
    o, _ = _rec(q, k, v, proj, block, sample, msl, q.shape[-1] ** -0.5, smooth)
    o.backward(do.float())
    return o.detach(), (q.grad, k.grad, v.grad)
