"""CPU oracle for the HyperAttention hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain PyTorch running on host cores, what the reference computes on the path
hash -> stable sort -> block-diagonal + sampled-column attention -> LSE merge -> causal half-split
recursion, forward and backward.  It exists to check the CUDA kernels and to serve as the timed CPU
baseline.  The product package never imports it: only the test-suite, the smoke check and the
benchmark's CPU-baseline leg do.

Parity status: the restatement is pinned against the reference itself.  The golden fixtures under
``tests/golden`` were produced by running the reference's own Python glue (``hyper_attention.py``)
and its own Triton kernels (under the Triton interpreter, fp16) and are compared with this file by
the CPU test-suite.  The one mode with no counterpart in the reference -- ``sample_idx`` other than
``arange(sample_size)`` -- is "parity unpinned".

Reference lines each function follows are cited by path inside the reference project.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

TILE = 128  # the reference's BLOCK_M = BLOCK_N (src/hyper_attn_triton.py:723-724)


# --------------------------------------------------------------------------------------------
# Angular LSH  (src/angular_lsh_triton.py:168-179 and the kernel :70-96)
# --------------------------------------------------------------------------------------------
def gray_table(num_projs: int) -> torch.Tensor:
    """perm[b] = b ^ (b >> 1): the table built recursively at src/angular_lsh_triton.py:168-173."""
    b = torch.arange(2 ** num_projs, dtype=torch.int64)
    return (b ^ (b >> 1)).to(torch.int32)


def lsh_projections(x: torch.Tensor, proj_dir: torch.Tensor) -> torch.Tensor:
    """x [..., n, d] times proj_dir [d, r] in float64 from the values as stored (no re-rounding)."""
    return x.to(torch.float64) @ proj_dir.reshape(proj_dir.shape[-2], proj_dir.shape[-1]).to(torch.float64)


def lsh_hash(x: torch.Tensor, proj_dir: torch.Tensor) -> torch.Tensor:
    """code = gray( sum_j 2^j [x . P_j > 0] ), int32, shape x.shape[:-1].

    Follows src/angular_lsh_triton.py:77-88 (strict '> 0', weights 2^j, table lookup).  The sum over
    d is done in float64, so the only tokens whose code can differ from an fp32-accumulating kernel
    are those with a projection within rounding distance of zero; see lsh_tie_mask.
    """
    r = proj_dir.shape[-1]
    bits = lsh_projections(x, proj_dir) > 0
    weights = (2 ** torch.arange(r, dtype=torch.int64))
    bin_ids = (bits.to(torch.int64) * weights).sum(-1)
    return gray_table(r)[bin_ids]


def lsh_tie_mask(x: torch.Tensor, proj_dir: torch.Tensor, rel: float = 2.0 ** -18) -> torch.Tensor:
    """True where some projection is so close to zero that fp32 summation order may flip its sign."""
    p2 = proj_dir.reshape(proj_dir.shape[-2], proj_dir.shape[-1]).to(torch.float64)
    proj = x.to(torch.float64) @ p2
    mag = x.to(torch.float64).abs() @ p2.abs()
    return (proj.abs() <= rel * mag).any(-1)


def stable_argsort(codes: torch.Tensor) -> torch.Tensor:
    """hyper_attention.py:116-117: torch.sort(codes, dim=2, stable=True) -> indices (int64)."""
    return torch.sort(codes, dim=-1, stable=True)[1]


# --------------------------------------------------------------------------------------------
# Index patterns of the fused kernel
# --------------------------------------------------------------------------------------------
def _cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def block_window_positions(n: int, block_size: int, smooth_block: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """For every 128-row tile t of one side, the sorted positions on the other side it pairs with.

    Forward (src/hyper_attn_triton.py:101-111): query tile t -> key positions.  The reference backward
    (src/hyper_attn_triton.py:289-325) applies the very same formula with the roles swapped
    (key tile t -> query positions).  Returns (pos [T, Bs'], valid [T, Bs']) with Bs' the block size
    rounded up to a multiple of 128 (triton.cdiv at :726).
    """
    bs = _cdiv(block_size, TILE)
    width = bs * TILE
    n_tiles = n // TILE
    t = torch.arange(n_tiles, dtype=torch.int64)
    beta = t // bs
    j = torch.arange(width, dtype=torch.int64)
    base = beta[:, None] * width + j[None, :]
    valid = base < torch.clamp((beta[:, None] + 1) * width, max=n)
    # the loop runs over whole 128-wide tiles starting below end_n (:104)
    tile_start = (base // TILE) * TILE
    valid = tile_start < torch.clamp((beta[:, None] + 1) * width, max=n)
    if smooth_block:
        offs = n + (t % bs) * TILE - ((bs - 1) * TILE) // 2
        pos = (base + offs[:, None]) % n
    else:
        pos = torch.where(valid, base, torch.zeros_like(base))
    return pos, valid


def _default_sample_idx(sample_size: int, device=None) -> torch.Tensor:
    s = _cdiv(sample_size, TILE) * TILE
    return torch.arange(s, dtype=torch.int64, device=device)


# --------------------------------------------------------------------------------------------
# Fused block-diagonal + sampled attention, one (batch, head) at a time
# --------------------------------------------------------------------------------------------
def uniform_sample_idx(seed: int, call: int, rows: int, sample_size: int, n: int) -> torch.Tensor:
    """Sampled key rows of the uniform mode: int64 [rows, sample_size], row = batch * heads + head.

    One draw from each of sample_size equal strata of [0, n): slot s of row r takes
    start_s + ((size_s * u) >> 24) with u = the top 24 bits of mix64(seed, call, r * sample_size + s), where mix64 is the
    splitmix64 finaliser.  Pure integer arithmetic in numpy uint64 -- a function of (seed, call, r, s) only, so the
    module (which evaluates the same function with torch integer ops on the device) and this restatement agree bit for
    bit.  No counterpart in the mounted reference (its sampled part reads rows 0..sample_size-1)."""
    import numpy as np
    with np.errstate(over='ignore'):
        ctr = np.arange(rows * sample_size, dtype=np.uint64)
        x = (np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15) + np.uint64(call) * np.uint64(0xD1B54A32D192ED03) + ctr)
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        x = x ^ (x >> np.uint64(31))
    u24 = (x >> np.uint64(40)).astype(np.int64).reshape(rows, sample_size)
    edges = (np.arange(sample_size + 1, dtype=np.int64) * n) // sample_size
    start, size = edges[:-1], edges[1:] - edges[:-1]
    return torch.from_numpy(start[None, :] + ((size[None, :] * u24) >> 24))


def sample_tile_weights(n, ki, block_size, sample_idx, smooth):
    """Weighted sampling (no counterpart in the mounted reference; "parity unpinned"): for every sorted query tile t,
    which sampled slots are dropped because their key already lies in the tile's block window, and the log of the
    importance weight (n - window size) / (number of kept slots) that makes the kept samples stand for all keys
    outside the window.  Returns (masked [T, S] bool, logw [T] float; -inf where nothing is kept)."""
    pos, valid = block_window_positions(n, block_size, smooth)
    inv = torch.empty(n, dtype=torch.int64)
    inv[ki] = torch.arange(n)
    spos = inv[sample_idx]                                           # sorted position of every sampled key
    count = valid.sum(-1)                                            # window size per tile
    first = pos[:, 0]
    masked = ((spos[None, :] - first[:, None]) % n) < count[:, None]
    kept = (~masked).sum(-1)
    logw = torch.where(kept > 0, torch.log((n - count).float() / kept.clamp_min(1).float()), torch.full((len(count),), float('-inf')))
    return masked, logw


def _hyper_fwd_head(q, k, v, qi, ki, block_size, sample_idx, scale, smooth, weighted=False):
    """q,k [n,d], v [n,dv] float32; qi,ki [n] int64; returns o [n,dv], lse [n] at original rows.

    src/hyper_attn_triton.py:70-192: for the sorted query tile t the key multiset is the block window
    (gathered through k_sort_idx) followed by the sampled rows (original order); one softmax over both.
    weighted=True switches the sampled part to the importance-weighted estimator of sample_tile_weights.
    """
    n, d = q.shape
    n_tiles = n // TILE
    pos, valid = block_window_positions(n, block_size, smooth)
    qs = q[qi].view(n_tiles, TILE, d)
    krows = ki[pos]                                   # [T, W]
    kb = k[krows]                                     # [T, W, d]
    vb = v[krows]
    s_blk = torch.einsum('tmd,twd->tmw', qs, kb) * scale
    s_blk = s_blk.masked_fill(~valid[:, None, :], float('-inf'))
    if sample_idx is not None and sample_idx.numel() > 0:
        ksm = k[sample_idx]
        vsm = v[sample_idx]
        s_smp = torch.einsum('tmd,sd->tms', qs, ksm) * scale
        if weighted:
            masked, logw = sample_tile_weights(n, ki, block_size, sample_idx, smooth)
            s_smp = (s_smp + logw[:, None, None]).masked_fill(masked[:, None, :], float('-inf'))
            s_smp = torch.nan_to_num(s_smp, nan=float('-inf'))
        s_all = torch.cat([s_blk, s_smp], dim=-1)
    else:
        s_all = s_blk
    lse_s = torch.logsumexp(s_all, dim=-1)            # [T, 128]
    p = torch.exp(s_all - lse_s[..., None])
    w = s_blk.shape[-1]
    o_s = torch.einsum('tmw,twe->tme', p[..., :w], vb)
    if s_all.shape[-1] > w:
        o_s = o_s + torch.einsum('tms,se->tme', p[..., w:], vsm)
    o = torch.empty(n, v.shape[-1], dtype=q.dtype)
    lse = torch.empty(n, dtype=q.dtype)
    o[qi] = o_s.reshape(n, -1)
    lse[qi] = lse_s.reshape(n)
    return o, lse


def _hyper_bwd_head(q, k, v, qi, ki, do, lse, delta, block_size, sample_idx, scale, smooth, exact_pattern, weighted=False):
    """Gradients for one head (all float32, original row order).

    src/hyper_attn_triton.py:289-388 (block part, enumerated per sorted *key* tile) and :573-663
    (sampled part: rows sample_idx against every query).  p = exp(s - lse_i); dV += p^T dO;
    dP = dO V^T; dS = p (dP - delta) scale; dK += dS^T Q; dQ += dS K.
    With smooth_block the reference's key-tile window is not the transpose of its forward window;
    exact_pattern=True enumerates the forward's pair set instead.
    """
    n, d = q.shape
    dv_dim = v.shape[-1]
    n_tiles = n // TILE
    dq = torch.zeros_like(q)
    dk = torch.zeros_like(k)
    dv = torch.zeros_like(v)
    pos, valid = block_window_positions(n, block_size, smooth)
    if exact_pattern or not smooth:
        # query tile major (the forward's pair set)
        qrows = qi.view(n_tiles, TILE)                # [T,128]
        krows = ki[pos]                               # [T,W]
        qs, dos = q[qrows], do[qrows]
        ls, dl = lse[qrows], delta[qrows]
        kb, vb = k[krows], v[krows]
        s = torch.einsum('tmd,twd->tmw', qs, kb) * scale
        p = torch.exp(s - ls[..., None]) * valid[:, None, :]
        dp = torch.einsum('tme,twe->tmw', dos, vb)
        ds = p * (dp - dl[..., None]) * scale
        dq.index_add_(0, qrows.reshape(-1), torch.einsum('tmw,twd->tmd', ds, kb).reshape(-1, d))
        dk.index_add_(0, krows.reshape(-1), torch.einsum('tmw,tmd->twd', ds, qs).reshape(-1, d))
        dv.index_add_(0, krows.reshape(-1), torch.einsum('tmw,tme->twe', p, dos).reshape(-1, dv_dim))
    else:
        # key tile major with the forward's window formula applied to query positions (:290-325)
        krows = ki.view(n_tiles, TILE)
        qrows = qi[pos]                               # [T,W]
        kb, vb = k[krows], v[krows]
        qs, dos = q[qrows], do[qrows]
        ls, dl = lse[qrows], delta[qrows]
        s = torch.einsum('twd,tnd->twn', qs, kb) * scale
        p = torch.exp(s - ls[..., None]) * valid[:, :, None]
        dp = torch.einsum('twe,tne->twn', dos, vb)
        ds = p * (dp - dl[..., None]) * scale
        dq.index_add_(0, qrows.reshape(-1), torch.einsum('twn,tnd->twd', ds, kb).reshape(-1, d))
        dk.index_add_(0, krows.reshape(-1), torch.einsum('twn,twd->tnd', ds, qs).reshape(-1, d))
        dv.index_add_(0, krows.reshape(-1), torch.einsum('twn,twe->tne', p, dos).reshape(-1, dv_dim))
    if sample_idx is not None and sample_idx.numel() > 0:
        ksm, vsm = k[sample_idx], v[sample_idx]
        s = (q @ ksm.t()) * scale
        if weighted:
            masked, logw = sample_tile_weights(n, ki, block_size, sample_idx, smooth)
            tile_of_row = torch.empty(n, dtype=torch.int64)
            tile_of_row[qi] = torch.arange(n) // TILE                  # sorted tile of every original row
            s = (s + logw[tile_of_row][:, None]).masked_fill(masked[tile_of_row], float('-inf'))
            s = torch.nan_to_num(s, nan=float('-inf'))
        p = torch.exp(s - lse[:, None])
        dp = do @ vsm.t()
        ds = p * (dp - delta[:, None]) * scale
        dq += ds @ ksm
        dk.index_add_(0, sample_idx, ds.t() @ q)
        dv.index_add_(0, sample_idx, p.t() @ do)
    return dq, dk, dv


def _to_bh(x):
    """[B, n, H, d] -> [B, H, n, d] float32 contiguous."""
    return x.transpose(1, 2).to(torch.float32).contiguous()


class _HyperAttnOracleFn(torch.autograd.Function):
    """Same calling convention and gradient conventions as HyperAttnFunc (src/hyper_attn_triton.py:895-945):
    inputs [B, n, H, d] views, o returned as [B, n, H, dv], lse [B, H, n]; the incoming gradient of lse
    is discarded (:923)."""

    @staticmethod
    def forward(ctx, q, k, v, q_sort_idx, k_sort_idx, block_size, sample_size, softmax_scale, smooth_block,
                sample_idx, exact_pattern, weighted=False):
        B, n, H, d = q.shape
        assert n % TILE == 0, 'sequence length must be divisible by 128 (src/hyper_attn_triton.py:695)'
        scale = softmax_scale or 1.0 / math.sqrt(d)
        qf, kf, vf = _to_bh(q), _to_bh(k), _to_bh(v)
        qi = q_sort_idx.transpose(1, 2).to(torch.int64)
        ki = k_sort_idx.transpose(1, 2).to(torch.int64)
        if sample_idx is None:
            sidx = _default_sample_idx(sample_size).expand(B, H, -1) if sample_size > 0 else None
        else:
            sidx = sample_idx.to(torch.int64)
        o = torch.empty(B, H, n, v.shape[-1], dtype=torch.float32)
        lse = torch.empty(B, H, n, dtype=torch.float32)
        for b in range(B):
            for h in range(H):
                o[b, h], lse[b, h] = _hyper_fwd_head(qf[b, h], kf[b, h], vf[b, h], qi[b, h], ki[b, h], block_size,
                                                     None if sidx is None else sidx[b, h], scale, bool(smooth_block), weighted)
        o_out = o.to(q.dtype).transpose(1, 2)          # [B, n, H, dv] view, like the reference's o
        ctx.save_for_backward(q, k, v, qi, ki, o_out, lse)
        ctx.sidx = sidx
        ctx.args = (block_size, scale, bool(smooth_block), bool(exact_pattern), bool(weighted))
        return o_out, lse

    @staticmethod
    def backward(ctx, do, dlse_unused=None):
        q, k, v, qi, ki, o, lse = ctx.saved_tensors
        block_size, scale, smooth, exact_pattern, weighted = ctx.args
        B, n, H, d = q.shape
        qf, kf, vf, dof, of = _to_bh(q), _to_bh(k), _to_bh(v), _to_bh(do), _to_bh(o)
        delta = (of * dof).sum(-1)                      # src/hyper_attn_triton.py:196-236
        dq = torch.empty_like(qf)
        dk = torch.empty_like(kf)
        dv = torch.empty_like(vf)
        for b in range(B):
            for h in range(H):
                dq[b, h], dk[b, h], dv[b, h] = _hyper_bwd_head(
                    qf[b, h], kf[b, h], vf[b, h], qi[b, h], ki[b, h], dof[b, h], lse[b, h], delta[b, h], block_size,
                    None if ctx.sidx is None else ctx.sidx[b, h], scale, smooth, exact_pattern, weighted)
        cast = lambda t, like: t.transpose(1, 2).to(like.dtype)
        return cast(dq, q), cast(dk, k), cast(dv, v), None, None, None, None, None, None, None, None, None


def hyper_attn_func(q, k, v, q_sort_idx, k_sort_idx, block_size, sample_size=0, softmax_scale=None,
                    smooth_block=False, sample_idx=None, exact_pattern=False, weighted=False):
    """Oracle twin of hyper_attn_func (src/hyper_attn_triton.py:948).  weighted=True (with an explicit sample_idx):
    importance-weighted sampled columns excluding the query tile's own block (sample_tile_weights)."""
    return _HyperAttnOracleFn.apply(q, k, v, q_sort_idx, k_sort_idx, block_size, sample_size, softmax_scale,
                                    smooth_block, sample_idx, exact_pattern, weighted)


# --------------------------------------------------------------------------------------------
# Exact attention (src/flash_attn_triton.py:149-241 forward, :342-625 backward)
# --------------------------------------------------------------------------------------------
def _flash_chunks(n_q: int, n_k: int) -> int:
    # bound the [chunk, n_k] score matrix to ~64 MB of float32
    return max(1, min(n_q, (16 * 1024 * 1024) // max(n_k, 1)))


class _FlashOracleFn(torch.autograd.Function):
    """FlashAttnFunc's conventions (src/flash_attn_triton.py:995-1042): [B, n, H, d] in, (o, lse) out with lse
    padded to a multiple of 128 rows (:826-827); causal means key j <= query i (:176-177); gradient of lse
    discarded (:1015)."""

    @staticmethod
    def forward(ctx, q, k, v, causal, softmax_scale):
        B, nq, H, d = q.shape
        nk = k.shape[1]
        scale = softmax_scale or 1.0 / math.sqrt(d)
        qf, kf, vf = _to_bh(q), _to_bh(k), _to_bh(v)
        o = torch.empty(B, H, nq, v.shape[-1], dtype=torch.float32)
        nq_r = _cdiv(nq, TILE) * TILE
        lse = torch.zeros(B, H, nq_r, dtype=torch.float32)
        ch = _flash_chunks(nq, nk)
        for s0 in range(0, nq, ch):
            s1 = min(nq, s0 + ch)
            kend = min(nk, s1) if causal else nk
            s = torch.einsum('bhmd,bhnd->bhmn', qf[:, :, s0:s1], kf[:, :, :kend]) * scale
            if causal:
                i = torch.arange(s0, s1)[:, None]
                j = torch.arange(kend)[None, :]
                s = s.masked_fill(j > i, float('-inf'))
            l = torch.logsumexp(s, dim=-1)
            lse[:, :, s0:s1] = l
            o[:, :, s0:s1] = torch.einsum('bhmn,bhne->bhme', torch.exp(s - l[..., None]), vf[:, :, :kend])
        o_out = o.to(q.dtype).transpose(1, 2)
        ctx.save_for_backward(q, k, v, o_out, lse)
        ctx.causal, ctx.scale = causal, scale
        return o_out, lse

    @staticmethod
    def backward(ctx, do, dlse_unused=None):
        q, k, v, o, lse = ctx.saved_tensors
        causal, scale = ctx.causal, ctx.scale
        B, nq, H, d = q.shape
        nk = k.shape[1]
        qf, kf, vf, dof, of = _to_bh(q), _to_bh(k), _to_bh(v), _to_bh(do), _to_bh(o)
        delta = (of * dof).sum(-1)
        dq = torch.zeros_like(qf)
        dk = torch.zeros_like(kf)
        dv = torch.zeros_like(vf)
        ch = _flash_chunks(nq, nk)
        for s0 in range(0, nq, ch):
            s1 = min(nq, s0 + ch)
            kend = min(nk, s1) if causal else nk
            s = torch.einsum('bhmd,bhnd->bhmn', qf[:, :, s0:s1], kf[:, :, :kend]) * scale
            p = torch.exp(s - lse[:, :, s0:s1, None])
            if causal:
                i = torch.arange(s0, s1)[:, None]
                j = torch.arange(kend)[None, :]
                p = p.masked_fill(j > i, 0.0)
            dp = torch.einsum('bhme,bhne->bhmn', dof[:, :, s0:s1], vf[:, :, :kend])
            ds = p * (dp - delta[:, :, s0:s1, None]) * scale
            dq[:, :, s0:s1] = torch.einsum('bhmn,bhnd->bhmd', ds, kf[:, :, :kend])
            dk[:, :, :kend] += torch.einsum('bhmn,bhmd->bhnd', ds, qf[:, :, s0:s1])
            dv[:, :, :kend] += torch.einsum('bhmn,bhme->bhne', p, dof[:, :, s0:s1])
        cast = lambda t, like: t.transpose(1, 2).to(like.dtype)
        return cast(dq, q), cast(dk, k), cast(dv, v), None, None


def flash_attn_func(q, k, v, bias=None, causal=False, softmax_scale=None):
    """Oracle twin of flash_attn_func (src/flash_attn_triton.py:1042).  bias is never passed on this path
    (hyper_attention.py:56, :113) and is rejected here."""
    assert bias is None, 'the attention-bias branch is outside the HyperAttention path'
    return _FlashOracleFn.apply(q, k, v, causal, softmax_scale)


# --------------------------------------------------------------------------------------------
# LSE merge  (src/attn_utils.py:6-24)
# --------------------------------------------------------------------------------------------
def add_self_attentions(attn1, lse1, attn2, lse2):
    """c = 1/(1+exp(lse2-lse1)) rounded to attn's dtype; attn = c a1 + (1-c) a2; lse = lse1 - log(c + eps)."""
    c = (1.0 / (1.0 + torch.exp(lse2 - lse1))).to(attn1.dtype)
    attn = c * attn1 + (1 - c) * attn2
    lse = lse1 - torch.log(c + torch.finfo(lse1.dtype).eps)
    return attn, lse


def merge_exact(attn1, lse1, attn2, lse2):
    """The same combination without the dtype rounding of c and without eps (log-sum-exp of the two)."""
    m = torch.maximum(lse1, lse2)
    w1, w2 = torch.exp(lse1 - m), torch.exp(lse2 - m)
    lse = m + torch.log(w1 + w2)
    attn = (attn1.float() * w1 + attn2.float() * w2) / (w1 + w2)
    return attn.to(attn1.dtype), lse


# --------------------------------------------------------------------------------------------
# Module-level restatement  (hyper_attention.py:25-132)
# --------------------------------------------------------------------------------------------
class HyperAttentionOracle:
    """Host-side orchestration of the reference module, restated.

    hash_fn(x [B,H,n,d]) -> int codes.  By default the float64 hash above with the stored proj_dir.
    grad conventions are those of the two Functions above, so autograd through this object reproduces
    the reference's gradients (including its dropped d(lse) terms).
    """

    def __init__(self, proj_dir: torch.Tensor, block_size=256, sample_size=256, min_seq_len=2048,
                 smooth_block=False, hash_fn=None, exact_pattern=False):
        self.proj_dir = proj_dir
        self.block_size = block_size
        self.sample_size = sample_size
        self.min_seq_len = min_seq_len
        self.smooth_block = smooth_block
        self.exact_pattern = exact_pattern
        self.hash_fn = hash_fn or (lambda x: lsh_hash(x, self.proj_dir))
        self.trace = []  # (kind, shape) of every attention call, for schedule checks

    # hyper_attention.py:103-132
    def no_causal(self, q, k, v, scale):
        n = q.shape[2]
        if self.min_seq_len > n:
            self.trace.append(('flash', tuple(q.shape), False))
            o, lse = flash_attn_func(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), None, False, scale)
        else:
            self.trace.append(('hyper', tuple(q.shape), False))
            qi = stable_argsort(self.hash_fn(q))
            ki = stable_argsort(self.hash_fn(k))
            o, lse = hyper_attn_func(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), qi.transpose(1, 2),
                                     ki.transpose(1, 2), self.block_size, self.sample_size, scale,
                                     self.smooth_block, None, self.exact_pattern)
        return o.transpose(1, 2), lse.unsqueeze(-1)

    # hyper_attention.py:25-101
    def __call__(self, q, k, v, scale=None, causal=False, return_lse=False):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        B, H, n, d = k.shape
        assert q.shape[2] == n
        scale = scale or d ** (-0.5)
        if not causal:
            o, lse = self.no_causal(q, k, v, scale)
        elif n <= self.min_seq_len:
            self.trace.append(('flash', tuple(q.shape), True))
            o, lse = flash_attn_func(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), None, True, scale)
            o = o.transpose(1, 2)          # lse stays [B, H, n_rounded] here, as in the reference (:52-57)
        else:
            odd = n % 2
            if odd:
                pad = lambda t: torch.nn.functional.pad(t, (0, 0, 0, 1))
                q, k, v = pad(q), pad(k), pad(v)
            m = q.shape[2] // 2
            fold = lambda t: t.reshape(B, 2 * H, m, t.shape[-1])
            o_d, l_d = self(fold(q), fold(k), fold(v), scale, True, True)
            o_d = o_d.reshape(B, H, 2 * m, -1)
            l_d = l_d.reshape(B, H, 2 * m, 1)
            o_r, l_r = self.no_causal(q[:, :, m:], k[:, :, :m], v[:, :, :m], scale)
            o_low, l_low = add_self_attentions(o_d[:, :, m:], l_d[:, :, m:], o_r, l_r)
            o = torch.cat([o_d[:, :, :m], o_low], dim=2)
            lse = torch.cat([l_d[:, :, :m], l_low], dim=2)
            if odd:
                o, lse = o[:, :, :-1], lse[:, :, :-1]
        return (o, lse) if return_lse else o
