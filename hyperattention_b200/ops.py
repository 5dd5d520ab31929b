"""Torch-facing operators over the C ABI: hashing, segmented sort, gather, the two attention Functions and the fused
causal Function.  PyTorch only provides device memory, streams and autograd plumbing here; all arithmetic on the path
runs in libhyperattn_b200.so.

Secondary API names mirror the reference's: hyper_attn_func (src/hyper_attn_triton.py:948), flash_attn_func
(src/flash_attn_triton.py:1042), add_self_attentions and indexing (src/attn_utils.py).
"""
import ctypes as C
import math

import torch

from . import _lib as L

_DT = {torch.bfloat16: L.BF16, torch.float16: L.FP16, torch.float32: L.FP32}


def _dtype_id(t):
    assert t.dtype in _DT, 'Only support fp16, bf16 and fp32'
    return _DT[t.dtype]


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


_STATUS = {}


def _status_words(device):
    """Per device: the int32 word in device memory that the kernels set when a bounded device-side wait expires
    (0 = healthy; CTAs that start later see it and return at once), and its twin in pinned host memory, which the
    kernels write as well and the host can read without synchronising."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _STATUS:
        _STATUS[key] = (torch.zeros(1, dtype=torch.int32, device=f'cuda:{key}'),
                        torch.zeros(1, dtype=torch.int32).pin_memory())
    return _STATUS[key]


def _status_word(device):
    return _status_words(device)[0]


def _set_status(p, device):
    """Fills the status pointers of a parameter struct.  Before that, looks at the host-visible word: a timeout
    reported by an earlier launch raises here, at the next call into the library, instead of going unnoticed (the
    outputs of the launch that timed out, and of everything launched since, are undefined)."""
    dev_w, host_w = _status_words(device)
    _raise_if_failed(dev_w, host_w)
    p.status, p.status_host = _ptr(dev_w), C.c_void_p(host_w.data_ptr())


def _status_text(v):
    return {L.DEV_TIMEOUT: 'a device-side wait timed out',
            L.DEV_BAD_INDEX: 'an index array holds a row outside its segment (index check)',
            L.DEV_BAD_LAUNCH: 'a kernel found its shared-memory window too small and did no work'}.get(v, 'the device reported a failure')


def _raise_if_failed(dev_w, host_w):
    v = int(host_w[0])
    if v != 0:
        host_w.zero_()
        dev_w.zero_()
        raise RuntimeError(f'hyperattention_b200: {_status_text(v)} in an earlier launch (status {v}); '
                           'results produced since then are undefined')


def check_device_status(device=None, reset=True):
    """Synchronises and raises if a kernel reported a timeout since the last check."""
    dev_w, host_w = _status_words(device if device is not None else torch.cuda.current_device())
    v = int(dev_w.item()) | int(host_w[0])
    if v != 0:
        if reset:
            dev_w.zero_()
            host_w.zero_()
        raise RuntimeError(f'hyperattention_b200: {_status_text(v)} (status {v})')


def _cuda(*ts):
    for t in ts:
        assert t is not None and t.is_cuda, 'tensors must be CUDA tensors (there is no CPU implementation)'


# ------------------------------------------------------------------------------------------------
def lsh_hash(x, proj_f32, out=None):
    """codes int32 [B,H,n] for x [B,H,n,d]; proj_f32 float32 [d, r] on the same device
    (replaces AngularLSHTriton.hash_triton, src/angular_lsh_triton.py:181-182).  out: optional contiguous int32
    [B,H,n] tensor to write into (lets q and k codes share one buffer and one sort call)."""
    _cuda(x, proj_f32)
    assert x.dim() == 4 and x.stride(-1) == 1
    B, H, n, d = x.shape
    assert proj_f32.dtype == torch.float32 and proj_f32.is_contiguous() and proj_f32.shape[0] == d
    r = proj_f32.shape[1]
    codes = out if out is not None else torch.empty(B, H, n, dtype=torch.int32, device=x.device)
    assert codes.shape == (B, H, n) and codes.dtype == torch.int32 and codes.is_contiguous() and codes.device == x.device
    with torch.cuda.device(x.device):
        rc = L.load().ha_lsh_hash(_ptr(x), x.stride(0), x.stride(1), x.stride(2), B, H, n, d, _dtype_id(x), _ptr(proj_f32), r,
                                  _ptr(codes), _stream())
    L.check(rc, 'ha_lsh_hash')
    return codes


def seg_sort(codes, key_bits=8, span=None, seg_off=0, seg_len=None):
    """Stable ascending argsort of every segment; codes int32 [..., n]; returns int32 [rows*(n/span), seg_len] of
    segment-local indices (replaces torch.sort(..., stable=True)[1], hyper_attention.py:116-117)."""
    _cuda(codes)
    assert codes.dtype == torch.int32 and codes.is_contiguous()
    n = codes.shape[-1]
    rows = codes.numel() // max(n, 1)
    span = n if span is None else span
    seg_len = span - seg_off if seg_len is None else seg_len
    lib = L.load()
    idx = torch.empty(rows * (n // span) if span else 0, seg_len, dtype=torch.int32, device=codes.device)
    if idx.numel() == 0:
        return idx
    ws_bytes = lib.ha_seg_sort_workspace_bytes(rows, n, span, seg_len, key_bits)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=codes.device)
    with torch.cuda.device(codes.device):
        rc = lib.ha_seg_sort(_ptr(codes), rows, n, span, seg_off, seg_len, key_bits, _ptr(idx), _ptr(ws), ws_bytes, _stream())
    L.check(rc, 'ha_seg_sort')
    return idx


def indexing(x, indices, chunk_size=-1):
    """out[b,h,i,:] = x[b,h,indices[b,h,i],:] (src/attn_utils.py:27-50); rows padded with zeros up to a multiple of
    chunk_size when chunk_size > 0."""
    _cuda(x, indices)
    assert x.dim() == 4 and x.stride(-1) == 1
    B, H, n, w = x.shape
    idx = indices.to(torch.int32).contiguous()
    s = idx.shape[-1]
    out = torch.empty(B, H, s, w, dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = L.load().ha_gather_rows(_ptr(x), x.stride(0), x.stride(1), x.stride(2), B, H, w, _dtype_id(x), _ptr(idx), s, _ptr(out),
                                     _stream())
    L.check(rc, 'ha_gather_rows')
    if chunk_size > 0 and s % chunk_size != 0:
        new_s = math.ceil(s / chunk_size) * chunk_size
        out = torch.nn.functional.pad(out, (0, 0, 0, new_s - s))
    return out


def lse_merge_(o1, lse1, o2, lse2, exact=False):
    """In-place (o1, lse1) <- merge with (o2, lse2) by ha_lse_merge; o* [..., dv] contiguous, lse* [...] float32."""
    _cuda(o1, lse1, o2, lse2)
    assert o1.is_contiguous() and o2.is_contiguous() and lse1.is_contiguous() and lse2.is_contiguous()
    assert lse1.dtype == torch.float32 and lse2.dtype == torch.float32 and o1.dtype == o2.dtype
    dv = o1.shape[-1]
    rows = o1.numel() // dv
    assert lse1.numel() == rows and lse2.numel() == rows
    with torch.cuda.device(o1.device):
        rc = L.load().ha_lse_merge(_ptr(o1), _ptr(lse1), _ptr(o2), _ptr(lse2), rows, dv, _dtype_id(o1), int(exact), _stream())
    L.check(rc, 'ha_lse_merge')
    return o1, lse1


def add_self_attentions(attn1, lse1, attn2, lse2):
    """src/attn_utils.py:6-24, differentiable (elementwise torch ops, any device)."""
    c = (1 / (1 + (lse2 - lse1).exp())).to(dtype=attn1.dtype)
    attn = c * attn1 + (1 - c) * attn2
    lse = lse1 - (c + torch.finfo(lse1.dtype).eps).log()
    return attn, lse


# ------------------------------------------------------------------------------------------------
def _bhn(t):
    """(stride_b, stride_h, stride_n) of a [B, n, H, d] view."""
    return t.stride(0), t.stride(2), t.stride(1)


def _fill_qkv(p, q, k, v):
    p.q, p.k, p.v = _ptr(q), _ptr(k), _ptr(v)
    p.q_sb, p.q_sh, p.q_sn = _bhn(q)
    p.k_sb, p.k_sh, p.k_sn = _bhn(k)
    p.v_sb, p.v_sh, p.v_sn = _bhn(v)


def _idx_rows(idx, B, n, H):
    """[B, n, H] (any int dtype, any strides) -> contiguous int32 [B*H, n]."""
    assert idx.shape == (B, n, H)
    return idx.transpose(1, 2).to(torch.int32).contiguous().view(B * H, n)


def sample_weights(k_idx_rows, sample_rows, n, block_size, sample_size, smooth_block):
    """Per sorted query tile: log importance weight of the kept sampled slots and the bit mask of the dropped ones
    (ha_sample_weights).  k_idx_rows int32 [segs, n]; sample_rows int32 [segs, sample_size] or None (rows 0..S-1).
    Returns (logw float32 [segs, n/128], mask int32 [segs, n/128, sample_size/32])."""
    segs = k_idx_rows.shape[0]
    dev = k_idx_rows.device
    inv = torch.empty(segs, n, dtype=torch.int32, device=dev)
    logw = torch.empty(segs, n // 128, dtype=torch.float32, device=dev)
    mask = torch.empty(segs, n // 128, sample_size // 32, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = L.load().ha_sample_weights(_ptr(k_idx_rows), _ptr(sample_rows), segs, n, block_size, sample_size,
                                        1 if smooth_block else 0, _ptr(inv), _ptr(logw), _ptr(mask), _stream())
    L.check(rc, 'ha_sample_weights')
    return logw, mask


class HyperAttnFunc(torch.autograd.Function):
    """Drop-in for HyperAttnFunc (src/hyper_attn_triton.py:895-945): q, k, v [B, n, H, d] views, permutations
    [B, n, H]; returns o [B, n, H, dv] and lse [B, H, n]; the gradient flowing into lse is discarded, as there."""

    @staticmethod
    def forward(ctx, q, k, v, q_sort_idx, k_sort_idx, block_size, sample_size=0, softmax_scale=None, smooth_block=False,
                sample_idx=None, flags=0, weighted=False):
        _cuda(q, k, v, q_sort_idx, k_sort_idx)
        q, k, v = [x if x.stride(-1) == 1 else x.contiguous() for x in (q, k, v)]
        assert sample_size % 128 == 0
        B, n, H, d = q.shape
        assert k.shape == (B, n, H, d), 'query and key sequence lengths must be equal'
        assert v.shape[:3] == (B, n, H)
        assert q.dtype == k.dtype == v.dtype, 'All tensors must have the same type'
        assert n % 128 == 0, 'keys sequence length must be divisible by 128'
        dv = v.shape[-1]
        scale = softmax_scale or 1.0 / math.sqrt(d)
        qi = _idx_rows(q_sort_idx, B, n, H)
        ki = _idx_rows(k_sort_idx, B, n, H)
        si = None
        if sample_idx is not None and sample_size > 0:
            si = sample_idx.to(torch.int32).contiguous().view(B * H, sample_size)
        # memory is [B, H, n, dv]; the reference-shaped [B, n, H, dv] result is a view of it
        o = torch.empty(B, H, n, dv, dtype=q.dtype, device=q.device).transpose(1, 2)
        lse = torch.empty(B, H, n, dtype=torch.float32, device=q.device)
        p = L.AttnParams()
        p.mode, p.dtype = L.MODE_HYPER, _dtype_id(q)
        p.flags = (L.FLAG_SMOOTH if smooth_block else 0) | flags
        p.B, p.H, p.n, p.d, p.dv = B, H, n, d, dv
        p.segs_per_head, p.span, p.q_off, p.k_off, p.m_q, p.m_k = 1, n, 0, 0, n, n
        p.block_size, p.sample_size, p.scale = block_size, sample_size, scale
        _fill_qkv(p, q, k, v)
        p.q_idx, p.k_idx, p.sample_idx = _ptr(qi), _ptr(ki), _ptr(si)
        p.o = _ptr(o)
        p.o_sb, p.o_sh, p.o_sn = _bhn(o)
        p.lse = _ptr(lse)
        _set_status(p, q.device)
        wts = None
        if weighted and sample_size > 0:
            # importance-weighted sampled columns, the query tile's own block excluded (not in the reference's code)
            wts = sample_weights(ki, si, n, block_size, sample_size, smooth_block)
            p.sample_logw, p.sample_mask = _ptr(wts[0]), _ptr(wts[1])
        with torch.cuda.device(q.device):
            rc = L.load().ha_attn_fwd(C.byref(p), _stream())
        L.check(rc, 'ha_attn_fwd')
        empty = torch.empty(0, device=q.device)
        ctx.save_for_backward(q, k, v, qi, ki, o, lse, si if si is not None else empty,
                              *(wts if wts is not None else (empty, empty)))
        ctx.cfg = (block_size, sample_size, scale, p.flags, si is not None, wts is not None)
        ctx.set_materialize_grads(False)          # the gradient of lse is never used: no zero tensor for it
        return o, lse

    @staticmethod
    def backward(ctx, do, dlse_unused=None):
        q, k, v, qi, ki, o, lse, si, logw, mask = ctx.saved_tensors
        block_size, sample_size, scale, flags, has_si, has_w = ctx.cfg
        if do is None:                            # only lse was used downstream: its gradient is dropped, as in the reference
            return (None,) * 12
        if do.stride(-1) != 1:
            do = do.contiguous()
        B, n, H, d = q.shape
        dv = v.shape[-1]
        dev = q.device
        delta = torch.empty(B, H, n, dtype=torch.float32, device=dev)
        lib = L.load()
        with torch.cuda.device(dev):
            rc = lib.ha_delta(_ptr(o), *_bhn(o), _ptr(do), *_bhn(do), B, H, n, dv, _dtype_id(q), _ptr(delta), _stream())
            L.check(rc, 'ha_delta')
            grads = hyper_bwd(q, k, v, qi, ki, si if has_si else None, o, lse, do, delta, block_size, sample_size, scale, flags,
                              (logw, mask) if has_w else None)
        return grads + (None,) * 9


def _bwd_params(q, k, v, qi, ki, si, o, lse, do, delta, block_size, sample_size, scale, flags, weights):
    B, n, H, d = q.shape
    p = L.AttnParams()
    p.mode, p.dtype, p.flags = L.MODE_HYPER, _dtype_id(q), flags
    p.B, p.H, p.n, p.d, p.dv = B, H, n, d, v.shape[-1]
    p.segs_per_head, p.span, p.q_off, p.k_off, p.m_q, p.m_k = 1, n, 0, 0, n, n
    p.block_size, p.sample_size, p.scale = block_size, sample_size, scale
    _fill_qkv(p, q, k, v)
    p.q_idx, p.k_idx, p.sample_idx = _ptr(qi), _ptr(ki), _ptr(si)
    p.o = _ptr(o)
    p.o_sb, p.o_sh, p.o_sn = _bhn(o)
    p.lse = _ptr(lse)
    p.d_o = _ptr(do)
    p.do_sb, p.do_sh, p.do_sn = _bhn(do)
    p.delta = _ptr(delta)
    _set_status(p, q.device)
    if weights is not None:
        p.sample_logw, p.sample_mask = _ptr(weights[0]), _ptr(weights[1])
    return p


def hyper_bwd(q, k, v, qi, ki, si, o, lse, do, delta, block_size, sample_size, scale, flags, weights=None, direct=None):
    """Backward of the hyper pattern on [B, n, H, *] views: returns (dq, dk, dv) as [B, n, H, *] views in the input dtype.
    On the tensor-core kernel dK/dV are stored directly (ha_attn_params.dk_out) unless direct=False; explicit sampled
    rows that may repeat keep the fp32 accumulators."""
    B, n, H, d = q.shape
    dv = v.shape[-1]
    r = B * H * n
    dev = q.device
    lib = L.load()
    p = _bwd_params(q, k, v, qi, ki, si, o, lse, do, delta, block_size, sample_size, scale, flags, weights)
    if direct is None:
        direct = si is None or weights is not None          # distinct sampled rows
    level = lib.ha_attn_bwd_direct_level(C.byref(p)) if direct else 0
    if level >= 1:
        segs = B * H
        out = torch.empty(r * (2 * d + dv), dtype=q.dtype, device=dev)           # dq | dk | dv
        sacc = torch.zeros(max(1, segs * sample_size * (d + dv)), dtype=torch.float32, device=dev)
        # level 2: dq rows are written directly; level 1: a zeroed fp32 accumulator, cast afterwards
        dq_acc = torch.zeros(r * d, dtype=torch.float32, device=dev) if level == 1 else None
        es = out.element_size()
        p.dq_acc = _ptr(dq_acc)
        p.dk_out, p.dv_out = C.c_void_p(out.data_ptr() + es * r * d), C.c_void_p(out.data_ptr() + es * 2 * r * d)
        p.dk_sacc, p.dv_sacc = C.c_void_p(sacc.data_ptr()), C.c_void_p(sacc.data_ptr() + 4 * segs * sample_size * d)
        if level == 2:
            p.dq_out = _ptr(out)
        L.check(lib.ha_attn_bwd(C.byref(p), _stream()), 'ha_attn_bwd')
        L.check(lib.ha_attn_bwd_finish(C.byref(p), _stream()), 'ha_attn_bwd_finish')
        if level == 1:
            L.check(lib.ha_cast_from_f32(_ptr(dq_acc), _ptr(out), r * d, _DT[q.dtype], _stream()), 'ha_cast_from_f32')
        return (out[:r * d].view(B, H, n, d).transpose(1, 2), out[r * d:2 * r * d].view(B, H, n, d).transpose(1, 2),
                out[2 * r * d:].view(B, H, n, dv).transpose(1, 2))
    acc = torch.zeros(r * (2 * d + dv), dtype=torch.float32, device=dev)
    p.dq_acc = C.c_void_p(acc.data_ptr())
    p.dk_acc, p.dv_acc = C.c_void_p(acc.data_ptr() + 4 * r * d), C.c_void_p(acc.data_ptr() + 8 * r * d)
    L.check(lib.ha_attn_bwd(C.byref(p), _stream()), 'ha_attn_bwd')
    return _cast_grads(lib, acc, q.dtype, B, H, n, d, dv)


def hyper_bwd_launch(q, k, v, qi, ki, si, o, lse, do, delta, acc, block_size, sample_size, scale, flags, weights=None, direct_out=None):
    """One ha_attn_bwd call (HA_MODE_HYPER) on [B, n, H, *] views and nothing else.  acc = zeroed fp32 buffer holding
    dq | dk | dv accumulators ([B,H,n,d], [B,H,n,d], [B,H,n,dv] back to back); with direct_out = (out, sacc) -- `out` in
    the input dtype holding dq | dk | dv, `sacc` the zeroed fp32 slot buffers [B*H*S*(d+dv)] -- only the dq part of acc is
    used, and only where the library cannot write dq directly."""
    B, n, H, d = q.shape
    r = B * H * n
    p = _bwd_params(q, k, v, qi, ki, si, o, lse, do, delta, block_size, sample_size, scale, flags, weights)
    p.dq_acc = C.c_void_p(acc.data_ptr())
    if direct_out is None:
        p.dk_acc, p.dv_acc = C.c_void_p(acc.data_ptr() + 4 * r * d), C.c_void_p(acc.data_ptr() + 8 * r * d)
    else:
        out, sacc = direct_out
        es = out.element_size()
        p.dk_out, p.dv_out = C.c_void_p(out.data_ptr() + es * r * d), C.c_void_p(out.data_ptr() + es * 2 * r * d)
        p.dk_sacc, p.dv_sacc = C.c_void_p(sacc.data_ptr()), C.c_void_p(sacc.data_ptr() + 4 * B * H * sample_size * d)
        if L.load().ha_attn_bwd_direct_level(C.byref(p)) == 2:
            p.dq_out = _ptr(out)
    rc = L.load().ha_attn_bwd(C.byref(p), _stream())
    L.check(rc, 'ha_attn_bwd')


def _cast_grads(lib, acc, dtype, B, H, n, d, dv):
    """fp32 accumulators [B,H,n,*] -> gradients in the input dtype, returned as [B, n, H, *] views."""
    r = B * H * n
    if dtype == torch.float32:
        out = acc
    else:
        out = torch.empty(acc.numel(), dtype=dtype, device=acc.device)
        rc = lib.ha_cast_from_f32(_ptr(acc), _ptr(out), acc.numel(), _DT[dtype], _stream())
        L.check(rc, 'ha_cast_from_f32')
    dq = out[:r * d].view(B, H, n, d).transpose(1, 2)
    dk = out[r * d:2 * r * d].view(B, H, n, d).transpose(1, 2)
    dvv = out[2 * r * d:].view(B, H, n, dv).transpose(1, 2)
    return dq, dk, dvv


def hyper_attn_func(q, k, v, q_sort_idx, k_sort_idx, block_size, sample_size=0, softmax_scale=None, smooth_block=False,
                    sample_idx=None, flags=0, weighted=False):
    return HyperAttnFunc.apply(q, k, v, q_sort_idx, k_sort_idx, block_size, sample_size, softmax_scale, smooth_block,
                               sample_idx, flags, weighted)


class FlashAttnFunc(torch.autograd.Function):
    """Drop-in for FlashAttnFunc (src/flash_attn_triton.py:995-1042) without the bias branch: q [B, n_q, H, d],
    k, v [B, n_k, H, d]; returns o [B, n_q, H, d] and lse [B, H, ceil(n_q/128)*128] (rows past n_q are zero)."""

    @staticmethod
    def forward(ctx, q, k, v, bias=None, causal=False, softmax_scale=None, flags=0):
        assert bias is None, 'attention bias is not part of the HyperAttention path'
        _cuda(q, k, v)
        q, k, v = [x if x.stride(-1) == 1 else x.contiguous() for x in (q, k, v)]
        B, nq, H, d = q.shape
        nk = k.shape[1]
        assert k.shape == (B, nk, H, d)
        assert v.shape[:3] == (B, nk, H)
        assert q.dtype == k.dtype == v.dtype, 'All tensors must have the same type'
        dv = v.shape[-1]
        scale = softmax_scale or 1.0 / math.sqrt(d)
        o = torch.empty(B, H, nq, dv, dtype=q.dtype, device=q.device).transpose(1, 2)
        lse = torch.empty(B, H, nq, dtype=torch.float32, device=q.device)
        p = _flash_params(q, k, v, o, lse, causal, scale, flags)
        with torch.cuda.device(q.device):
            rc = L.load().ha_attn_fwd(C.byref(p), _stream())
        L.check(rc, 'ha_attn_fwd')
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.cfg = (causal, scale, flags)
        nq_r = math.ceil(nq / 128) * 128
        lse_out = lse if nq_r == nq else torch.nn.functional.pad(lse, (0, nq_r - nq))
        return o, lse_out

    @staticmethod
    def backward(ctx, do, dlse_unused=None):
        q, k, v, o, lse = ctx.saved_tensors
        causal, scale, flags = ctx.cfg
        if do.stride(-1) != 1:
            do = do.contiguous()
        B, nq, H, d = q.shape
        nk, dv = k.shape[1], v.shape[-1]
        assert nq == nk, 'backward is implemented for equal query/key lengths'
        dev = q.device
        n = nq
        acc = torch.zeros(B * H * n * (2 * d + dv), dtype=torch.float32, device=dev)
        dq_acc, dk_acc, dv_acc = acc[:B * H * n * d], acc[B * H * n * d:2 * B * H * n * d], acc[2 * B * H * n * d:]
        delta = torch.empty(B, H, n, dtype=torch.float32, device=dev)
        lib = L.load()
        with torch.cuda.device(dev):
            rc = lib.ha_delta(_ptr(o), *_bhn(o), _ptr(do), *_bhn(do), B, H, n, dv, _dtype_id(q), _ptr(delta), _stream())
            L.check(rc, 'ha_delta')
            p = _flash_params(q, k, v, o, lse, causal, scale, flags)
            p.d_o = _ptr(do)
            p.do_sb, p.do_sh, p.do_sn = _bhn(do)
            p.delta, p.dq_acc, p.dk_acc, p.dv_acc = _ptr(delta), _ptr(dq_acc), _ptr(dk_acc), _ptr(dv_acc)
            rc = lib.ha_attn_bwd(C.byref(p), _stream())
            L.check(rc, 'ha_attn_bwd')
            grads = _cast_grads(lib, acc, q.dtype, B, H, n, d, dv)
        return grads + (None,) * 4


def _flash_params(q, k, v, o, lse, causal, scale, flags):
    B, nq, H, d = q.shape
    nk, dv = k.shape[1], v.shape[-1]
    n = nq
    p = L.AttnParams()
    p.mode, p.dtype = L.MODE_FLASH, _dtype_id(q)
    p.flags = (L.FLAG_CAUSAL if causal else 0) | flags
    p.B, p.H, p.n, p.d, p.dv = B, H, n, d, dv
    p.segs_per_head, p.span, p.q_off, p.k_off, p.m_q, p.m_k = 1, n, 0, 0, nq, nk
    p.scale = scale
    _fill_qkv(p, q, k, v)
    p.o = _ptr(o)
    p.o_sb, p.o_sh, p.o_sn = _bhn(o)
    p.lse = _ptr(lse)
    _set_status(p, q.device)
    return p


def flash_attn_func(q, k, v, bias=None, causal=False, softmax_scale=None, flags=0):
    return FlashAttnFunc.apply(q, k, v, bias, causal, softmax_scale, flags)


# ------------------------------------------------------------------------------------------------
class CausalHyperFunc(torch.autograd.Function):
    """The whole causal recursion (hyper_attention.py:51-96) as one call on contiguous [B, H, n, *] tensors.
    grad_reference=True keeps every part's own output so that the backward reproduces the reference's gradient
    convention (each part differentiated with its own rowwise o.do, d(lse) dropped); False gives the gradient of the
    merged output."""

    @staticmethod
    def forward(ctx, q, k, v, proj_f32, levels, block_size, sample_size, scale, flags, grad_reference, min_seq_len=0):
        _cuda(q, k, v, proj_f32)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        B, H, n, d = q.shape
        dv = v.shape[-1]
        dev = q.device
        need_grad = any(t.requires_grad for t in (q, k, v))
        o = torch.empty(B, H, n, dv, dtype=q.dtype, device=dev)
        lse = torch.empty(B, H, n, dtype=torch.float32, device=dev)
        p = L.CausalParams()
        p.dtype, p.flags = _dtype_id(q), flags
        p.B, p.H, p.n, p.d, p.dv = B, H, n, d, dv
        p.levels, p.block_size, p.sample_size, p.lsh_bits = levels, block_size, sample_size, proj_f32.shape[1]
        p.keep_parts = 1 if (grad_reference and need_grad) else 0
        p.min_seq_len = min_seq_len
        p.kv_group = H // k.shape[1]
        p.scale = scale
        p.q, p.k, p.v, p.proj, p.o, p.lse = _ptr(q), _ptr(k), _ptr(v), _ptr(proj_f32), _ptr(o), _ptr(lse)
        _set_status(p, dev)
        lib = L.load()
        saved_bytes = lib.ha_causal_saved_bytes(C.byref(p))
        scratch_bytes = lib.ha_causal_scratch_bytes(C.byref(p), 0)
        assert saved_bytes >= 0 and scratch_bytes >= 0, \
            'causal schedule: n must be divisible by 2^levels with 128-row multiples at every depth'
        saved = torch.empty(saved_bytes, dtype=torch.uint8, device=dev)
        scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=dev)
        p.saved, p.saved_bytes, p.scratch, p.scratch_bytes = _ptr(saved), saved_bytes, _ptr(scratch), scratch_bytes
        with torch.cuda.device(dev):
            rc = lib.ha_causal_fwd(C.byref(p), _stream())
        L.check(rc, 'ha_causal_fwd')
        ctx.save_for_backward(q, k, v, o, lse, saved, proj_f32)
        ctx.cfg = (levels, block_size, sample_size, scale, flags, p.keep_parts, min_seq_len)
        return o, lse

    @staticmethod
    def backward(ctx, do, dlse_unused=None):
        q, k, v, o, lse, saved, proj_f32 = ctx.saved_tensors
        levels, block_size, sample_size, scale, flags, keep_parts, min_seq_len = ctx.cfg
        do = do.contiguous()
        B, H, n, d = q.shape
        dv = v.shape[-1]
        dev = q.device
        dq, dk, dvv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        p = L.CausalParams()
        p.dtype, p.flags = _dtype_id(q), flags
        p.B, p.H, p.n, p.d, p.dv = B, H, n, d, dv
        p.levels, p.block_size, p.sample_size, p.lsh_bits = levels, block_size, sample_size, proj_f32.shape[1]
        p.keep_parts, p.scale, p.min_seq_len = keep_parts, scale, min_seq_len
        p.kv_group = H // k.shape[1]
        p.q, p.k, p.v, p.proj, p.o, p.lse = _ptr(q), _ptr(k), _ptr(v), _ptr(proj_f32), _ptr(o), _ptr(lse)
        p.saved, p.saved_bytes = _ptr(saved), saved.numel()
        _set_status(p, dev)
        lib = L.load()
        scratch_bytes = lib.ha_causal_scratch_bytes(C.byref(p), 1)
        scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=dev)
        p.scratch, p.scratch_bytes = _ptr(scratch), scratch_bytes
        p.d_o, p.dq, p.dk, p.dv_out = _ptr(do), _ptr(dq), _ptr(dk), _ptr(dvv)
        with torch.cuda.device(dev):
            rc = lib.ha_causal_bwd(C.byref(p), _stream())
        L.check(rc, 'ha_causal_bwd')
        return dq, dk, dvv, None, None, None, None, None, None, None, None


class NonCausalHyperFunc(torch.autograd.Function):
    """forward_no_causal_mask on sequences of at least min_seq_len (hyper_attention.py:116-130: hash, stable sort,
    hyper_attn_func) as ONE library call each way (ha_noncausal_fwd / ha_noncausal_bwd) on contiguous [B, H, n, *] tensors:
    two calls into the library per training step instead of nine, which is what bounds the step when a rank owns few
    heads.  Returns o [B, H, n, dv] and lse [B, H, n]; the gradient flowing into lse is discarded, as in the reference."""

    @staticmethod
    def _params(q, k, v, proj_f32, block_size, sample_size, scale, flags):
        B, H, n, d = q.shape
        p = L.CausalParams()
        p.dtype, p.flags = _dtype_id(q), flags
        p.B, p.H, p.n, p.d, p.dv = B, H, n, d, v.shape[-1]
        p.block_size, p.sample_size, p.lsh_bits, p.scale = block_size, sample_size, proj_f32.shape[1], scale
        p.kv_group = H // k.shape[1]
        p.q, p.k, p.v, p.proj = _ptr(q), _ptr(k), _ptr(v), _ptr(proj_f32)
        _set_status(p, q.device)
        return p

    @staticmethod
    def forward(ctx, q, k, v, proj_f32, block_size, sample_size, scale, flags):
        _cuda(q, k, v, proj_f32)
        assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
        assert q.dtype == k.dtype == v.dtype, 'All tensors must have the same type'
        B, H, n, d = q.shape
        assert k.shape[0] == B and k.shape[2:] == (n, d), 'query and key sequence lengths must be equal'
        assert H % k.shape[1] == 0 and v.shape[:3] == k.shape[:3], 'query heads must be a multiple of the key/value heads'
        assert n % 128 == 0, 'keys sequence length must be divisible by 128'
        assert sample_size % 128 == 0
        dev = q.device
        o = torch.empty(B, H, n, v.shape[-1], dtype=q.dtype, device=dev)
        lse = torch.empty(B, H, n, dtype=torch.float32, device=dev)
        p = NonCausalHyperFunc._params(q, k, v, proj_f32, block_size, sample_size, scale, flags)
        p.o, p.lse = _ptr(o), _ptr(lse)
        lib = L.load()
        saved_bytes, scratch_bytes = lib.ha_noncausal_saved_bytes(C.byref(p)), lib.ha_noncausal_scratch_bytes(C.byref(p), 0)
        assert saved_bytes >= 0 and scratch_bytes >= 0, 'shape not accepted (n and sample_size multiples of 128, sample_size <= n)'
        saved = torch.empty(saved_bytes, dtype=torch.uint8, device=dev)
        scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=dev)
        p.saved, p.saved_bytes, p.scratch, p.scratch_bytes = _ptr(saved), saved_bytes, _ptr(scratch), scratch_bytes
        with torch.cuda.device(dev):
            rc = lib.ha_noncausal_fwd(C.byref(p), _stream())
        L.check(rc, 'ha_noncausal_fwd')
        ctx.save_for_backward(q, k, v, o, lse, saved, proj_f32)
        ctx.cfg = (block_size, sample_size, scale, flags)
        ctx.set_materialize_grads(False)
        return o, lse

    @staticmethod
    def backward(ctx, do, dlse_unused=None):
        q, k, v, o, lse, saved, proj_f32 = ctx.saved_tensors
        block_size, sample_size, scale, flags = ctx.cfg
        if do is None:
            return (None,) * 8
        do = do.contiguous()
        dev = q.device
        # one buffer for the three gradients (dq | dk | dv): one allocation per step
        nq, nk, nv = q.numel(), k.numel(), v.numel()
        out = torch.empty(nq + nk + nv, dtype=q.dtype, device=dev)
        dq, dk, dvv = out[:nq].view_as(q), out[nq:nq + nk].view_as(k), out[nq + nk:].view_as(v)
        p = NonCausalHyperFunc._params(q, k, v, proj_f32, block_size, sample_size, scale, flags)
        p.o, p.lse = _ptr(o), _ptr(lse)
        p.saved, p.saved_bytes = _ptr(saved), saved.numel()
        p.d_o, p.dq, p.dk, p.dv_out = _ptr(do), _ptr(dq), _ptr(dk), _ptr(dvv)
        lib = L.load()
        scratch_bytes = lib.ha_noncausal_scratch_bytes(C.byref(p), 1)
        scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=dev)
        p.scratch, p.scratch_bytes = _ptr(scratch), scratch_bytes
        with torch.cuda.device(dev):
            rc = lib.ha_noncausal_bwd(C.byref(p), _stream())
        L.check(rc, 'ha_noncausal_bwd')
        return dq, dk, dvv, None, None, None, None, None


def launch_count():
    return int(L.load().ha_launch_count())
