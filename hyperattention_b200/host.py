"""HyperAttention.forward (and its backward) for tensors that live in HOST memory.

Heads are independent on this path (one LSH projection shared by all of them, everything else per head), so a
step over host-resident q, k, v is streamed through the GPU in chunks of heads on three CUDA streams:

    copy-in stream :  H2D chunk c+1   |  H2D chunk c+2  | ...
    compute stream :  kernels chunk c |  kernels c+1    | ...
    copy-out stream:  D2H chunk c-1   |  D2H chunk c    | ...

PCIe is full duplex, so the step costs about max(bytes in, bytes out) / link bandwidth plus one chunk of latency,
instead of the sum of copy-in, compute and copy-out.  The arithmetic is the module's own (hyper_attention.py:23-132
in the reference, which has no host-buffer entry point of its own); results per head do not depend on the chunking.

Host tensors should be pinned (torch.Tensor.pin_memory); pageable memory works but the copies then block the host.
"""
from __future__ import annotations

import torch

from . import ops


class HostStream:
    """Streams [B, H, n, d] host tensors through `module` (a HyperAttention on a CUDA device) in chunks of heads.

    heads_per_chunk: heads per chunk (default: at least four chunks per call, so that copy-in, kernels and copy-out
    overlap, and at most about 160 MB of inputs per chunk: the first copy-in and the last copy-out overlap with nothing, so
    chunks are kept small -- measured at 32 heads x 131072 x 64 bf16 over PCIe 5: 8 heads per chunk 56 ms, 4 49 ms, 2 48 ms,
    1 62 ms per forward + backward); the first and the last chunk are half that size.
    Two chunks of inputs are resident at a time; outputs are written into pinned host buffers that are kept and
    reused between calls (pass out=... to supply your own)."""

    def __init__(self, module, heads_per_chunk=None, device=None):
        self.module = module
        p = next(iter(module.buffers()), None)
        self.device = torch.device(device) if device is not None else (p.device if p is not None else torch.device('cuda'))
        assert self.device.type == 'cuda', 'the module must live on a CUDA device (there is no CPU implementation)'
        self.heads_per_chunk = heads_per_chunk
        self._streams = None
        self._out = {}

    # ---------------------------------------------------------------------------------------------------------
    def _setup(self):
        if self._streams is None:
            with torch.cuda.device(self.device):
                self._streams = (torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream())
        return self._streams

    def _chunking(self, q, n_inputs):
        B, H, n, d = q.shape
        hpc = self.heads_per_chunk
        if hpc is None:
            per_head = max(1, B * n * d * q.element_size() * n_inputs)
            hpc = max(1, min(max(1, H // 4), (160 << 20) // per_head))
            # the first chunk's copy-in and the last chunk's copy-out are the two transfers nothing overlaps: half-size chunks
            # at both ends
            edge = max(1, hpc // 2)
            if edge < hpc and H >= 2 * edge + hpc:
                cuts = [0, edge] + list(range(edge + hpc, H - edge, hpc)) + [H - edge, H]
                cuts = sorted(set(cuts))
                return [(a, b) for a, b in zip(cuts[:-1], cuts[1:])]
        return [(h0, min(H, h0 + hpc)) for h0 in range(0, H, hpc)]

    def _host_out(self, key, like, shape):
        t = self._out.get(key)
        if t is None or t.shape != shape or t.dtype != like.dtype:
            t = torch.empty(shape, dtype=like.dtype, pin_memory=True)
            self._out[key] = t
        return t

    def _run(self, host_in, causal, backward, out):
        q = host_in[0]
        assert all(t.device.type == 'cpu' for t in host_in), 'HostStream takes host tensors'
        assert all(t.dim() == 4 and t.shape[:3] == q.shape[:3] for t in host_in)
        B, H, n, d = q.shape
        dv = host_in[2].shape[-1]
        names = ('o', 'dq', 'dk', 'dv') if backward else ('o',)
        shapes = {'o': (B, H, n, dv), 'dq': (B, H, n, d), 'dk': (B, H, n, d), 'dv': (B, H, n, dv)}
        if out is None:
            out = tuple(self._host_out(nm, q, shapes[nm]) for nm in names)
        assert len(out) == len(names) and all(o.shape == shapes[nm] for o, nm in zip(out, names))
        s_in, s_comp, s_out = self._setup()
        chunks = self._chunking(q, len(host_in))
        caller = torch.cuda.current_stream(self.device)
        for s in (s_in, s_comp, s_out):
            s.wait_stream(caller)
        staged = {}          # chunk index -> (device inputs, event "copy-in done")
        computed = []        # events "compute of chunk c done": gate the reuse of an input slot two chunks later

        def copy_in(c):
            h0, h1 = chunks[c]
            with torch.cuda.stream(s_in):
                if c >= 2:
                    s_in.wait_event(computed[c - 2])     # at most two chunks of inputs are resident
                # one copy per batch index: t[b, h0:h1] is contiguous, t[:, h0:h1] is not when B > 1 (a strided host
                # slice would go through a pageable temporary and block)
                dev_in = [torch.empty((B, h1 - h0) + tuple(t.shape[2:]), dtype=t.dtype, device=self.device) for t in host_in]
                for dst, t in zip(dev_in, host_in):
                    for b in range(B):
                        dst[b].copy_(t[b, h0:h1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_in)
            staged[c] = (dev_in, ev)

        with torch.cuda.device(self.device):
            copy_in(0)
            for c, (h0, h1) in enumerate(chunks):
                if c + 1 < len(chunks):
                    copy_in(c + 1)
                dev_in, ev_in = staged.pop(c)
                with torch.cuda.stream(s_comp):
                    s_comp.wait_event(ev_in)
                    for t in dev_in:
                        t.record_stream(s_comp)
                    if backward:
                        qd, kd, vd = [t.requires_grad_() for t in dev_in[:3]]
                        o = self.module(qd, kd, vd, causal=causal)
                        res = (o.detach(),) + torch.autograd.grad(o, (qd, kd, vd), dev_in[3])
                    else:
                        with torch.no_grad():
                            res = (self.module(*dev_in[:3], causal=causal),)
                    ev_c = torch.cuda.Event()
                    ev_c.record(s_comp)
                computed.append(ev_c)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_c)
                    for dst, src in zip(out, res):
                        src.record_stream(s_out)
                        for b in range(B):
                            dst[b, h0:h1].copy_(src[b], non_blocking=True)
                del dev_in, res
            for s in (s_in, s_comp, s_out):
                caller.wait_stream(s)
        return out

    # ---------------------------------------------------------------------------------------------------------
    def forward(self, q, k, v, causal=False, out=None):
        """q, k, v host tensors [B, H, n, d]; returns the pinned host tensor o [B, H, n, dv].  The result is complete
        once the caller's current CUDA stream has been synchronised (torch.cuda.current_stream().synchronize())."""
        return self._run((q, k, v), causal, False, None if out is None else (out,))[0]

    def forward_backward(self, q, k, v, do, causal=False, out=None):
        """Forward and backward for host tensors: returns pinned host tensors (o, dq, dk, dv), complete once the caller's
        current CUDA stream has been synchronised."""
        return self._run((q, k, v, do), causal, True, out)


def check_after(device=None):
    """Convenience: synchronise and raise if a kernel of the step reported a device-side timeout."""
    torch.cuda.synchronize(device)
    ops.check_device_status(device)
