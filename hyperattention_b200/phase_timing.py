"""Per-role cycle counters of the warp-specialised backward (and, with --forward, forward) kernel (a developer diagnostic, not
part of the product path).

    python hyperattention_b200/csrc/build.py --timing          # builds libhyperattn_b200_timing.so (-DHA_PHASE_TIMING)
    python -m hyperattention_b200.phase_timing [--heads 32] [--seq-len 131072]

Runs one non-causal forward + backward of the headline shape with the instrumented library and prints, per role of
attn_tc_bwd_ws_kernel (thread 0 of each role, averaged over the CTAs), how its cycles divide between waiting on each
barrier and working.  The counters use clock64 between the phases of every loop iteration; they perturb the kernel a
little, so the absolute kernel time is taken from bench.py, not from here.
"""
import argparse
import ctypes as C
import os

import torch

from . import _lib

ROLES = {0: ('elementwise group 0', ['wait S^T/dP^T ready', 'wait lse/delta (+ scaling)', 'wait dS buffer free', 'loads + math + stores',
                                       'store-wait, fences, arrivals']),
         1: ('elementwise group 1', ['wait S^T/dP^T ready', 'wait lse/delta (+ scaling)', 'wait dS buffer free', 'loads + math + stores',
                                       'store-wait, fences, arrivals']),
         2: ('drain group', ['wait accumulators full', 'index loads, staging writes, coalesced stores / reductions', 'wait dQ full', 'dQ rows',
                             'accumulator -> registers (issuers blocked)', 'wait staging tile free (whole-tile additions)', 'proxy fence',
                             'whole-tile additions: barrier, issue (thread 0 of the group: + the read of the tile)']),
         3: ('K loader warp', ['index loads, L2 prefetch', 'wait stage empty', 'issuing the copies of a tile']),
         4: ('S^T issuer', ['loop', 'wait stage columns free (dV of the previous pair)', 'wait K / Q tiles', 'fences, 4 MMAs, commits']),
         5: ('dV issuer', ['loop', 'wait P^T ready', 'wait accumulator drained', 'fences, 4 MMAs, commits']),
         6: ('dQ issuer', ['loop', 'wait dS slabs full', 'wait dQ drained', 'fences, 8 MMAs, commits']),
         7: ('Q / dO loader warp', ['index loads, L2 prefetch', 'wait stage empty', 'issuing the copies of two tiles'])}

# attn_tc_fwd_ws_kernel, softmax group 0: (counter slot, phase)
FWD_PHASES = [(0, 'item set-up, loop (row index, accumulator clear)'), (1, 'wait S ready'),
              (3, 'max pass, previous product (wait + fold), exp pass, P store'), (4, "the item's last product: wait + fold"),
              (6, 'epilogue: normalise, pack, row stores'), (5, 'lse store')]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--heads', type=int, default=32)
    ap.add_argument('--seq-len', type=int, default=131072)
    ap.add_argument('--forward', action='store_true', help='the forward kernel (attn_tc_fwd_ws_kernel) instead of the backward')
    a = ap.parse_args()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'libhyperattn_b200_timing.so')
    assert os.path.exists(path), 'build the instrumented library first: python hyperattention_b200/csrc/build.py --timing'
    _lib.LIB_PATH = path
    lib = _lib.load()
    from .module import HyperAttention
    torch.manual_seed(0)
    q, k, v, do = [torch.randn(1, a.heads, a.seq_len, 64, device='cuda', dtype=torch.bfloat16) for _ in range(4)]
    mod = HyperAttention(input_dim=64).to(device='cuda', dtype=torch.bfloat16)
    buf = torch.zeros(4096 * 16, dtype=torch.int64, device='cuda')
    n_cta = min(148, a.heads * a.seq_len // 256)
    if a.forward:
        with torch.no_grad():
            mod(q, k, v)
            torch.cuda.synchronize()
            setter = lib.ha_debug_set_timing_buffer_fwd_ws
            setter.restype, setter.argtypes = C.c_int, [C.c_void_p]
            setter(C.c_void_p(buf.data_ptr()))
            mod(q, k, v)
            torch.cuda.synchronize()
        b = buf.view(4096, 16).cpu().float()[:n_cta, :8]
        tot = b.sum(1).mean().item()
        print(f'softmax group 0 (thread 0): {round(tot)} cycles per CTA, {round(tot / max(1, a.heads * a.seq_len // 256 / n_cta))} per work item')
        for i, ph in FWD_PHASES:
            print(f'   {ph:58s} {b[:, i].mean().item():11.0f} {100 * b[:, i].mean().item() / max(tot, 1):5.1f}%')
        return
    qg, kg, vg = [t.clone().requires_grad_() for t in (q, k, v)]
    for rep in range(2):
        o = mod(qg, kg, vg)
        if rep == 1:
            setter = lib.ha_debug_set_timing_buffer_bwd_ws
            setter.restype, setter.argtypes = C.c_int, [C.c_void_p]
            setter(C.c_void_p(buf.data_ptr()))
        o.backward(do)
        torch.cuda.synchronize()
    b = buf.view(4096, 16).cpu().float()[:n_cta * 8].view(n_cta, 8, 16)
    for r, (name, phases) in ROLES.items():
        bb = b[:, r]
        tot = bb[:, :8].sum(1).mean().item()
        print(f'{name}: {round(tot)} cycles per CTA')
        for i, ph in enumerate(phases):
            print(f'   {ph:46s} {bb[:, i].mean().item():11.0f} {100 * bb[:, i].mean().item() / max(tot, 1):5.1f}%')


if __name__ == '__main__':
    main()
