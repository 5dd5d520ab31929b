"""Sequence-length sweep (benchmark configuration 3): batch 1, 32 heads, head_dim 64, bf16, i.i.d. N(0,1) inputs, causal and
non-causal, smooth_block off/on; each point is timed (CUDA events, median of `reps`) forward and forward+backward and
compared with exact attention of the same shape (torch scaled_dot_product_attention).  One JSON line per point.

    python -m hyperattention_b200.sweep [--max-len 524288] [--heads 32] [--reps 5] [--no-exact]
"""
import argparse
import json

import torch
import torch.nn.functional as F

from .module import HyperAttention


def _time(fn, reps):
    fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--min-len', type=int, default=4096)
    ap.add_argument('--max-len', type=int, default=524288)
    ap.add_argument('--heads', type=int, default=32)
    ap.add_argument('--reps', type=int, default=5)
    ap.add_argument('--no-exact', action='store_true')
    a = ap.parse_args()
    dev = torch.device('cuda')
    n = a.min_len
    while n <= a.max_len:
        g = torch.Generator(device=dev).manual_seed(3)
        q, k, v, do = [torch.randn(1, a.heads, n, 64, device=dev, dtype=torch.bfloat16, generator=g) for _ in range(4)]
        q, k, v = [t.requires_grad_() for t in (q, k, v)]
        exact = {}
        for causal in (False, True):
            if not a.no_exact:
                def ef():
                    with torch.no_grad():
                        return F.scaled_dot_product_attention(q, k, v, is_causal=causal)
                def efb():
                    o = F.scaled_dot_product_attention(q, k, v, is_causal=causal)
                    torch.autograd.grad(o, (q, k, v), do)
                reps = max(1, min(a.reps, 3 if n >= 262144 else a.reps))
                exact[causal] = (_time(ef, reps), _time(efb, reps))
            for smooth in (False, True):
                mod = HyperAttention(input_dim=64, block_size=256, sample_size=256, min_seq_len=2048, smooth_block=smooth,
                                     rng=torch.Generator().manual_seed(1234)).to(device=dev, dtype=torch.bfloat16)
                def hf():
                    with torch.no_grad():
                        return mod(q, k, v, causal=causal)
                def hfb():
                    o = mod(q, k, v, causal=causal)
                    torch.autograd.grad(o, (q, k, v), do)
                tf, tfb = _time(hf, a.reps), _time(hfb, a.reps)
                rec = {'seq_len': n, 'heads': a.heads, 'causal': causal, 'smooth_block': smooth, 'hyper_fwd_ms': tf, 'hyper_fwd_bwd_ms': tfb,
                       'tokens_per_s_fwd_bwd': n / tfb * 1e3}
                if causal in exact:
                    rec.update({'exact_fwd_ms': exact[causal][0], 'exact_fwd_bwd_ms': exact[causal][1],
                                'speedup_fwd': exact[causal][0] / tf, 'speedup_fwd_bwd': exact[causal][1] / tfb})
                print(json.dumps(rec), flush=True)
        del q, k, v, do
        torch.cuda.empty_cache()
        n *= 2


if __name__ == '__main__':
    main()
