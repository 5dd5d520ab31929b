"""Benchmark of the HyperAttention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2] [--impl reference] [--seq-len n] [--heads H]

A step is one forward+backward pass of the HyperAttention module over one synthetic batch of the headline shape
(batch 1, 32 heads, head_dim 64, 131072 tokens, bf16; benchmark configuration 1 = non-causal, config 2 = causal).  The
heads are partitioned over the GPUs (no collective on the data path); the time of a step is the maximum over ranks,
measured with CUDA events.  One JSON line is printed by rank 0.

--impl reference times the CPU restatement of the reference (the oracle) on the host cores on a bounded sample of
the same workload (a subset of heads), as the reference's own attention kernels cannot run on a CPU.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch

HEADS, DIM, SEQ = 32, 64, 131072
BLOCK, SAMPLE, MIN_SEQ, BITS = 256, 256, 2048, 8


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='b200', choices=['b200', 'reference'])
    ap.add_argument('--workload', default='c1', choices=['c1', 'c2'])
    ap.add_argument('--seq-len', type=int, default=SEQ)
    ap.add_argument('--heads', type=int, default=HEADS)
    ap.add_argument('--no-extras', action='store_true', help='skip the exact-flash comparator, cpu baseline and per-kernel roofline legs')
    ap.add_argument('--cpu-heads', type=int, default=1, help='heads in the CPU-baseline sample')
    return ap.parse_args()


def clustered_inputs(heads, n, d, seed, device='cpu', dtype=torch.bfloat16, first_head=0):
    """Benchmark configurations 1/2: per head 64 unit-norm centroids shared by Q and K, per-token Gaussian noise of total
    norm ~0.3, V ~ N(0,1), dO ~ N(0,1).  Every head has its own generator (seed, head index), so a rank that owns heads
    [first_head, first_head + heads) produces exactly the slice a single process would."""
    outs = [[], [], [], []]
    for h in range(first_head, first_head + heads):
        g = torch.Generator().manual_seed(seed * 100003 + h)
        cent = torch.randn(64, d, generator=g)
        cent = cent / cent.norm(dim=-1, keepdim=True)
        def draw():
            a = torch.randint(0, 64, (n,), generator=g)
            return cent[a] + torch.randn(n, d, generator=g) * (0.3 / math.sqrt(d))
        outs[0].append(draw().to(dtype))
        outs[1].append(draw().to(dtype))
        outs[2].append(torch.randn(n, d, generator=g).to(dtype))
        outs[3].append(torch.randn(n, d, generator=g).to(dtype))
    return [torch.stack(o).unsqueeze(0).to(device) for o in outs]


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = 'index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,' \
        'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap'

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.idx), f'--query-gpu={self.Q}', '--format=csv,noheader,nounits',
                                          '-lms', '200'], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(',')]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), f[4:8]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        sm.sort()
        return {'sm_mhz': sm[len(sm) // 2] if sm else None, 'sm_max_mhz': mx, 'reasons': sorted(reasons), 'samples': len(sm)}


def timed(fn, steps, warmup, sync_all, stats=None):
    """warmup untimed calls, then `steps` calls between CUDA events on the current stream; returns ms per step (total
    time of the K steps / K).  With stats (a dict): an event after every step as well, from which the median and the 0.2 /
    0.8 quantiles of the per-step times are taken (the reference's protocol, benchmark_single_attention.py:40-52); if fn
    returns a CUDA event recorded inside the step (end of its forward), the forward and backward shares too."""
    for _ in range(warmup):
        fn()
    sync_all()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    mids = []
    ev[0].record()
    for i in range(steps):
        m = fn()
        if stats is not None and isinstance(m, torch.cuda.Event):
            mids.append(m)
        ev[i + 1].record()
    ev[-1].synchronize()
    sync_all()
    if stats is not None:
        per = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(steps))
        q = lambda f: per[min(steps - 1, int(f * steps))]
        stats.update({'median_ms': q(0.5), 'q20_ms': q(0.2), 'q80_ms': q(0.8), 'reps': steps})
        if len(mids) == steps:
            f = sorted(ev[i].elapsed_time(mids[i]) for i in range(steps))
            b = sorted(mids[i].elapsed_time(ev[i + 1]) for i in range(steps))
            stats.update({'fwd_median_ms': f[steps // 2], 'bwd_median_ms': b[steps // 2]})
    return ev[0].elapsed_time(ev[-1]) / steps


def cpu_baseline(workload, n, d, heads_sample, total_heads, seed, target_seconds=12.0):
    """The reference's host-side path restated on the CPU (oracle): its glue, hash, stable sort and merge, with the two
    device-only attention callables replaced by the oracle's PyTorch Functions.  Timed on a sample of heads (one head
    first; if that is quick, as many heads as fit in about `target_seconds`) and scaled linearly to `total_heads`."""
    from oracle import hyper_oracle as O
    # every host core: torchrun exports OMP_NUM_THREADS=1 to its ranks, which would make this a one-thread baseline
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(1234)
    proj = torch.randn(1, 1, d, BITS, generator=g)

    def run(hs):
        q, k, v, do = clustered_inputs(hs, n, d, seed, dtype=torch.float32)
        orc = O.HyperAttentionOracle(proj, BLOCK, SAMPLE, MIN_SEQ, False)
        q, k, v = [t.requires_grad_() for t in (q, k, v)]
        t0 = time.perf_counter()
        o = orc(q, k, v, causal=(workload == 'c2'))
        t1 = time.perf_counter()
        o.backward(do)
        t2 = time.perf_counter()
        return t1 - t0, t2 - t1

    hs = max(1, heads_sample)
    f, b = run(hs)
    if heads_sample <= 1 and (f + b) < target_seconds / 2:
        hs = int(max(1, min(total_heads, target_seconds // max(f + b, 1e-3))))
        if hs > 1:
            f, b = run(hs)
    scale = total_heads / hs
    sec = (f + b) * scale
    return {'value': n / sec, 'unit': 'tokens/s', 'cores': torch.get_num_threads(), 'kind': 'port',
            'sample': f'{hs} of {total_heads} heads at n={n}, fp32, fwd {f:.2f}s + bwd {b:.2f}s, scaled x{scale:g} '
                      f'(reference glue/hash/sort/merge restated in PyTorch; attention kernels restated because the '
                      f'reference has none for CPU)',
            'host_cpus': os.cpu_count(), 'fwd_s_scaled': f * scale, 'fwd_bwd_s_scaled': sec, 'heads_sampled': hs}


def main():
    args = parse()
    rank = int(os.environ.get('RANK', 0))
    world = int(os.environ.get('WORLD_SIZE', 1))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))
    n, d, heads = args.seq_len, DIM, args.heads
    causal = args.workload == 'c2'
    seed = 1 if args.workload == 'c1' else 2
    config = {'workload': f"benchmark configuration {'2 (causal)' if causal else '1 (non-causal)'}: batch 1, {heads} heads, head_dim {d}, "
                          f"seq_len {n}, bf16, block 256, sample 256, lsh 8 bits" + (', min_seq_len 2048' if causal else ''),
              'step': 'forward + backward of HyperAttention.forward', 'heads_per_gpu': heads // max(world, 1),
              'partition': 'heads over GPUs, no collective', 'l2': 'inputs (4 x 537 MB per step at 1 GPU) exceed the 126 MB L2',
              'grad_mode': 'reference'}

    if args.impl == 'reference':
        if rank != 0:
            return
        # every step is a bounded sample of the workload (whole heads at full length), sized so that the K steps together
        # stay within about three minutes of host time
        per_step = min(12.0, max(2.0, 150.0 / max(1, args.steps)))
        cb = cpu_baseline(args.workload, n, d, args.cpu_heads, heads, seed, target_seconds=per_step)
        vals = [cb['value']]
        for _ in range(max(0, args.steps - 1)):
            vals.append(cpu_baseline(args.workload, n, d, cb['heads_sampled'], heads, seed)['value'])
        val = sum(vals) / len(vals)
        cb['value'] = val
        line = {'impl': 'reference', 'metric': 'hyperattention_fwd_bwd_tokens_per_s', 'value': val, 'unit': 'tokens/s', 'n_gpus': args.gpus,
                'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': 1e3 * n / val, 'higher_is_better': True, 'scaling': 'strong',
                'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic', 'config': config, 'cpu_baseline': cb,
                'e2e': {'value': val, 'unit': 'tokens/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}}
        print(json.dumps(line))
        return

    assert torch.cuda.is_available(), 'bench.py needs a CUDA device'
    import hyperattention_b200 as ha
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group('nccl', device_id=dev)
    assert heads % world == 0
    hpg = heads // world

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    # same data on every world size: every head has its own seed, a rank generates only the heads it owns
    from hyperattention_b200.partition import head_slice
    mine = head_slice(heads, rank, world)
    assert mine.stop - mine.start == hpg
    host = [t.contiguous().pin_memory() for t in clustered_inputs(hpg, n, d, seed, first_head=mine.start)]
    q, k, v, do = [t.to(dev) for t in host]
    q, k, v = [t.requires_grad_() for t in (q, k, v)]
    gen = torch.Generator().manual_seed(1234)
    mod = ha.HyperAttention(input_dim=d, lsh_num_projs=BITS, block_size=BLOCK, sample_size=SAMPLE, min_seq_len=MIN_SEQ,
                            rng=gen).to(device=dev, dtype=torch.bfloat16)

    def fwd():
        with torch.no_grad():
            return mod(q, k, v, causal=causal)

    def fwd_bwd():
        o = mod(q, k, v, causal=causal)
        mid = torch.cuda.Event(enable_timing=True)
        mid.record()
        torch.autograd.grad(o, (q, k, v), do)
        return mid

    sampler = ClockSampler(torch.cuda.current_device() if 'CUDA_VISIBLE_DEVICES' not in os.environ else local_rank)
    launches0 = ha.launch_count()
    fwd_bwd()   # first call: allocator growth
    sync_all()
    sampler.start()
    l0 = ha.launch_count()
    step_stats = {}
    ms = timed(fwd_bwd, args.steps, args.warmup, sync_all, step_stats)
    launches = (ha.launch_count() - l0) // (args.steps + args.warmup) * args.steps
    ms_fwd = timed(fwd, args.steps, args.warmup, sync_all)
    # host time to enqueue one step without waiting for the device (what bounds the step when a rank owns few heads)
    sync_all()
    t0 = time.perf_counter()
    for _ in range(5):
        fwd_bwd()
    host_enqueue_ms = (time.perf_counter() - t0) / 5 * 1e3
    sync_all()
    # the causal configuration (benchmark configuration 2) on the same tensors and the same ranks: times do not depend on the values
    def c_fwd():
        with torch.no_grad():
            return mod(q, k, v, causal=True)
    def c_fwd_bwd():
        oo = mod(q, k, v, causal=True)
        mid = torch.cuda.Event(enable_timing=True)
        mid.record()
        torch.autograd.grad(oo, (q, k, v), do)
        return mid
    c_stats = {}
    c_steps = max(3, args.steps // 2)
    c_fwd_bwd()
    tc_fb = timed(c_fwd_bwd, c_steps, 2, sync_all, c_stats)
    tc_f = timed(c_fwd, c_steps, 2, sync_all)
    if dist is not None:
        t = torch.tensor([ms, ms_fwd, tc_fb, tc_f, host_enqueue_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_fwd, tc_fb, tc_f, host_enqueue_ms = t.tolist()
    causal2 = {'fwd_ms': tc_f, 'fwd_bwd_ms': tc_fb, 'fwd_bwd_tokens_per_s': n / (tc_fb * 1e-3), 'steps': c_steps, 'timing': 'max over ranks', **c_stats}

    # end to end through the public host-buffer API: pinned H2D of q, k, v, do and D2H of o and the three gradients every
    # step, streamed over chunks of heads (copy-in, kernels and copy-out overlap; PCIe is full duplex)
    from hyperattention_b200.host import HostStream
    outs = tuple(torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in host)
    hs = HostStream(mod)
    def e2e_step():
        hs.forward_backward(*host, causal=causal, out=outs)
    ms_e2e = timed(e2e_step, args.steps, args.warmup, sync_all)
    if dist is not None:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = t.item()
    ha.check_device_status(dev)
    clocks = sampler.stop()
    bytes_io = sum(t.numel() * t.element_size() for t in host)

    line = {'metric': 'hyperattention_fwd_bwd_tokens_per_s', 'value': n / (ms * 1e-3), 'unit': 'tokens/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': ms, 'higher_is_better': True, 'scaling': 'strong',
            'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic', 'config': config, 'fwd_ms': ms_fwd, 'fwd_tokens_per_s': n / (ms_fwd * 1e-3),
            'clocks': clocks, 'gpu_launches': int(launches), 'step_stats': step_stats, 'host_enqueue_ms': host_enqueue_ms,
            'causal_config2': causal2,
            'e2e': {'value': n / (ms_e2e * 1e-3), 'unit': 'tokens/s', 'ms_per_step': ms_e2e, 'h2d_bytes_per_step': bytes_io,
                    'd2h_bytes_per_step': bytes_io, 'api': 'hyperattention_b200.host.HostStream.forward_backward',
                    'pcie_gbs_each_way': bytes_io / (ms_e2e * 1e-3) / 1e9}}

    if rank == 0 and not args.no_extras:
        line.update(extras(args, ha, mod, q, k, v, do, causal, n, d, hpg, heads, seed, dev, tc_f, tc_fb))
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def kernel_traffic(kernel, rows):
    """Measured DRAM traffic of one launch of `kernel` over `rows` rows (dram__bytes_read.sum + dram__bytes_write.sum of an
    ncu capture on a smaller case, which scales with the rows: fixed work per row), from the tracked table of captures;
    None when no capture of this kernel is on record."""
    path = os.path.join(ROOT, 'profiles', 'kernel_dram_traffic.json')
    try:
        entry = json.load(open(path))[kernel]
        return entry['dram_bytes'] / entry['rows'] * rows
    except (OSError, KeyError, ValueError):
        return None


def extras(args, ha, mod, q, k, v, do, causal, n, d, hpg, heads, seed, dev, tc_f, tc_fb):
    """Kernel-alone timings and rooflines (CUDA events on the launching stream), the exact-flash comparator, the causal
    configuration's times, the CPU baseline."""
    from hyperattention_b200 import ops
    peaks = {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'src': 'fallback'}
    pk = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(pk):
        m = json.load(open(pk))
        peaks = {'hbm_gbs': m['hbm_gbs'], 'bf16_tflops': m['bf16_tflops'], 'src': 'measured'}
    sync = torch.cuda.synchronize
    out = {}
    rows = hpg * n
    T = lambda t: t.transpose(1, 2)
    with torch.no_grad():
        qd, kd, vd = q.detach(), k.detach(), v.detach()
        proj = mod.lsh.proj_f32()
        t_hash = timed(lambda: ops.lsh_hash(qd, proj), 10, 3, sync)
        codes = ops.lsh_hash(qd, proj)
        t_sort = timed(lambda: ops.seg_sort(codes, BITS), 10, 3, sync)
        qi = ops.seg_sort(codes, BITS).view(1, hpg, n)
        ki = ops.seg_sort(ops.lsh_hash(kd, proj), BITS).view(1, hpg, n)
        t_gather = timed(lambda: ops.indexing(qd, qi), 10, 3, sync)
        t_fwd = timed(lambda: ops.hyper_attn_func(T(qd), T(kd), T(vd), T(qi), T(ki), BLOCK, SAMPLE), 10, 3, sync)
        o, lse = ops.hyper_attn_func(T(qd), T(kd), T(vd), T(qi), T(ki), BLOCK, SAMPLE)
        # the backward kernel alone: delta and the zeroed accumulators are prepared outside the timed launches
        qi32, ki32 = qi.view(hpg, n).contiguous(), ki.view(hpg, n).contiguous()
        delta = (o.float() * T(do).float()).sum(-1).transpose(1, 2).contiguous()
        # (as in the step: dq into the zeroed fp32 accumulator, dk/dv stored directly, sampled rows into the slot buffers)
        acc = torch.zeros(rows * d, dtype=torch.float32, device=dev)
        out_kv = torch.empty(rows * 3 * d, dtype=q.dtype, device=dev)
        sacc = torch.zeros(hpg * SAMPLE * 2 * d, dtype=torch.float32, device=dev)
        bwd = lambda: ops.hyper_bwd_launch(T(qd), T(kd), T(vd), qi32, ki32, None, o, lse, T(do), delta, acc, BLOCK, SAMPLE, d ** -0.5, 0,
                                           None, (out_kv, sacc))
        t_bwd = timed(bwd, 10, 3, sync)
        del acc, delta, out_kv, sacc
    fl_fwd = 4.0 * (BLOCK + SAMPLE) * d * rows
    fl_bwd = 10.0 * (BLOCK + SAMPLE) * d * rows
    tf = lambda fl, ms: fl / (ms * 1e-3) / 1e12
    gbs = lambda by, ms: by / (ms * 1e-3) / 1e9
    out['kernels_ms'] = {'lsh_hash_per_tensor': t_hash, 'seg_sort_per_tensor': t_sort, 'gather_rows_per_tensor': t_gather,
                         'attn_tc_fwd_kernel': t_fwd, 'attn_tc_bwd_kernel': t_bwd}
    st = {
        'lsh_hash': {'bound': 'hbm', 'achieved': gbs(rows * (d * 2 + 4), t_hash), 'peak': peaks['hbm_gbs'], 'unit': 'GB/s'},
        'seg_sort': {'bound': 'hbm', 'achieved': gbs(rows * 8, t_sort), 'peak': peaks['hbm_gbs'], 'unit': 'GB/s'},
        'gather_rows': {'bound': 'hbm', 'achieved': gbs(rows * (2 * d * 2 + 4), t_gather), 'peak': peaks['hbm_gbs'], 'unit': 'GB/s'},
        'attn_tc_fwd_kernel': {'bound': 'tensor', 'achieved': tf(fl_fwd, t_fwd), 'peak': peaks['bf16_tflops'], 'unit': 'TFLOP/s'},
        'attn_tc_fwd_kernel_hbm': {'bound': 'hbm', 'achieved': gbs(rows * (4 * d * 2 + 12), t_fwd), 'peak': peaks['hbm_gbs'], 'unit': 'GB/s'},
    }
    for r_ in st.values():
        r_['frac'] = r_['achieved'] / r_['peak']
    out['stage_rooflines'] = st
    ach = tf(fl_bwd, t_bwd)
    out['roofline'] = {'bound': 'tensor', 'kernel': 'attn_tc_bwd_ws_kernel (hyper pattern, one launch per backward; the longest kernel of the step)', 'achieved': ach,
                       'peak': peaks['bf16_tflops'], 'unit': 'TFLOP/s', 'frac': ach / peaks['bf16_tflops'],
                       'traffic': kernel_traffic('attn_tc_bwd_ws_kernel', rows),
                       'peak_source': peaks['src'], 'launch_ms': t_bwd, 'algorithmic_flops_per_launch': fl_bwd,
                       'algorithmic_bytes_per_launch': rows * (7 * d * 2 + 8)}
    # the same step with uniformly sampled, importance-weighted key columns (fresh draws every call)
    if not causal:
        umod = ha.HyperAttention(input_dim=d, lsh_num_projs=BITS, block_size=BLOCK, sample_size=SAMPLE, min_seq_len=MIN_SEQ,
                                 rng=torch.Generator().manual_seed(1234), sampling='uniform').to(device=dev, dtype=torch.bfloat16)
        def u_fwd_bwd():
            oo = umod(q, k, v)
            return torch.autograd.grad(oo, (q, k, v), do)
        u_fwd_bwd()
        out['uniform_sampling'] = {'fwd_bwd_ms': timed(u_fwd_bwd, 5, 2, sync)}
    # exact attention of the same shape: our sm_100a flash kernel and the library kernel behind torch SDPA
    with torch.no_grad():
        t_ours = timed(lambda: ops.flash_attn_func(T(qd), T(kd), T(vd), None, True), 2, 1, sync)
    out['exact_flash'] = {'ours_causal_fwd_ms': t_ours, 'ours_causal_fwd_tflops': 2.0 * n * n * d * hpg / (t_ours * 1e-3) / 1e12}
    try:
        import torch.nn.functional as F
        qs, ks, vs = [t.detach().clone().requires_grad_() for t in (q, k, v)]
        f = lambda: F.scaled_dot_product_attention(qs, ks, vs, is_causal=True)
        t_f = timed(lambda: f(), 2, 1, sync)
        def fb():
            oo = f()
            torch.autograd.grad(oo, (qs, ks, vs), do)
        t_fb = timed(fb, 2, 1, sync)
        out['exact_flash'].update({'sdpa_causal_fwd_ms': t_f, 'sdpa_causal_fwd_bwd_ms': t_fb,
                                   'causal_fwd_speedup_vs_sdpa': t_f / tc_f, 'causal_fwd_bwd_speedup_vs_sdpa': t_fb / tc_fb})
        del qs, ks, vs
    except Exception as e:   # the comparator is informative only
        out['exact_flash']['sdpa_error'] = str(e)[:200]
    try:
        out['cpu_baseline'] = cpu_baseline(args.workload, n, d, args.cpu_heads, heads, seed)
    except Exception as e:
        out['cpu_baseline'] = {'error': str(e)[:200]}
    return out


if __name__ == '__main__':
    main()
