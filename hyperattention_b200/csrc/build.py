"""Builds libhyperattn_b200.so for sm_100a with nvcc, in-tree (next to the Python package).

    python hyperattention_b200/csrc/build.py [--force] [--verbose] [--timing]

Object files are cached under csrc/build/ and rebuilt when a source or header is newer.  --timing builds a second
library, libhyperattn_b200_timing.so, with the kernels' per-phase cycle counters compiled in (-DHA_PHASE_TIMING; read by
``python -m hyperattention_b200.phase_timing``); the product library never carries them.
"""
import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
SOURCES = ['stream_kernels.cu', 'seg_sort.cu', 'attn_simt.cu', 'attn_tc_fwd.cu', 'attn_tc_fwd_ws.cu', 'attn_tc_bwd.cu', 'attn_tc_bwd_ws.cu', 'attn_api.cu', 'causal.cu']
LIB = os.path.join(PKG, 'libhyperattn_b200.so')
NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-std=c++17', '-lineinfo', '-Xcompiler', '-fPIC',
              '-I' + os.path.join(ROOT, 'include'), '-I' + HERE]


def _newer(path, deps):
    if not os.path.exists(path):
        return True
    t = os.path.getmtime(path)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, timing=False):
    nvcc = os.environ.get('NVCC', 'nvcc')
    bdir = os.path.join(HERE, 'build', 'timing') if timing else os.path.join(HERE, 'build')
    lib = os.path.join(PKG, 'libhyperattn_b200_timing.so') if timing else LIB
    flags = NVCC_FLAGS + (['-DHA_PHASE_TIMING'] if timing else [])
    os.makedirs(bdir, exist_ok=True)
    headers = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith('.cuh')]
    headers.append(os.path.join(ROOT, 'include', 'hyperattn_b200.h'))
    sources = [f for f in SOURCES if os.path.exists(os.path.join(HERE, f))]
    extra = sorted(f for f in os.listdir(HERE) if f.endswith('.cu') and f not in SOURCES)
    sources += extra
    objs = []
    jobs = []
    for src in sources:
        s = os.path.join(HERE, src)
        o = os.path.join(bdir, src[:-3] + '.o')
        objs.append(o)
        if force or _newer(o, [s] + headers):
            cmd = [nvcc] + flags + (['-Xptxas', '-v'] if verbose else []) + ['-c', s, '-o', o]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(' '.join(cmd) + '\n' + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError('nvcc failed for ' + cmd[-3])
    if force or jobs or _newer(lib, objs):
        cmd = [nvcc, '-shared', '-o', lib] + objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError('link failed')
    return lib


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--force', action='store_true')
    ap.add_argument('--verbose', action='store_true')
    ap.add_argument('--timing', action='store_true')
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.timing))
