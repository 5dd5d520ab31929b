"""ha_seg_sort_noalloc: the sort for embedders that cannot allocate device memory.

Such a caller (a serving process whose pools own all of HBM, a plug-in without torch or cudaMalloc rights) passes
only its input and output buffers; the scratch is the library's own fixed array.  The test drives the entry point
directly through the C ABI and requires the permutation to be identical to the one the workspace-taking entry point
produces, on two calls in a row: the second call is smaller and of a different key width, so it runs on top of the
counters the first one left behind.  This file sorts last in collection order on purpose.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_BYTES = 4 << 20


def _noalloc_sort(lib, codes, bits):
    rows, n = codes.shape
    idx = torch.full((rows, n), -1, dtype=torch.int32, device=codes.device)
    rc = lib.ha_seg_sort_noalloc(C.c_void_p(codes.data_ptr()), rows, n, n, 0, n, bits, C.c_void_p(idx.data_ptr()),
                                 C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, idx


def test_noalloc_sort_matches_workspace_sort_on_consecutive_calls():
    import hyperattention_b200 as ha
    from hyperattention_b200 import _lib
    lib = _lib.load()
    torch.manual_seed(7)
    for rows, n, bits in [(8, 65536, 8), (3, 5000, 16), (2, 4096, 5)]:
        codes = torch.randint(0, 2 ** bits, (rows, n), dtype=torch.int32, device='cuda')
        want = ha.seg_sort(codes, bits)                       # existing entry point, caller-provided workspace
        assert lib.ha_seg_sort_workspace_bytes(rows, n, n, n, bits) <= STATIC_BYTES
        rc, got = _noalloc_sort(lib, codes, bits)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.equal(got, want)                         # integer result: bit-exact
        assert torch.equal(got.cpu().long(), torch.sort(codes.cpu(), dim=-1, stable=True)[1])


def test_noalloc_sort_refuses_what_does_not_fit():
    from hyperattention_b200 import _lib
    lib = _lib.load()
    rows, n = 64, 131072                                      # 8 MiB of counters: beyond the built-in array
    assert lib.ha_seg_sort_workspace_bytes(rows, n, n, n, 8) > STATIC_BYTES
    codes = torch.zeros(1, dtype=torch.int32, device='cuda')  # never dereferenced: the call is refused up front
    launches = lib.ha_launch_count()
    rc = lib.ha_seg_sort_noalloc(C.c_void_p(codes.data_ptr()), rows, n, n, 0, n, 8, C.c_void_p(codes.data_ptr()), None)
    assert rc == -5 and lib.ha_launch_count() == launches
    with pytest.raises(RuntimeError, match='built-in array'):
        _lib.check(rc, 'ha_seg_sort_noalloc')
