"""CPU-side checks of the boundary: the shared library loads, exports every symbol the header declares, rejects bad
arguments with the documented status codes (no kernel is launched), and the module mirrors the reference's surface."""
import ctypes as C
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope='module')
def lib():
    from hyperattention_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        import __graft_entry__
        __graft_entry__.build()
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    from hyperattention_b200 import _lib
    header = open(os.path.join(ROOT, 'include', 'hyperattn_b200.h')).read()
    declared = set(re.findall(r'\b(ha_[a-z0-9_]+)\s*\(', header))
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    for name in declared:
        assert getattr(lib, name) is not None
    assert b'sm_100a' in lib.ha_version()


def test_struct_layout_matches_header(lib):
    """sizes computed from the header's field lists with natural alignment"""
    from hyperattention_b200 import _lib
    assert C.sizeof(_lib.AttnParams) == 18 * 4 + 3 * 8 + 9 * 8 + 3 * 8 + 8 + 3 * 8 + 3 * 8 + 8 + 3 * 8 + 4 * 8 + 2 * 8 + 2 * 8 + 5 * 8
    assert C.sizeof(_lib.CausalParams) == 15 * 4 + 4 + 6 * 8 + 4 * 8 + 6 * 8


def test_argument_validation_without_a_gpu(lib):
    from hyperattention_b200 import _lib
    assert lib.ha_lsh_hash(None, 0, 0, 0, 1, 1, 1, 64, 0, None, 8, None, None) == -1
    assert lib.ha_seg_sort(None, 1, 128, 128, 0, 128, 8, None, None, 0, None) == -1
    assert lib.ha_seg_sort_workspace_bytes(32, 131072, 131072, 131072, 8) == 32 * 128 * 256 * 4
    p = _lib.AttnParams()
    assert lib.ha_attn_fwd(C.byref(p), None) == -1
    dummy = C.c_void_p(256)
    p.mode, p.dtype, p.B, p.H, p.n, p.d, p.dv = _lib.MODE_HYPER, 7, 1, 1, 256, 64, 64
    assert lib.ha_attn_fwd(C.byref(p), None) == -2            # dtype
    p.dtype = _lib.BF16
    p.segs_per_head, p.span, p.m_q, p.m_k, p.block_size, p.sample_size = 1, 256, 200, 200, 128, 128
    p.q = p.k = p.v = p.o = p.lse = p.q_idx = p.k_idx = dummy
    assert lib.ha_attn_fwd(C.byref(p), None) == -1            # 200 rows: not a multiple of 128
    p.m_q = p.m_k = 256
    p.sample_size = 100
    assert lib.ha_attn_fwd(C.byref(p), None) == -1            # sample_size % 128
    p.sample_size = 384
    assert lib.ha_attn_fwd(C.byref(p), None) == -1            # more sampled rows than keys
    p.sample_size = 128
    p.sample_logw = dummy
    assert lib.ha_attn_fwd(C.byref(p), None) == -1            # log weights without the dropped-slot mask
    p.sample_logw = None
    p.d_o = p.delta = p.dq_acc = dummy
    assert lib.ha_attn_bwd(C.byref(p), None) == -1            # neither accumulators nor direct outputs for dk / dv
    p.dk_out = dummy
    assert lib.ha_attn_bwd(C.byref(p), None) == -1            # dk_out without dv_out
    p.dv_out = dummy
    assert lib.ha_attn_bwd(C.byref(p), None) == -1            # sampled rows but no slot buffers
    p.mode, p.dk_sacc, p.dv_sacc = _lib.MODE_FLASH, dummy, dummy
    assert lib.ha_attn_bwd(C.byref(p), None) == -1            # direct dk / dv exists for the hyper pattern only
    p.mode, p.scale = _lib.MODE_HYPER, 0.125
    assert lib.ha_attn_bwd_direct_level(C.byref(p)) == 1      # 128 sampled rows: dk / dv only
    p.sample_size = 256
    assert lib.ha_attn_bwd_direct_level(C.byref(p)) == 1      # block size 128: one key tile per block
    p.block_size = 256
    assert lib.ha_attn_bwd_direct_level(C.byref(p)) == 2
    p.flags = _lib.FLAG_SMOOTH | _lib.FLAG_BWD_REF_SMOOTH
    assert lib.ha_attn_bwd_direct_level(C.byref(p)) == 1
    p.flags = _lib.FLAG_FORCE_SIMT
    assert lib.ha_attn_bwd_direct_level(C.byref(p)) == 0
    assert lib.ha_attn_bwd(C.byref(p), None) == -1            # ... and on the tensor-core kernel only
    p.flags, p.block_size, p.sample_size = 0, 128, 128
    p.dk_out = p.dv_out = p.dk_sacc = p.dv_sacc = None
    p.dq_out = dummy
    p.dk_acc = p.dv_acc = dummy
    assert lib.ha_attn_bwd(C.byref(p), None) == -1            # dq_out without dk_out / dv_out
    p.dq_out = p.dk_acc = p.dv_acc = None
    assert lib.ha_sample_weights(dummy, None, 1, 200, 128, 128, 0, dummy, dummy, dummy, None) == -1   # rows % 128
    assert lib.ha_sample_weights(dummy, None, 1, 256, 128, 384, 0, dummy, dummy, dummy, None) == -1   # more slots than rows
    assert lib.ha_sample_weights(None, None, 0, 256, 128, 128, 0, None, None, None, None) == 0        # nothing to do
    c = _lib.CausalParams()
    c.dtype, c.B, c.H, c.n, c.d, c.dv, c.levels, c.block_size, c.sample_size, c.lsh_bits = 0, 1, 32, 131072, 64, 64, 6, 256, 256, 8
    rows = 32 * 131072
    assert lib.ha_causal_saved_bytes(C.byref(c)) == 6 * 2 * (rows // 2 * 4)
    c.n = 131072 + 64
    assert lib.ha_causal_saved_bytes(C.byref(c)) == -1
    c.n, c.sample_size = 131072, 4096
    assert lib.ha_causal_saved_bytes(C.byref(c)) == -1        # leaves of 2048 rows cannot hold 4096 sampled rows


def test_module_surface_matches_reference():
    import hyperattention_b200 as ha
    import inspect
    sig = inspect.signature(ha.HyperAttention.__init__)
    assert list(sig.parameters)[:7] == ['self', 'input_dim', 'lsh_num_projs', 'block_size', 'sample_size', 'min_seq_len',
                                        'smooth_block']
    assert [sig.parameters[k].default for k in list(sig.parameters)[1:7]] == [64, 8, 256, 256, 2048, False]
    fsig = inspect.signature(ha.HyperAttention.forward)
    assert list(fsig.parameters) == ['self', 'query', 'key', 'value', 'scale', 'causal', 'return_lse']
    m = ha.HyperAttention(input_dim=128, lsh_num_projs=7)
    assert m.lsh.proj_dir.shape == (1, 1, 128, 7) and m.lsh.perm.dtype == torch.int32 and m.lsh.enc_vec.dtype == torch.int64
    assert len(m.state_dict()) == 0
    m16 = m.to(dtype=torch.bfloat16)
    assert m16.lsh.proj_dir.dtype == torch.bfloat16 and m16.lsh.perm.dtype == torch.int32
    # hash_torch is the reference's formula and runs on CPU
    x = torch.randn(1, 2, 50, 128)
    from oracle import hyper_oracle as O
    m32 = ha.HyperAttention(input_dim=128, lsh_num_projs=7)
    assert torch.equal(m32.lsh.hash_torch(x).int(), O.lsh_hash(x, m32.lsh.proj_dir))
    g = torch.Generator().manual_seed(5)
    a = ha.HyperAttention(rng=g).lsh.proj_dir
    b = ha.HyperAttention(rng=torch.Generator().manual_seed(5)).lsh.proj_dir
    assert torch.equal(a, b)


def test_cpu_tensors_fail_loudly():
    import hyperattention_b200 as ha
    m = ha.HyperAttention()
    q = torch.randn(1, 1, 2048, 64)
    with pytest.raises(AssertionError):
        m(q, q, q)


def test_causal_level_arithmetic():
    import hyperattention_b200 as ha
    m = ha.HyperAttention(min_seq_len=2048)
    assert m._causal_levels(131072) == 6 and m._regular_causal(131072)
    assert m._causal_levels(32768) == 4
    assert m._causal_levels(4096) == 1
    assert not m._regular_causal(2048 * 3 + 2)     # leaves not 128-aligned
    m2 = ha.HyperAttention(min_seq_len=256, sample_size=512)
    assert not m2._regular_causal(4096)            # leaves too short for the sampled rows


def test_counter_based_sample_indices_agree_with_the_oracle():
    """The uniform sampling mode's draws are a function of (seed, call, batch*head, slot) in integer arithmetic: the
    module's torch int64 version (run here on the CPU) and the oracle's numpy uint64 restatement agree bit for bit."""
    import torch
    import hyperattention_b200 as ha
    from oracle import hyper_oracle as O
    mod = ha.HyperAttention(input_dim=64, sample_size=256, sampling='uniform', sample_seed=2024)
    for call, (rows, n) in enumerate([(6, 4096), (3, 1000), (32, 131072)]):
        mod.sample_calls = call
        S = mod.sample_size
        u = mod._counter_u24(rows, S, 'cpu')
        edges = (torch.arange(S + 1, dtype=torch.int64) * n) // S
        size = edges[1:] - edges[:-1]
        idx = edges[:-1] + ((size * u) >> 24)
        want = O.uniform_sample_idx(2024, call, rows, S, n)
        assert torch.equal(idx, want)
        assert int(idx.min()) >= 0 and int(idx.max()) < n and bool((idx[:, 1:] > idx[:, :-1]).all())      # distinct, in range
    assert 0.45 < float(u.float().mean()) / 2 ** 24 < 0.55
