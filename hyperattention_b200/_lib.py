"""ctypes binding of libhyperattn_b200.so (declared in include/hyperattn_b200.h).

The library is built in-tree by ``hyperattention_b200/csrc/build.py``.  There is no fallback: if it is missing or a
call returns a non-zero status, an exception is raised.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'libhyperattn_b200.so')

HA_OK = 0
BF16, FP16, FP32 = 0, 1, 2
MODE_HYPER, MODE_FLASH = 0, 1
FLAG_CAUSAL, FLAG_SMOOTH, FLAG_MERGE, FLAG_MERGE_EXACT, FLAG_BWD_REF_SMOOTH, FLAG_FORCE_SIMT, FLAG_BWD_KV_INIT, FLAG_NO_WS = 1, 2, 4, 8, 16, 32, 64, 128
FLAG_CHECK_INDICES = 256
DEV_TIMEOUT, DEV_BAD_INDEX, DEV_BAD_LAUNCH = 1, 2, 3

_STATUS = {-1: 'invalid argument (shape / stride / size not accepted)', -2: 'unsupported dtype',
           -3: 'workspace missing or too small', -4: 'CUDA runtime error', 1: 'device-side wait timed out',
           -5: 'beyond a size limit of this entry point (too many segments / work items for one launch, or -- '
               'ha_seg_sort_noalloc -- more scratch than the built-in array holds: use ha_seg_sort with a workspace)'}

i32, i64, f32, vp = C.c_int32, C.c_int64, C.c_float, C.c_void_p


class AttnParams(C.Structure):
    _fields_ = [
        ('mode', i32), ('flags', i32), ('dtype', i32),
        ('B', i32), ('H', i32), ('n', i32), ('d', i32), ('dv', i32),
        ('segs_per_head', i32), ('span', i32), ('q_off', i32), ('k_off', i32), ('m_q', i32), ('m_k', i32),
        ('block_size', i32), ('sample_size', i32), ('kv_group', i32), ('scale', f32),
        ('q', vp), ('k', vp), ('v', vp),
        ('q_sb', i64), ('q_sh', i64), ('q_sn', i64), ('k_sb', i64), ('k_sh', i64), ('k_sn', i64),
        ('v_sb', i64), ('v_sh', i64), ('v_sn', i64),
        ('q_idx', vp), ('k_idx', vp), ('sample_idx', vp),
        ('o', vp), ('o_sb', i64), ('o_sh', i64), ('o_sn', i64),
        ('lse', vp), ('part_o', vp), ('part_lse', vp),
        ('d_o', vp), ('do_sb', i64), ('do_sh', i64), ('do_sn', i64),
        ('delta', vp), ('dq_acc', vp), ('dk_acc', vp), ('dv_acc', vp),
        ('status', vp), ('status_host', vp),
        ('sample_logw', vp), ('sample_mask', vp),
        ('dk_out', vp), ('dv_out', vp), ('dk_sacc', vp), ('dv_sacc', vp), ('dq_out', vp),
    ]


class CausalParams(C.Structure):
    _fields_ = [
        ('dtype', i32), ('flags', i32),
        ('B', i32), ('H', i32), ('n', i32), ('d', i32), ('dv', i32),
        ('levels', i32), ('block_size', i32), ('sample_size', i32), ('lsh_bits', i32), ('keep_parts', i32),
        ('min_seq_len', i32), ('kv_group', i32), ('scale', f32),
        ('q', vp), ('k', vp), ('v', vp), ('proj', vp), ('o', vp), ('lse', vp),
        ('saved', vp), ('saved_bytes', i64), ('scratch', vp), ('scratch_bytes', i64),
        ('d_o', vp), ('dq', vp), ('dk', vp), ('dv_out', vp), ('status', vp), ('status_host', vp),
    ]


# name -> (restype, argtypes); every symbol include/hyperattn_b200.h declares
SIGNATURES = {
    'ha_version': (C.c_char_p, []),
    'ha_last_cuda_error': (C.c_char_p, []),
    'ha_launch_count': (i64, []),
    'ha_lsh_hash': (C.c_int, [vp, i64, i64, i64, i32, i32, i32, i32, i32, vp, i32, vp, vp]),
    'ha_seg_sort_workspace_bytes': (i64, [i32, i32, i32, i32, i32]),
    'ha_seg_sort': (C.c_int, [vp, i32, i32, i32, i32, i32, i32, vp, vp, i64, vp]),
    'ha_seg_sort_noalloc': (C.c_int, [vp, i32, i32, i32, i32, i32, i32, vp, vp]),
    'ha_gather_rows': (C.c_int, [vp, i64, i64, i64, i32, i32, i32, i32, vp, i32, vp, vp]),
    'ha_attn_fwd': (C.c_int, [C.POINTER(AttnParams), vp]),
    'ha_attn_bwd': (C.c_int, [C.POINTER(AttnParams), vp]),
    'ha_attn_bwd_direct_level': (C.c_int, [C.POINTER(AttnParams)]),
    'ha_attn_bwd_finish': (C.c_int, [C.POINTER(AttnParams), vp]),
    'ha_sample_weights': (C.c_int, [vp, vp, i32, i32, i32, i32, i32, vp, vp, vp, vp]),
    'ha_delta': (C.c_int, [vp, i64, i64, i64, vp, i64, i64, i64, i32, i32, i32, i32, i32, vp, vp]),
    'ha_cast_from_f32': (C.c_int, [vp, vp, i64, i32, vp]),
    'ha_lse_merge': (C.c_int, [vp, vp, vp, vp, i64, i32, i32, i32, vp]),
    'ha_noncausal_saved_bytes': (i64, [C.POINTER(CausalParams)]),
    'ha_noncausal_scratch_bytes': (i64, [C.POINTER(CausalParams), i32]),
    'ha_noncausal_fwd': (C.c_int, [C.POINTER(CausalParams), vp]),
    'ha_noncausal_bwd': (C.c_int, [C.POINTER(CausalParams), vp]),
    'ha_wait_probe': (C.c_int, [vp, vp, i32, vp]),
    'ha_causal_saved_bytes': (i64, [C.POINTER(CausalParams)]),
    'ha_causal_scratch_bytes': (i64, [C.POINTER(CausalParams), i32]),
    'ha_causal_fwd': (C.c_int, [C.POINTER(CausalParams), vp]),
    'ha_causal_bwd': (C.c_int, [C.POINTER(CausalParams), vp]),
}

_lib = None


def load():
    """Loads the shared library (once) and declares every entry point.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f'{LIB_PATH} is missing: build it with `python hyperattention_b200/csrc/build.py` '
                               '(there is no fallback implementation)')
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc, what):
    if rc != HA_OK:
        detail = _STATUS.get(rc, f'status {rc}')
        if rc == -4:
            detail += ': ' + load().ha_last_cuda_error().decode()
        if rc == -1:
            raise AssertionError(f'{what}: {detail}')   # the reference signals these conditions with assert
        raise RuntimeError(f'{what}: {detail}')
