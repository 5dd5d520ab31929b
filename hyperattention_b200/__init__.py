"""B200-native HyperAttention: drop-in for the reference's HyperAttention module and operator functions."""
from .module import AngularLSH, HyperAttention
from .ops import (add_self_attentions, check_device_status, flash_attn_func, hyper_attn_func, indexing, launch_count, lse_merge_, lsh_hash,
                  sample_weights, seg_sort)

AngularLSHTriton = AngularLSH  # the reference's class name

__all__ = ['HyperAttention', 'AngularLSH', 'AngularLSHTriton', 'hyper_attn_func', 'flash_attn_func', 'add_self_attentions',
           'indexing', 'lsh_hash', 'seg_sort', 'lse_merge_', 'launch_count', 'check_device_status', 'sample_weights']
