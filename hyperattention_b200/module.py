"""The HyperAttention module: same constructor, attributes, forward signature and return values as the reference's
torch.nn.Module (hyper_attention.py:9-132), computed by the sm_100a kernels of this package.

Additional keyword arguments (all optional, accepted through **kwargs like the reference's unused kwargs):
  grad_mode   'reference' (default): gradients follow the reference's conventions (d(lse) dropped by both attention
              Functions, every merged part differentiated on its own); 'exact': gradient of the returned output.
  merge_mode  'reference' (default): the merge of src/attn_utils.py:21-24 (weight rounded to the tensor dtype, eps
              inside the log); 'exact': plain log-sum-exp combine.
  rng         torch.Generator used to draw proj_dir (the reference's AngularLSHTriton has the same argument).
  fused_causal  True (default): run regular causal shapes through the single-call schedule; False: always use the
              per-level path built from the individual operators.
  fused_calls True (default): a non-causal call on contiguous inputs is one library call each way (hash, sort and attention;
              delta, backward and finishing pass); False: one call per operator, as strided inputs and the uniform
              sampling mode always do.
"""
import math

import torch

from . import _lib as L
from . import ops


class AngularLSH(torch.nn.Module):
    """Sign-random-projection LSH with Gray-coded bucket ids; buffers and methods as AngularLSHTriton
    (src/angular_lsh_triton.py:148-185): perm int32 [2^r], proj_dir [*dim, r], enc_vec int64 [1,1,1,r], all
    non-persistent."""

    def __init__(self, num_projs, dim, rng=None):
        super().__init__()
        self.num_projs = num_projs
        if num_projs > 0:
            b = torch.arange(2 ** num_projs, dtype=torch.int64)
            self.register_buffer('perm', (b ^ (b >> 1)).to(torch.int32), persistent=False)
            self.register_buffer('proj_dir', torch.randn(dim + (num_projs,), generator=rng), persistent=False)
            self.register_buffer('enc_vec', 2 ** torch.arange(self.num_projs).view(1, 1, 1, -1), persistent=False)
        else:
            raise ValueError("Invalid value for num_projs")
        self._proj_cache = None

    def proj_f32(self):
        """proj_dir as a contiguous float32 [d, r] tensor (values exactly those of the stored dtype)."""
        pd = self.proj_dir
        key = (pd.data_ptr(), pd._version, pd.dtype, pd.device)
        if self._proj_cache is None or self._proj_cache[0] != key:
            self._proj_cache = (key, pd.detach().reshape(pd.shape[-2], pd.shape[-1]).to(torch.float32).contiguous())
        return self._proj_cache[1]

    def hash_torch(self, mat):
        """The reference's PyTorch formulation (src/angular_lsh_triton.py:175-179), kept for comparisons."""
        mask = torch.einsum('...nd,...dr -> ...nr', mat, self.proj_dir)
        mask = mask > 0
        bin_ids = (mask * self.enc_vec).sum(-1)
        return self.perm[bin_ids]

    def hash_cuda(self, mat, out=None):
        assert self.proj_dir.shape[:-2] == (1,) * (self.proj_dir.dim() - 2), 'one projection shared by all heads'
        assert mat.dtype == self.proj_dir.dtype, 'All three tensors must have the same type'
        return ops.lsh_hash(mat, self.proj_f32(), out)

    hash_triton = hash_cuda   # the name callers of the reference use

    def __repr__(self):
        return f"AngularLSH(num_proj={self.num_projs}, proj_dir.shape={self.proj_dir.shape})"


class HyperAttention(torch.nn.Module):

    def __init__(self, input_dim=64, lsh_num_projs=8, block_size=256, sample_size=256, min_seq_len=2048,
                 smooth_block=False, **kwargs):
        """block_size and sample_size must be divisible by 128 (as in the reference)."""
        super().__init__()
        self.input_dim = input_dim
        self.lsh_num_projs = lsh_num_projs
        self.block_size = block_size
        self.sample_size = sample_size
        self.min_seq_len = min_seq_len
        self.smooth_block = smooth_block
        self.grad_mode = kwargs.get('grad_mode', 'reference')
        self.merge_mode = kwargs.get('merge_mode', 'reference')
        self.fused_causal = kwargs.get('fused_causal', True)
        self.fused_calls = kwargs.get('fused_calls', True)
        self.kernel_flags = kwargs.get('kernel_flags', 0)
        # 'reference': sampled part = key rows 0..sample_size-1, unweighted (what the reference's kernels compute).
        # 'uniform':   sample_size distinct key rows per (batch, head), one uniform draw per stratum, the query tile's own block
        #              excluded, importance-weighted to stand for all keys outside the block (no reference counterpart).
        self.sampling = kwargs.get('sampling', 'reference')
        self.sample_generator = kwargs.get('sample_generator')   # torch.Generator on the inputs' device, or None
        # Without a generator the draws come from a counter-based function of (sample_seed, number of the call, batch*head,
        # slot) evaluated with integer ops on the device: reproducible, and computable bit for bit on the host.
        self.sample_seed = int(kwargs.get('sample_seed', 0))
        self.sample_calls = 0
        self.last_sample_idx = None
        assert self.grad_mode in ('reference', 'exact') and self.merge_mode in ('reference', 'exact')
        assert self.sampling in ('reference', 'uniform')
        self.lsh = AngularLSH(num_projs=self.lsh_num_projs, dim=(1, 1, input_dim), rng=kwargs.get('rng'))

    # ------------------------------------------------------------------------------------------
    def _counter_u24(self, rows, S, device):
        """24 uniform bits per (row, slot): top bits of the splitmix64 finaliser of (sample_seed, call number, row * S + slot),
        in int64 arithmetic (wrap-around products; logical right shifts written as arithmetic shift + mask)."""
        def c(v):                                   # a 64-bit constant as a signed Python int
            return v - (1 << 64) if v >= (1 << 63) else v
        def shr(x, k):
            return (x >> k) & ((1 << (64 - k)) - 1)
        def wrap(v):
            v &= (1 << 64) - 1
            return c(v)
        base = wrap(self.sample_seed * 0x9E3779B97F4A7C15 + self.sample_calls * 0xD1B54A32D192ED03)
        x = torch.arange(rows * S, device=device, dtype=torch.int64) + base
        x = (x ^ shr(x, 30)) * c(0xBF58476D1CE4E5B9)
        x = (x ^ shr(x, 27)) * c(0x94D049BB133111EB)
        x = x ^ shr(x, 31)
        return shr(x, 40).view(rows, S)

    def _flags(self):
        f = self.kernel_flags
        if self.smooth_block:
            f |= L.FLAG_SMOOTH
            if self.grad_mode == 'reference':
                f |= L.FLAG_BWD_REF_SMOOTH
        if self.merge_mode == 'exact':
            f |= L.FLAG_MERGE_EXACT
        return f

    def _causal_levels(self, n):
        levels = 0
        while (n >> levels) > self.min_seq_len and (n >> levels) % 2 == 0:
            levels += 1
        return levels

    def _regular_causal(self, n):
        """True when the single-call schedule applies: n halves evenly down to leaves <= min_seq_len, every rectangle is
        a whole number of 128-row tiles and those on the hyper pattern hold the sampled rows.  (Rectangles shorter than
        min_seq_len -- only the deepest ones can be -- are exact, hyper_attention.py:109-113; the schedule does the same.)"""
        levels = self._causal_levels(n)
        leaf = n >> levels
        smallest_hyper = 2 * leaf if self.min_seq_len > leaf else leaf
        return levels >= 1 and leaf <= self.min_seq_len and leaf % 128 == 0 and self.sample_size % 128 == 0 \
            and (self.sample_size <= smallest_hyper or (levels == 1 and self.min_seq_len > leaf))

    def forward(self, query: torch.tensor, key: torch.tensor, value: torch.tensor, scale=None, causal=False,
                return_lse=False):
        """query, key [B, H, n, d]; value [B, H, n, dv]; returns attn [B, H, n, dv] (and lse, float32 [B, H, n, 1];
        [B, H, ceil(n/128)*128] when a causal call is short enough to be a single exact leaf, as in the reference)."""
        # The reference copies its inputs here (hyper_attention.py:38-40).  The kernels take (batch, head, row) strides,
        # so only a tensor whose rows are not contiguous is copied; the causal schedule below, which addresses
        # [B, H, n, d] memory directly, makes its own copies where it needs them.
        query, key, value = [t if t.stride(-1) == 1 else t.contiguous() for t in (query, key, value)]
        n_query = query.shape[2]
        batch_size, n_heads, n_key, dim = key.shape
        scale = scale or dim ** (-0.5)
        assert n_query == n_key
        if n_heads != query.shape[1]:
            # Grouped-query attention: fewer K/V heads than query heads (not in the reference, which is handed K/V already
            # expanded to every query head, chatglm_fast_attention.py:53-58).  The single-call paths hash and sort K once
            # per K/V head and never expand; every other path expands here.
            assert query.shape[1] % n_heads == 0 and value.shape[1] == n_heads, 'query heads must be a multiple of the K/V heads'
            grouped_ok = self.sampling == 'reference' and n_key >= self.min_seq_len and all(
                t.is_contiguous() for t in (query, key, value)) and \
                ((causal and n_key > self.min_seq_len and self.fused_causal and self._regular_causal(n_key)) or (not causal and self.fused_calls and query.dtype == self.lsh.proj_dir.dtype))
            if not grouped_ok:
                rep = query.shape[1] // n_heads
                key, value = key.repeat_interleave(rep, dim=1), value.repeat_interleave(rep, dim=1)

        if causal is False:
            attn, lse = self.forward_no_causal_mask(query, key, value, scale)
        elif n_key <= self.min_seq_len:
            attn, lse = ops.flash_attn_func(query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), None, True,
                                            scale, self.kernel_flags & L.FLAG_FORCE_SIMT)
            attn = attn.transpose(1, 2)
        elif self.fused_causal and self.sampling == 'reference' and self._regular_causal(n_key):
            attn, lse = ops.CausalHyperFunc.apply(query, key, value, self.lsh.proj_f32(), self._causal_levels(n_key),
                                                  self.block_size, self.sample_size, scale, self._flags(),
                                                  self.grad_mode == 'reference', self.min_seq_len)
            lse = lse.unsqueeze(-1)
        else:
            attn, lse = self._causal_by_levels(query.contiguous(), key.contiguous(), value.contiguous(), scale)
        if not return_lse:
            return attn
        return attn, lse

    def _causal_by_levels(self, query, key, value, scale):
        """One half-split built from the individual operators (any shape the reference accepts, including the
        zero-row padding of odd lengths, hyper_attention.py:59-96); recurses through forward()."""
        B, H, n, dim = key.shape
        odd = n % 2
        if odd:
            query, key, value = [torch.nn.functional.pad(t, (0, 0, 0, 1)) for t in (query, key, value)]
        m = query.shape[2] // 2
        halves = lambda t: t.reshape(B, 2 * H, m, t.shape[-1])
        attn_d, lse_d = self.forward(halves(query), halves(key), halves(value), scale, True, True)
        attn_d = attn_d.reshape(B, H, 2 * m, -1)
        lse_d = lse_d.reshape(B, H, 2 * m, 1)          # fails like the reference when a leaf is not 128-aligned
        attn_r, lse_r = self.forward_no_causal_mask(query[:, :, m:], key[:, :, :m], value[:, :, :m], scale)
        if self.merge_mode == 'exact':
            mx = torch.maximum(lse_d[:, :, m:], lse_r)
            w1, w2 = (lse_d[:, :, m:] - mx).exp(), (lse_r - mx).exp()
            low = ((attn_d[:, :, m:] * w1 + attn_r * w2) / (w1 + w2)).to(attn_r.dtype)
            lse_low = mx + (w1 + w2).log()
        else:
            low, lse_low = ops.add_self_attentions(attn_d[:, :, m:], lse_d[:, :, m:], attn_r, lse_r)
        attn = torch.cat((attn_d[:, :, :m], low), dim=-2)
        lse = torch.cat((lse_d[:, :, :m], lse_low), dim=-2)
        if odd:
            attn, lse = attn[:, :, :-1], lse[:, :, :-1]
        return attn, lse

    def forward_no_causal_mask(self, query, key, value, scale):
        """hyper_attention.py:103-132: exact attention below min_seq_len, otherwise hash -> stable sort -> fused
        block-diagonal + sampled attention."""
        B, H, n_query, dim = query.shape
        if self.min_seq_len > n_query:
            attn, lse = ops.flash_attn_func(query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), None, False,
                                            scale, self.kernel_flags & L.FLAG_FORCE_SIMT)
        elif self.sampling == 'reference' and self.fused_calls and query.is_contiguous() and key.is_contiguous() \
                and value.is_contiguous() and query.dtype == self.lsh.proj_dir.dtype:
            # hash, sort, attention (and, in the backward, delta, the backward kernel, the finishing pass) in one library call
            attn, lse = ops.NonCausalHyperFunc.apply(query, key, value, self.lsh.proj_f32(), self.block_size, self.sample_size,
                                                     scale, self._flags())
            return attn, lse.unsqueeze(-1)
        else:
            bits = self.lsh_num_projs
            # codes of q and k side by side: one segmented sort call covers both
            codes = torch.empty(2, B, H, n_query, dtype=torch.int32, device=query.device)
            self.lsh.hash_cuda(query, codes[0])
            self.lsh.hash_cuda(key, codes[1])
            idx = ops.seg_sort(codes.view(2 * B * H, n_query), bits)
            q_idx, k_idx = idx[:B * H].view(B, H, n_query), idx[B * H:].view(B, H, n_query)
            sample_idx, weighted = None, False
            if self.sampling == 'uniform' and self.sample_size > 0:
                # distinct rows with equal inclusion probability per (batch, head): one uniform draw from each of
                # sample_size equal strata of the key range (cheaper than a draw without replacement, lower variance)
                n_k, S = key.shape[2], self.sample_size
                edges = (torch.arange(S + 1, device=key.device, dtype=torch.int64) * n_k) // S
                size = edges[1:] - edges[:-1]
                if self.sample_generator is not None:
                    u = torch.rand(B * H, S, device=key.device, generator=self.sample_generator)
                    sample_idx = (edges[:-1] + torch.minimum((u * size).long(), size - 1)).to(torch.int32)
                else:
                    sample_idx = (edges[:-1] + ((size * self._counter_u24(B * H, S, key.device)) >> 24)).to(torch.int32)
                    self.sample_calls += 1
                self.last_sample_idx = sample_idx.view(B, H, self.sample_size)
                weighted = True
            attn, lse = ops.hyper_attn_func(query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2),
                                            q_idx.transpose(1, 2), k_idx.transpose(1, 2), self.block_size, self.sample_size,
                                            scale, self.smooth_block, sample_idx, self._flags() & ~L.FLAG_SMOOTH, weighted)
        attn = attn.transpose(1, 2)
        return attn, lse.unsqueeze(-1)
