"""ChatGLM2-style integration of HyperAttention: the attention-layer patch of the reference and a random-init decoder of
the ChatGLM2-6B shape to run it in (benchmark configuration 4).

* ``FastCoreAttention`` and ``patch_attention_layers`` mirror chatglm_fast_attention.py:8-70 and
  replace_llm_attention.py:6-44 of the reference: same constructor arguments, same layer-selection options, same
  [sq, b, heads, head_dim] calling convention, causal prefill only.
* ``ChatGLM2ShapedDecoder`` is written from the public description of the architecture (hidden 4096, 32 query heads of
  128, multi-query attention with 2 key/value groups, rotary embedding on half of each head, RMSNorm, SwiGLU MLP of
  13696, vocabulary 65024, 28 blocks), with the module nesting the patch expects
  (``model.transformer.encoder.layers[i].self_attention.core_attention``).  Weights are random (N(0, 0.02)); there
  is no checkpoint or tokenizer in this environment.  Everything outside the attention core is plain PyTorch.
"""
import math
from types import SimpleNamespace

import torch
import torch.nn.functional as F

from .module import HyperAttention

NUM_TOTAL_LAYERS = {
    'chatglm2-6b-32k': 28,
}


def select_patch_layers(num_total_layers, patch_config, num_patch_layers):
    """Indices of the blocks whose attention core is replaced (replace_llm_attention.py:10-35)."""
    n = num_total_layers if num_patch_layers < 0 else num_patch_layers
    t = num_total_layers
    table = {
        'last': lambda: range(t - 1, t - n - 1, -1),
        'first': lambda: range(n),
        'odd': lambda: range(1, t, 2),
        'even': lambda: range(0, t, 2),
        'odd_first': lambda: range(1, 2 * n, 2),
        'odd_last': lambda: range(t - 1, t - n, -1),
        'even_first': lambda: range(0, t, 2)[:n],
        'even_last': lambda: range(1, t, 2)[-n:],
    }
    if patch_config not in table:
        raise NotImplementedError(f"Invalid patch_config option: {patch_config}")
    return list(table[patch_config]())


class FastCoreAttention(torch.nn.Module):
    """Drop-in for the ChatGLM2 attention core backed by HyperAttention (chatglm_fast_attention.py:8-70)."""

    def __init__(self, config, layer_number, **kwargs):
        super().__init__()
        self.apply_query_key_layer_scaling = config.apply_query_key_layer_scaling
        self.attention_softmax_in_fp32 = config.attention_softmax_in_fp32 or self.apply_query_key_layer_scaling
        self.layer_number = max(1, layer_number)
        projection_size = config.kv_channels * config.num_attention_heads
        self.hidden_size_per_partition = projection_size
        self.hidden_size_per_attention_head = projection_size // config.num_attention_heads
        self.num_attention_heads_per_partition = config.num_attention_heads
        self.norm_factor = math.sqrt(self.hidden_size_per_attention_head)
        self.coeff = None
        if self.apply_query_key_layer_scaling:
            self.coeff = self.layer_number
            self.norm_factor *= self.coeff
        self.attention_dropout = torch.nn.Dropout(config.attention_dropout)
        # grouped_kv=True: the caller may hand over K/V with fewer heads than Q (multi-query / grouped-query models); K is then
        # hashed and sorted once per K/V head and never expanded.  False (default): heads already expanded, as the
        # reference's callers do (chatglm_fast_attention.py:53-58).
        self.grouped_kv = bool(kwargs.get('grouped_kv', False))
        self.attn_method = kwargs.get('attn_method')
        if self.attn_method != 'hyper':
            raise NotImplementedError("Invalid attn_method option")
        self.attn = HyperAttention(
            input_dim=self.hidden_size_per_attention_head,   # 128 for ChatGLM2 (hard-coded in the reference)
            lsh_num_projs=kwargs.get('lsh_num_projs'), block_size=kwargs.get('block_size'),
            sample_size=kwargs.get('sample_size'), min_seq_len=kwargs.get('min_seq_len'),
            smooth_block=kwargs.get('smooth_block'),
            **{k: v for k, v in kwargs.items() if k in ('grad_mode', 'merge_mode', 'rng', 'fused_causal')})

    def forward(self, query_layer, key_layer, value_layer, attention_mask):
        # [sq, b, heads, head_dim] -> [b, heads, sq, head_dim]
        query_layer, key_layer, value_layer = [t.permute(1, 2, 0, 3) for t in (query_layer, key_layer, value_layer)]
        assert attention_mask is None and query_layer.shape[2] == key_layer.shape[2], \
            'only causal prefill (no mask, equal query and key lengths) goes through HyperAttention'
        context_layer = self.attn(query_layer, key_layer, value_layer, causal=True)
        context_layer = context_layer.permute(2, 0, 1, 3)
        return context_layer.reshape(*context_layer.shape[:-2], self.hidden_size_per_partition)


def patch_attention_layers(model, model_name, patch_config, num_patch_layers, **kwargs):
    """Swaps ``core_attention`` of the selected blocks for FastCoreAttention (replace_llm_attention.py:6-44).
    ``num_total_layers`` may be passed to patch a model of the same structure with another depth."""
    total = kwargs.pop('num_total_layers', None) or NUM_TOTAL_LAYERS[model_name]
    indices = select_patch_layers(total, patch_config, num_patch_layers)
    if model_name != 'chatglm2-6b-32k':
        raise NotImplementedError(f'unsupported model {model_name}')
    print(f"patch_config: {patch_config}, attn_method: {kwargs['attn_method']}, num_patch_layers: {num_patch_layers}, "
          f"patch_indices: {indices}")
    ref = next(model.parameters())
    for i in indices:
        core = FastCoreAttention(model.config, i, **kwargs).to(device=ref.device, dtype=ref.dtype)
        model.transformer.encoder.layers[i].self_attention.core_attention = core
    return indices


# ------------------------------------------------------------------------------------------------
# a decoder of the ChatGLM2-6B shape
# ------------------------------------------------------------------------------------------------
def chatglm2_config(**over):
    cfg = dict(num_layers=28, hidden_size=4096, num_attention_heads=32, kv_channels=128, multi_query_group_num=2,
               ffn_hidden_size=13696, padded_vocab_size=65024, layernorm_epsilon=1e-5, rope_ratio=50.0,
               apply_query_key_layer_scaling=True, attention_softmax_in_fp32=True, attention_dropout=0.0)
    cfg.update(over)
    return SimpleNamespace(**cfg)


class RMSNorm(torch.nn.Module):
    def __init__(self, dim, eps):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        v = x.float().pow(2).mean(-1, keepdim=True)
        return (self.weight * (x.float() * torch.rsqrt(v + self.eps))).to(x.dtype)


class ExactCoreAttention(torch.nn.Module):
    """The stock attention core: exact causal softmax attention on [sq, b, heads, head_dim] tensors."""

    def __init__(self, config, layer_number):
        super().__init__()
        self.hidden = config.kv_channels * config.num_attention_heads

    def forward(self, q, k, v, attention_mask):
        q, k, v = [t.permute(1, 2, 0, 3) for t in (q, k, v)]
        o = F.scaled_dot_product_attention(q, k, v, is_causal=attention_mask is None and q.shape[2] == k.shape[2])
        o = o.permute(2, 0, 1, 3)
        return o.reshape(*o.shape[:-2], self.hidden)


def _rope_cache(seq_len, rot_dim, ratio, device, dtype):
    """cos/sin of the rotary angles for positions 0..seq_len-1 over rot_dim/2 frequency pairs."""
    base = 10000.0 * ratio
    inv = 1.0 / (base ** (torch.arange(0, rot_dim, 2, device=device, dtype=torch.float32) / rot_dim))
    ang = torch.outer(torch.arange(seq_len, device=device, dtype=torch.float32), inv)      # [sq, rot_dim/2]
    return torch.stack([ang.cos(), ang.sin()], dim=-1).to(dtype)                          # [sq, rot_dim/2, 2]


def _apply_rope(x, cache):
    """x [sq, b, heads, hn]; rotates consecutive element pairs of the first half of hn."""
    sq, b, h, hn = x.shape
    rot = cache.shape[1] * 2
    xr, xp = x[..., :rot], x[..., rot:]
    xr = xr.reshape(sq, b, h, rot // 2, 2)
    c = cache[:sq].view(sq, 1, 1, rot // 2, 2)
    out = torch.stack([xr[..., 0] * c[..., 0] - xr[..., 1] * c[..., 1], xr[..., 1] * c[..., 0] + xr[..., 0] * c[..., 1]], -1)
    return torch.cat([out.flatten(3), xp], dim=-1)


class SelfAttention(torch.nn.Module):
    def __init__(self, config, layer_number):
        super().__init__()
        self.heads, self.hn, self.groups = config.num_attention_heads, config.kv_channels, config.multi_query_group_num
        proj = self.heads * self.hn
        self.query_key_value = torch.nn.Linear(config.hidden_size, proj + 2 * self.groups * self.hn, bias=True)
        self.core_attention = ExactCoreAttention(config, layer_number)
        self.dense = torch.nn.Linear(proj, config.hidden_size, bias=False)

    def forward(self, x, rope):
        sq, b, _ = x.shape
        qkv = self.query_key_value(x)
        q, k, v = qkv.split([self.heads * self.hn, self.groups * self.hn, self.groups * self.hn], dim=-1)
        q = q.view(sq, b, self.heads, self.hn)
        k = k.view(sq, b, self.groups, self.hn)
        v = v.view(sq, b, self.groups, self.hn)
        q, k = _apply_rope(q, rope), _apply_rope(k, rope)
        rep = self.heads // self.groups
        # multi-query: every key/value group serves heads/groups query heads; expanded before the core, as the
        # attention core of the original model expects equal head counts
        if not getattr(self.core_attention, 'grouped_kv', False):
            k = k.unsqueeze(3).expand(-1, -1, -1, rep, -1).reshape(sq, b, self.heads, self.hn)
            v = v.unsqueeze(3).expand(-1, -1, -1, rep, -1).reshape(sq, b, self.heads, self.hn)
        return self.dense(self.core_attention(q, k, v, None))


class MLP(torch.nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense_h_to_4h = torch.nn.Linear(config.hidden_size, 2 * config.ffn_hidden_size, bias=False)
        self.dense_4h_to_h = torch.nn.Linear(config.ffn_hidden_size, config.hidden_size, bias=False)

    def forward(self, x):
        a, g = self.dense_h_to_4h(x).chunk(2, dim=-1)
        return self.dense_4h_to_h(F.silu(a) * g)


class GLMBlock(torch.nn.Module):
    def __init__(self, config, layer_number):
        super().__init__()
        self.input_layernorm = RMSNorm(config.hidden_size, config.layernorm_epsilon)
        self.self_attention = SelfAttention(config, layer_number)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.layernorm_epsilon)
        self.mlp = MLP(config)

    def forward(self, x, rope):
        x = x + self.self_attention(self.input_layernorm(x), rope)
        return x + self.mlp(self.post_attention_layernorm(x))


class _Encoder(torch.nn.Module):
    def __init__(self, config):
        super().__init__()
        self.layers = torch.nn.ModuleList([GLMBlock(config, i + 1) for i in range(config.num_layers)])
        self.final_layernorm = RMSNorm(config.hidden_size, config.layernorm_epsilon)


class _Transformer(torch.nn.Module):
    def __init__(self, config):
        super().__init__()
        self.embedding = torch.nn.Embedding(config.padded_vocab_size, config.hidden_size)
        self.encoder = _Encoder(config)
        self.output_layer = torch.nn.Linear(config.hidden_size, config.padded_vocab_size, bias=False)


class ChatGLM2ShapedDecoder(torch.nn.Module):
    """Random-init decoder of the ChatGLM2-6B shape; ``forward(input_ids [b, sq]) -> logits [b, sq, vocab]`` (prefill)."""

    def __init__(self, config=None, seed=0, last_token_logits_only=False, device=None, dtype=None):
        super().__init__()
        self.config = config or chatglm2_config()
        with torch.device(device or 'cpu'):
            self.transformer = _Transformer(self.config)
        if dtype is not None:
            self.to(dtype=dtype)
        self.last_only = last_token_logits_only
        dev = next(self.parameters()).device
        g = torch.Generator(device=dev).manual_seed(seed)
        with torch.no_grad():
            for name, prm in self.named_parameters():
                if prm.dim() >= 2:
                    prm.copy_(torch.randn(prm.shape, generator=g, device=dev, dtype=torch.float32) * 0.02)
                elif name.endswith('bias'):
                    prm.zero_()

    def forward(self, input_ids):
        b, sq = input_ids.shape
        x = self.transformer.embedding(input_ids).transpose(0, 1).contiguous()      # [sq, b, hidden]
        rope = _rope_cache(sq, self.config.kv_channels // 2, self.config.rope_ratio, x.device, x.dtype)
        for layer in self.transformer.encoder.layers:
            x = layer(x, rope)
        x = self.transformer.encoder.final_layernorm(x)
        if self.last_only:
            x = x[-1:]
        return self.transformer.output_layer(x).transpose(0, 1)
