"""Prefill benchmark of the ChatGLM2-6B-shaped decoder (benchmark configuration 4): batch 1 x 32768 uniformly random token ids,
attention of the last 14 of 28 blocks replaced by HyperAttention; reports prefill tokens/s of the all-exact and the
patched model and the deviation of the last-position logits.

    python -m hyperattention_b200.llm_bench [--seq-len 32768] [--layers 28] [--patch-layers 14] [--steps 3]
"""
import argparse
import json

import torch

from .llm import ChatGLM2ShapedDecoder, chatglm2_config, patch_attention_layers


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--seq-len', type=int, default=32768)
    ap.add_argument('--layers', type=int, default=28)
    ap.add_argument('--patch-layers', type=int, default=14)
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--hidden', type=int, default=4096)
    ap.add_argument('--ffn', type=int, default=13696)
    ap.add_argument('--vocab', type=int, default=65024)
    a = ap.parse_args()
    assert torch.cuda.is_available()
    dev = torch.device('cuda')
    cfg = chatglm2_config(num_layers=a.layers, hidden_size=a.hidden, num_attention_heads=a.hidden // 128, ffn_hidden_size=a.ffn,
                          padded_vocab_size=a.vocab)
    model = ChatGLM2ShapedDecoder(cfg, seed=0, last_token_logits_only=True, device=dev, dtype=torch.bfloat16).eval()
    ids = torch.randint(0, a.vocab, (1, a.seq_len), generator=torch.Generator().manual_seed(4)).to(dev)

    def timed(fn):
        with torch.no_grad():
            out = fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.steps):
                out = fn()
            e1.record()
            e1.synchronize()
        return e0.elapsed_time(e1) / a.steps, out

    ms_exact, logits_exact = timed(lambda: model(ids))
    patch_attention_layers(model, 'chatglm2-6b-32k', 'last', a.patch_layers, num_total_layers=a.layers, attn_method='hyper',
                           lsh_num_projs=8, block_size=256, sample_size=256, min_seq_len=2048, smooth_block=False)
    ms_hyper, logits_hyper = timed(lambda: model(ids))
    # the same patched model with K/V handed over un-expanded (2 K/V groups instead of 32 expanded heads)
    for layer in model.transformer.encoder.layers:
        if hasattr(layer.self_attention.core_attention, 'grouped_kv'):
            layer.self_attention.core_attention.grouped_kv = True
    ms_grouped, logits_grouped = timed(lambda: model(ids))
    le, lh = logits_exact.float(), logits_hyper.float()
    dev_rel = ((lh - le).norm() / le.norm()).item()
    top1 = bool((le.argmax(-1) == lh.argmax(-1)).all())
    print(json.dumps({'workload': f'ChatGLM2-6B-shaped decoder, random init, {a.layers} blocks, hidden {a.hidden}, prefill 1 x {a.seq_len}',
                      'patched_blocks': a.patch_layers, 'exact_prefill_ms': ms_exact, 'hyper_prefill_ms': ms_hyper,
                      'exact_tokens_per_s': a.seq_len / ms_exact * 1e3, 'hyper_tokens_per_s': a.seq_len / ms_hyper * 1e3,
                      'speedup': ms_exact / ms_hyper, 'last_logits_rel_deviation': dev_rel, 'last_token_top1_same': top1,
                      'hyper_grouped_kv_prefill_ms': ms_grouped, 'speedup_grouped_kv': ms_exact / ms_grouped,
                      'grouped_vs_expanded_logits_rel_deviation': ((logits_grouped.float() - lh).norm() / lh.norm()).item()}))


if __name__ == '__main__':
    main()
