"""ChatGLM2-style integration: layer selection, the module nesting the patch relies on, and (GPU) that a patched model
equals the exact one when every causal call is short enough to run as an exact leaf."""
import pytest
import torch

from hyperattention_b200.llm import (ChatGLM2ShapedDecoder, ExactCoreAttention, FastCoreAttention, chatglm2_config,
                                     patch_attention_layers, select_patch_layers)


def test_layer_selection_matches_reference_rules():
    # replace_llm_attention.py:10-35 evaluated by hand for 28 layers
    assert select_patch_layers(28, 'last', 14) == list(range(27, 13, -1))
    assert select_patch_layers(28, 'first', 3) == [0, 1, 2]
    assert select_patch_layers(28, 'odd', 5) == list(range(1, 28, 2))
    assert select_patch_layers(28, 'even', 5) == list(range(0, 28, 2))
    assert select_patch_layers(28, 'odd_first', 3) == [1, 3, 5]
    assert select_patch_layers(28, 'odd_last', 3) == [27, 26]
    assert select_patch_layers(28, 'even_first', 3) == [0, 2, 4]
    assert select_patch_layers(28, 'even_last', 3) == [23, 25, 27]
    assert select_patch_layers(28, 'last', -1) == list(range(27, -1, -1))
    with pytest.raises(NotImplementedError):
        select_patch_layers(28, 'middle', 3)


def _small(device='cpu', dtype=torch.float32):
    cfg = chatglm2_config(num_layers=4, hidden_size=256, num_attention_heads=2, ffn_hidden_size=512, padded_vocab_size=1000)
    return ChatGLM2ShapedDecoder(cfg, seed=1, device=device, dtype=dtype).eval()


def test_decoder_structure_and_cpu_forward():
    m = _small()
    assert isinstance(m.transformer.encoder.layers[3].self_attention.core_attention, ExactCoreAttention)
    ids = torch.randint(0, 1000, (2, 64))
    with torch.no_grad():
        logits = m(ids)
    assert logits.shape == (2, 64, 1000) and torch.isfinite(logits).all()
    # causal: logits at position t do not depend on later tokens
    ids2 = ids.clone()
    ids2[:, 40:] = torch.randint(0, 1000, (2, 24))
    with torch.no_grad():
        assert torch.allclose(m(ids2)[:, :40], logits[:, :40], atol=1e-5)
    c = chatglm2_config()
    assert (c.num_layers, c.hidden_size, c.num_attention_heads, c.kv_channels, c.multi_query_group_num, c.ffn_hidden_size,
            c.padded_vocab_size) == (28, 4096, 32, 128, 2, 13696, 65024)


@pytest.mark.gpu
def test_patched_model_on_gpu():
    m = _small('cuda', torch.bfloat16)
    ids = torch.randint(0, 1000, (1, 1024), device='cuda')
    with torch.no_grad():
        exact = m(ids)
    idx = patch_attention_layers(m, 'chatglm2-6b-32k', 'last', 2, num_total_layers=4, attn_method='hyper', lsh_num_projs=8,
                                 block_size=256, sample_size=256, min_seq_len=2048, smooth_block=False)
    assert idx == [3, 2] and isinstance(m.transformer.encoder.layers[3].self_attention.core_attention, FastCoreAttention)
    assert isinstance(m.transformer.encoder.layers[1].self_attention.core_attention, ExactCoreAttention)
    with torch.no_grad():
        same = m(ids)          # 1024 <= min_seq_len: every patched call is one exact causal leaf
    rel = ((same.float() - exact.float()).norm() / exact.float().norm()).item()
    assert rel < 2e-2
    # longer than min_seq_len: the approximate path runs (two half-splits), output stays close and finite
    for layer in (2, 3):
        m.transformer.encoder.layers[layer].self_attention.core_attention.attn.min_seq_len = 256
    with torch.no_grad():
        approx = m(ids)
    assert torch.isfinite(approx).all()
    rel2 = ((approx.float() - exact.float()).norm() / exact.float().norm()).item()
    assert rel2 < 0.5
    with pytest.raises(AssertionError):
        m.transformer.encoder.layers[3].self_attention.core_attention(torch.zeros(4, 1, 2, 128, device='cuda'),
                                                                      torch.zeros(8, 1, 2, 128, device='cuda'),
                                                                      torch.zeros(8, 1, 2, 128, device='cuda'), None)
