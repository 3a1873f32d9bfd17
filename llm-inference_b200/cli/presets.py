"""Named model shapes (config.json contents) for random-weight models."""

from __future__ import annotations


def _qwen2(layers, hidden, heads, kv_heads, inter, vocab, tied, max_pos=32768, **extra):
    config = {
        "architectures": ["Qwen2ForCausalLM"],
        "model_type": "qwen2",
        "num_hidden_layers": layers,
        "hidden_size": hidden,
        "num_attention_heads": heads,
        "num_key_value_heads": kv_heads,
        "intermediate_size": inter,
        "vocab_size": vocab,
        "rope_theta": 1000000.0,
        "rms_norm_eps": 1e-6,
        "tie_word_embeddings": tied,
        "use_sliding_window": False,
        "max_position_embeddings": max_pos,
        "eos_token_id": 2,
    }
    config.update(extra)
    return config


PRESETS = {
    "tiny-a": _qwen2(2, 64, 4, 2, 176, 256, True, 128, rope_theta=10000.0),
    "tiny-b": _qwen2(3, 96, 3, 1, 272, 311, False, 256, rms_norm_eps=1e-5, use_sliding_window=True,
                     sliding_window=24, max_window_layers=1),
    "qwen2.5-1.5b": _qwen2(28, 1536, 12, 2, 8960, 151936, True, eos_token_id=151643),
    "qwen2.5-7b": _qwen2(28, 3584, 28, 4, 18944, 152064, False, eos_token_id=151643),
    "qwen2.5-14b": _qwen2(48, 5120, 40, 8, 13824, 152064, False, eos_token_id=151643),
}
