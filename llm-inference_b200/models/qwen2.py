"""Qwen2 / Qwen2.5 dense decoder as a recipe of parts.

Per layer, in the reference's order (python/instinct/backends/dense.py:87-129):
RMSNorm -> q/k/v projections with bias -> rotary encoding of q and k -> cache write ->
causal grouped-query attention -> output projection without bias -> residual add ->
RMSNorm -> SwiGLU feed-forward -> residual add; then a last RMSNorm and the output head,
which shares the embedding table when ``tie_word_embeddings`` is set.
"""

from __future__ import annotations

from ..config.model_config import Qwen2Config
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from ..parts.model import ModelRecipe


def qwen2_recipe(config: Qwen2Config) -> ModelRecipe:
    layers = []
    for index in range(config.num_hidden_layers):
        prefix = f"model.layers.{index}."
        mixer = PartSpec(
            "gqa_attention",
            dict(
                prefix=prefix + "self_attn.",
                hidden_size=config.hidden_size,
                q_heads=config.num_attention_heads,
                kv_heads=config.num_key_value_heads,
                head_dim=config.head_dim,
                qkv_bias=True,
                window=config.layer_window(index),
                position=PartSpec("rotary", dict(head_dim=config.head_dim, theta=config.rope_theta)),
            ),
        )
        feed_forward = PartSpec(
            "swiglu",
            dict(prefix=prefix + "mlp.", hidden_size=config.hidden_size, intermediate_size=config.intermediate_size),
        )

        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", dict(name=prefix + name, hidden_size=config.hidden_size, eps=config.rms_norm_eps))

        layers.append(
            PartSpec(
                "pre_norm_residual",
                dict(
                    mixer=mixer,
                    feed_forward=feed_forward,
                    mixer_norm=norm("input_layernorm"),
                    feed_forward_norm=norm("post_attention_layernorm"),
                ),
            )
        )
    return ModelRecipe(
        config=config,
        embedding=PartSpec(
            "token_embedding",
            dict(name="model.embed_tokens", vocab_size=config.vocab_size, hidden_size=config.hidden_size),
        ),
        layers=layers,
        final_norm=PartSpec("rmsnorm", dict(name="model.norm", hidden_size=config.hidden_size, eps=config.rms_norm_eps)),
        head=PartSpec(
            "linear_head",
            dict(
                name="lm_head",
                vocab_size=config.vocab_size,
                hidden_size=config.hidden_size,
                tied_to="model.embed_tokens" if config.tie_word_embeddings else None,
            ),
        ),
    )


register_architecture(
    Qwen2Config.ARCHITECTURE, Qwen2Config.from_json_dict, qwen2_recipe, model_types=(Qwen2Config.MODEL_TYPE,)
)
