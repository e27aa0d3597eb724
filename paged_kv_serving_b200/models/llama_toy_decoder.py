"""The Llama-style toy decoder of the reference (src/paged_kv_serving/engine/model.py):
pre-norm RMSNorm, rotary position encoding, causal attention, SwiGLU feed-forward, a head tied
to the embedding; generalised to grouped-query heads and an optional separate head.

This module is all that is specific to the architecture: which parts a layer has, with which
constants of the configuration, in which order the layers run, and the tensor names of a
model folder (the reference's, src/paged_kv_serving/engine/model.py:84-92,130-139).
"""

from __future__ import annotations

from paged_kv_serving_b200.config.model_config import ModelConfig
from paged_kv_serving_b200.config.registry import register_architecture
from paged_kv_serving_b200.models.layout import LayerCall, ModelLayout
from paged_kv_serving_b200.parts import PagedAttention, PreNormBlock, RMSNorm, RotaryEncoding, SwiGLU

__all__ = ["LlamaToyDecoder"]

# The reference clips the argument of the sigmoid's exponential to this range
# (src/paged_kv_serving/engine/model.py:49-51); it is a constant of the architecture, not of a
# model folder.
SILU_CLIP = 60.0


@register_architecture("LlamaToyDecoder")
class LlamaToyDecoder:
    """Builds the layout of the toy decoder from a configuration."""

    @staticmethod
    def layout(config: ModelConfig) -> ModelLayout:
        rotary = RotaryEncoding(config.head_dim, config.rope_theta, config.max_seq_len)
        blocks = []
        names = {}
        for index in range(config.n_layers):
            attn_norm = RMSNorm(config.d_model, config.norm_eps)
            mixer = PagedAttention(config.d_model, config.n_heads, config.n_kv_heads, config.head_dim, rotary)
            ffn_norm = RMSNorm(config.d_model, config.norm_eps)
            feed_forward = SwiGLU(config.d_model, config.d_ff, SILU_CLIP)
            blocks.append(PreNormBlock(attn_norm, mixer, ffn_norm, feed_forward))
            prefix = f"layers.{index}."
            names[prefix + "attn_norm"] = (attn_norm, "weight")
            names[prefix + "qkv_proj"] = (mixer, "qkv_proj")
            names[prefix + "out_proj"] = (mixer, "out_proj")
            names[prefix + "ffn_norm"] = (ffn_norm, "weight")
            names[prefix + "gate_proj"] = (feed_forward, "gate_proj")
            names[prefix + "up_proj"] = (feed_forward, "up_proj")
            names[prefix + "down_proj"] = (feed_forward, "down_proj")
        final_norm = RMSNorm(config.d_model, config.norm_eps)
        names["final_norm"] = (final_norm, "weight")
        return ModelLayout(
            width=config.d_model,
            vocab_size=config.vocab_size,
            max_positions=config.max_seq_len,
            blocks=blocks,
            order=[LayerCall(index) for index in range(config.n_layers)],
            final_norm=final_norm,
            names=names,
            embedding_name="token_embedding",
            head_name=None if config.tie_embeddings else "lm_head",
        )
