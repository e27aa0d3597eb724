"""Named configurations (the contents of a ``config.json``) for the random-weights mode,
benchmarks and demos. They are data: nothing in the model code depends on them."""

from __future__ import annotations

from paged_kv_serving_b200.config.model_config import ModelConfig

__all__ = ["PRESETS", "preset"]

PRESETS: dict[str, dict] = {
    # the reference's default random checkpoint (src/paged_kv_serving/engine/weights.py:209-239)
    "reference-default": dict(vocab_size=512, d_model=128, n_layers=4, n_heads=4, d_ff=320, max_seq_len=1024),
    "tiny-a": dict(vocab_size=256, d_model=64, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=172,
                   max_seq_len=128, rope_theta=10000.0, norm_eps=1e-5, tie_embeddings=False),
    "tiny-b": dict(vocab_size=384, d_model=96, n_layers=3, n_heads=3, n_kv_heads=3, head_dim=32, d_ff=256,
                   max_seq_len=256, rope_theta=500000.0, norm_eps=1e-6, tie_embeddings=True),
    "llama-3-8b": dict(vocab_size=128256, d_model=4096, n_layers=32, n_heads=32, n_kv_heads=8, head_dim=128,
                       d_ff=14336, max_seq_len=8192, rope_theta=500000.0, norm_eps=1e-5, tie_embeddings=False),
    "llama-2-13b": dict(vocab_size=32000, d_model=5120, n_layers=40, n_heads=40, n_kv_heads=40, head_dim=128,
                        d_ff=13824, max_seq_len=4096, rope_theta=10000.0, norm_eps=1e-5, tie_embeddings=False),
    "llama-3.2-1b": dict(vocab_size=128256, d_model=2048, n_layers=16, n_heads=32, n_kv_heads=8, head_dim=64,
                         d_ff=8192, max_seq_len=8192, rope_theta=500000.0, norm_eps=1e-5, tie_embeddings=True),
}


def preset(name: str, **overrides) -> ModelConfig:
    try:
        data = dict(PRESETS[name])
    except KeyError:
        raise ValueError(f"unknown preset {name!r}; known: {', '.join(sorted(PRESETS))}") from None
    data.update(overrides)
    return ModelConfig.from_dict(data)
