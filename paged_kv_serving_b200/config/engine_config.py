"""Scheduling and memory limits of one engine instance.

Field names and meanings follow the reference's ``EngineConfig``
(src/paged_kv_serving/engine/config.py:98-160). The knobs of its deadline admission control
are left out with that subsystem; ``dtype`` and ``max_prefill_chunk`` are this engine's.
"""

from __future__ import annotations

from dataclasses import dataclass

__all__ = ["DTYPES", "EngineConfig"]

DTYPES = ("bfloat16", "float32")


@dataclass(frozen=True, slots=True)
class EngineConfig:
    """Limits for one engine.

    ``max_batched_tokens`` is the token budget of one step, shared by decoding sequences (one
    token each, taken first) and portions of prompts. ``num_blocks`` pages of ``block_size``
    tokens are given to every layer group of the cache. ``watermark`` is the fraction of pages
    kept free when a new prompt is admitted while others run. ``max_prefill_chunk`` (0 = off)
    caps one sequence's portion in a step.
    """

    block_size: int = 16
    num_blocks: int = 512
    max_batched_tokens: int = 256
    max_running_seqs: int = 32
    max_prompt_tokens: int = 512
    max_new_tokens: int = 128
    max_context_tokens: int = 1024
    enable_prefix_cache: bool = True
    watermark: float = 0.02
    lower_class_prefill_share: float = 1.0
    max_prefill_chunk: int = 0
    dtype: str = "bfloat16"

    def __post_init__(self) -> None:
        for name in ("block_size", "num_blocks", "max_batched_tokens", "max_running_seqs",
                     "max_prompt_tokens", "max_new_tokens"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be >= 1")
        if self.max_context_tokens < self.max_prompt_tokens + self.max_new_tokens:
            raise ValueError("max_context_tokens must cover max_prompt_tokens + max_new_tokens")
        if not 0.0 <= self.watermark < 1.0:
            raise ValueError("watermark must be in [0, 1)")
        if not 0.0 < self.lower_class_prefill_share <= 1.0:
            raise ValueError("lower_class_prefill_share must be in (0, 1]")
        if self.max_prefill_chunk < 0:
            raise ValueError("max_prefill_chunk must be >= 0")
        if self.num_blocks * self.block_size < self.max_context_tokens:
            raise ValueError("the KV cache cannot hold a single max-length sequence")
        if self.dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {', '.join(DTYPES)}")

    @property
    def cache_capacity_tokens(self) -> int:
        return self.num_blocks * self.block_size

    @property
    def lower_class_prefill_tokens(self) -> int:
        """Prefill tokens a step leaves to classes below the highest one that has work."""
        return max(1, int(self.max_batched_tokens * self.lower_class_prefill_share))
