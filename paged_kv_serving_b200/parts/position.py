"""Position-encoding parts."""

from __future__ import annotations

import numpy as np
import torch

from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.parts.base import Part

__all__ = ["NoPositionEncoding", "PositionEncoding", "RotaryEncoding"]


class PositionEncoding(Part):
    """Interface of a position encoding used by an attention mixer.

    ``fused_tables`` returns ``(cos, sin)`` float32 tables ``[positions, rotated/2]`` when the
    encoding is a half-split rotation of queries and keys that the attention kernels apply
    themselves; an encoding of another kind returns ``None`` and implements ``apply_qk``, which
    rewrites the query and key columns of the fused ``qkv`` buffer in place before the keys are
    stored. Keys are cached after encoding, so an encoding must depend on a key's own absolute
    position only.
    """

    graph_safe = True

    def fused_tables(self, device: torch.device) -> tuple[torch.Tensor, torch.Tensor] | None:
        return None

    def apply_qk(self, qkv: torch.Tensor, positions: torch.Tensor, n_heads: int, n_kv: int, head_dim: int) -> None:
        return None


@register_part("position", "none")
class NoPositionEncoding(PositionEncoding):
    """Leaves queries and keys as they are."""


@register_part("position", "rotary")
class RotaryEncoding(PositionEncoding):
    """Rotary encoding, half-split form: ``inv_freq_j = theta^(-2j/hd)``, ``angle = p * inv_freq_j``
    computed in float64 and cast to float32 tables, as the reference does
    (src/paged_kv_serving/engine/model.py:60-81)."""

    def __init__(self, head_dim: int, theta: float, max_positions: int) -> None:
        if head_dim % 2:
            raise ValueError("head_dim must be even for rotary position encoding")
        if not theta > 1.0:
            raise ValueError("rope theta must be > 1")
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self._tables: dict[str, tuple[torch.Tensor, torch.Tensor]] = {}

    def host_tables(self) -> tuple[np.ndarray, np.ndarray]:
        half = self.head_dim // 2
        inv_freq = 1.0 / (self.theta ** (np.arange(half, dtype=np.float64) * 2.0 / self.head_dim))
        angles = np.outer(np.arange(self.max_positions, dtype=np.float64), inv_freq)
        return np.cos(angles).astype(np.float32), np.sin(angles).astype(np.float32)

    def fused_tables(self, device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
        key = str(device)
        if key not in self._tables:
            cos, sin = self.host_tables()
            self._tables[key] = (torch.from_numpy(cos).to(device), torch.from_numpy(sin).to(device))
        return self._tables[key]
