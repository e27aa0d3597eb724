"""Typed configuration of a model, read from the ``config.json`` of a model folder.

The keys are those of the reference's ``ModelConfig`` (its ``manifest.json["architecture"]``
dictionary: src/paged_kv_serving/engine/config.py:35-95 and
src/paged_kv_serving/engine/weights.py:90,113-114), plus what the reference fixes in code and
this engine makes data: the architecture's registry name, the number of key/value heads,
an explicit head size and whether the output head is tied to the embedding.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Any

__all__ = ["CONFIG_FILE", "ModelConfig"]

CONFIG_FILE = "config.json"


@dataclass(frozen=True, slots=True)
class ModelConfig:
    """Shape and constants of a decoder. Every value a part needs is a field here.

    ``n_kv_heads`` and ``head_dim`` default to the reference's fixed choices
    (``n_heads`` and ``d_model // n_heads``, src/paged_kv_serving/engine/config.py:64-66);
    ``tie_embeddings`` defaults to the reference's tied head
    (src/paged_kv_serving/engine/model.py:261-264).
    """

    vocab_size: int
    d_model: int
    n_layers: int
    n_heads: int
    d_ff: int
    max_seq_len: int
    rope_theta: float = 10_000.0
    norm_eps: float = 1e-5
    n_kv_heads: int | None = None
    head_dim: int | None = None
    tie_embeddings: bool = True
    architecture: str = "LlamaToyDecoder"

    def __post_init__(self) -> None:
        for name in ("vocab_size", "d_model", "n_layers", "n_heads", "d_ff", "max_seq_len"):
            value = getattr(self, name)
            if not isinstance(value, int) or isinstance(value, bool) or value < 1:
                raise ValueError(f"{name} must be an integer >= 1, found {value!r}")
        if self.n_kv_heads is None:
            object.__setattr__(self, "n_kv_heads", self.n_heads)
        if self.head_dim is None:
            if self.d_model % self.n_heads:
                raise ValueError("d_model must be divisible by n_heads when head_dim is not given")
            object.__setattr__(self, "head_dim", self.d_model // self.n_heads)
        for name in ("n_kv_heads", "head_dim"):
            value = getattr(self, name)
            if not isinstance(value, int) or isinstance(value, bool) or value < 1:
                raise ValueError(f"{name} must be an integer >= 1, found {value!r}")
        if self.n_heads % self.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if self.head_dim % 2:
            raise ValueError("head_dim must be even for rotary position encoding")
        if not float(self.rope_theta) > 1.0:
            raise ValueError("rope_theta must be > 1")
        if not float(self.norm_eps) > 0.0:
            raise ValueError("norm_eps must be > 0")
        if not isinstance(self.tie_embeddings, bool):
            raise ValueError("tie_embeddings must be true or false")
        if not isinstance(self.architecture, str) or not self.architecture:
            raise ValueError("architecture must be a non-empty string")
        object.__setattr__(self, "rope_theta", float(self.rope_theta))
        object.__setattr__(self, "norm_eps", float(self.norm_eps))

    # --- derived sizes -------------------------------------------------------------------

    @property
    def q_width(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def parameter_count(self) -> int:
        """Number of parameters, a tied head counted once
        (reference: src/paged_kv_serving/engine/config.py:68-75, widened for grouped heads)."""
        d = self.d_model
        attention = d * (self.q_width + 2 * self.kv_width) + self.q_width * d
        feed_forward = 3 * d * self.d_ff
        embedding = self.vocab_size * d * (1 if self.tie_embeddings else 2)
        return embedding + self.n_layers * (attention + feed_forward + 2 * d) + d

    # --- (de)serialisation ---------------------------------------------------------------

    def to_dict(self) -> dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in fields(self)}

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "ModelConfig":
        known = {f.name for f in fields(cls)}
        unknown = sorted(set(data) - known)
        if unknown:
            raise ValueError(f"unknown model config fields: {', '.join(unknown)}")
        required = [
            f.name for f in fields(cls)
            if f.name in ("vocab_size", "d_model", "n_layers", "n_heads", "d_ff", "max_seq_len")
        ]
        missing = [name for name in required if name not in data]
        if missing:
            raise ValueError(f"missing model config fields: {', '.join(missing)}")
        return cls(**data)

    @classmethod
    def from_json_file(cls, path: str | Path) -> "ModelConfig":
        path = Path(path)
        if path.is_dir():
            path = path / CONFIG_FILE
        with open(path, encoding="utf-8") as handle:
            data = json.load(handle)
        if not isinstance(data, dict):
            raise ValueError(f"{path}: a model configuration must be a JSON object")
        return cls.from_dict(data)

    def write_json(self, path: str | Path) -> None:
        path = Path(path)
        if path.is_dir():
            path = path / CONFIG_FILE
        path.write_text(json.dumps(self.to_dict(), indent=2, sort_keys=True) + "\n", encoding="utf-8")
