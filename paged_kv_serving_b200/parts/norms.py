"""Normalisation parts."""

from __future__ import annotations

import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.ops import gemm
from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.parts.base import ParamSpec, Part

__all__ = ["RMSNorm"]


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """``y = (x / sqrt(mean(x^2) + eps)) * weight`` in float32
    (reference: src/paged_kv_serving/engine/model.py:43-46), fused with the residual add in
    front of it: the stream ``hidden`` (float32) first takes the pending ``delta``."""

    graph_safe = True


    def __init__(self, width: int, eps: float) -> None:
        self.width = int(width)
        self.eps = float(eps)
        self.weight: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.width,), "vector")}

    def add_norm(self, hidden: torch.Tensor, delta: torch.Tensor | None, out_dtype: torch.dtype,
                 rows: torch.Tensor | None = None) -> torch.Tensor:
        """``hidden += delta`` in place, then the normalised rows (all, or only ``rows``; with
        ``rows`` the stream itself is not updated)."""
        return ops.add_rmsnorm(hidden, delta, self.weight, self.eps, out_dtype, rows)

    def add_norm_of_linear(self, hidden: torch.Tensor, x: torch.Tensor, w_nk: torch.Tensor,
                           out_dtype: torch.dtype, chain: bool = False) -> torch.Tensor:
        """``add_norm(hidden, x @ w_nk^T)`` for a producer whose last step is that product: the
        product's kernel carries the residual add, and the norm is left to the product that reads
        the result, where the kernels can do that. ``chain`` as in ``ops.gemm.linear``."""
        return gemm.linear_add_norm(x, w_nk, hidden, self.weight, self.eps, out_dtype, chain=chain)
