"""Feed-forward parts."""

from __future__ import annotations

import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import gemm
from paged_kv_serving_b200.parts.base import ParamSpec, Part, StepContext

__all__ = ["SwiGLU"]


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """Dense gated feed-forward: ``(silu(x @ gate) * (x @ up)) @ down`` without biases, the
    argument of the sigmoid's exponential clipped to ``[-clip, clip]``
    (reference: src/paged_kv_serving/engine/model.py:49-51, 256-259).

    The gate and up matrices are concatenated at load so that one matrix product feeds the
    fused ``silu * up`` kernel.
    """

    graph_safe = True


    def __init__(self, width: int, inner: int, clip: float = 60.0) -> None:
        self.width = int(width)
        self.inner = int(inner)
        self.clip = float(clip)
        self.gate_up: torch.Tensor | None = None   # [width, 2 * inner]
        self.down_proj: torch.Tensor | None = None  # [inner, width]

    def param_specs(self) -> dict[str, ParamSpec]:
        return {
            "gate_proj": ParamSpec((self.width, self.inner)),
            "up_proj": ParamSpec((self.width, self.inner)),
            "down_proj": ParamSpec((self.inner, self.width)),
        }

    def load(self, params: dict[str, torch.Tensor]) -> None:
        self.gate_up = torch.cat([params["gate_proj"], params["up_proj"]], dim=1).contiguous()
        self.down_proj = params["down_proj"].contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        gate_up = gemm.matmul(x, self.gate_up)
        return gemm.matmul(ops.silu_mul(gate_up, self.clip), self.down_proj)
