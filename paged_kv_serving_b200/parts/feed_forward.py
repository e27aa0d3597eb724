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

    Weights are re-laid at load as ``[out, in]``. Gate and up become one matrix so that a single
    product feeds the ``silu * up`` step: in bfloat16 their rows are interleaved in blocks of
    128 (padded with zero rows to a multiple of 128), which lets the tensor-core kernel apply the
    step in its epilogue; in float32 they are simply stacked.
    """

    graph_safe = True
    BLOCK = 128

    def __init__(self, width: int, inner: int, clip: float = 60.0) -> None:
        self.width = int(width)
        self.inner = int(inner)
        self.clip = float(clip)
        self.gate_up: torch.Tensor | None = None    # [2 * inner (padded), width]
        self.down_proj: torch.Tensor | None = None  # [width, inner]
        self.interleave = 0

    def param_specs(self) -> dict[str, ParamSpec]:
        return {
            "gate_proj": ParamSpec((self.width, self.inner)),
            "up_proj": ParamSpec((self.width, self.inner)),
            "down_proj": ParamSpec((self.inner, self.width)),
        }

    def load(self, params: dict[str, torch.Tensor]) -> None:
        gate, up = params["gate_proj"].t(), params["up_proj"].t()          # [inner, width]
        if gate.dtype == torch.bfloat16:
            block = self.BLOCK
            blocks = -(-self.inner // block)
            fused = torch.zeros((blocks, 2, block, self.width), dtype=gate.dtype, device=gate.device)
            flat = fused.view(blocks, 2, block * self.width)
            padded = torch.zeros((2, blocks * block, self.width), dtype=gate.dtype, device=gate.device)
            padded[0, :self.inner] = gate
            padded[1, :self.inner] = up
            flat[:, 0] = padded[0].view(blocks, block * self.width)
            flat[:, 1] = padded[1].view(blocks, block * self.width)
            self.gate_up = fused.view(2 * blocks * block, self.width)
            self.interleave = block
        else:
            self.gate_up = torch.cat([gate, up], dim=0).contiguous()
            self.interleave = 0
        self.down_proj = params["down_proj"].t().contiguous()

    fuses_last_linear = True
    accepts_pending_norm = True

    def forward(self, x: torch.Tensor, ctx: StepContext, finish=None) -> torch.Tensor:
        gated = gemm.linear_silu_mul(x, self.gate_up, self.inner, self.interleave, self.clip, chain=True)
        if finish is not None:
            return finish(gated, self.down_proj)
        return gemm.linear(gated, self.down_proj, chain=True)
