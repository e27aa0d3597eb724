"""Arrangement of the parts of one layer."""

from __future__ import annotations

import torch

from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.parts.base import CacheBinding, Part, StepContext

__all__ = ["PreNormBlock"]


@register_part("block", "prenorm_residual")
class PreNormBlock(Part):
    """Pre-norm residual arrangement: ``h += mixer(norm(h)); h += feed_forward(norm(h))``
    (reference: src/paged_kv_serving/engine/model.py:283-287, src/paged_kv_serving/engine/runner.py:213-214).

    The residual stream ``hidden`` is float32 and is updated in place. Each residual add is
    fused with the norm that follows it: a block receives the previous block's output as a
    pending ``delta`` and returns its own feed-forward output as the next pending delta.
    """

    @property
    def graph_safe(self) -> bool:
        return all(child.graph_safe for child in self.sub_parts().values())


    def __init__(self, mixer_norm: Part, mixer: Part, ff_norm: Part, feed_forward: Part) -> None:
        self.mixer_norm = mixer_norm
        self.mixer = mixer
        self.ff_norm = ff_norm
        self.feed_forward = feed_forward

    def sub_parts(self) -> dict[str, Part]:
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ff_norm": self.ff_norm,
                "feed_forward": self.feed_forward}

    def cache_request(self):
        return self.mixer.cache_request()

    def plan_step(self, ctx: StepContext, binding: CacheBinding | None) -> None:
        for child in self.sub_parts().values():
            child.plan_step(ctx, binding)

    def forward(self, hidden: torch.Tensor, delta: torch.Tensor | None, ctx: StepContext,
                binding: CacheBinding | None) -> torch.Tensor:
        normed = self.mixer_norm.add_norm(hidden, delta, ctx.dtype)
        mixed = self.mixer.forward(normed, ctx, binding)
        normed = self.ff_norm.add_norm(hidden, mixed, ctx.dtype)
        return self.feed_forward.forward(normed, ctx)
