"""Arrangement of the parts of one layer."""

from __future__ import annotations

import torch

from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import gemm
from paged_kv_serving_b200.parts.base import Block, CacheBinding, Normed, Part, StepContext

__all__ = ["PreNormBlock"]


@register_part("block", "prenorm_residual")
class PreNormBlock(Block):
    """Pre-norm residual arrangement: ``h += mixer(norm(h)); h += feed_forward(norm(h))``
    (reference: src/paged_kv_serving/engine/model.py:283-287, src/paged_kv_serving/engine/runner.py:213-214).

    The hand-over between blocks (pending updates, ``Normed``) is the one ``parts.base.Block``
    describes: a block receives the previous block's output as a pending update and returns its
    own feed-forward output as the next one, or the stream already normalised for the next block.
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
        # only the children that plan anything (this runs for every layer of every step)
        planners = self.__dict__.get("_planners")
        if planners is None:
            planners = self._planners = [child for child in self.sub_parts().values()
                                         if type(child).plan_step is not Part.plan_step]
        for child in planners:
            child.plan_step(ctx, binding)

    @property
    def first_norm(self) -> Part:
        """The norm this block applies to the stream it is given (with the pending update)."""
        return self.mixer_norm

    def forward(self, hidden: torch.Tensor, pending: "torch.Tensor | Normed | None", ctx: StepContext,
                binding: CacheBinding | None, next_norm: Part | None = None) -> "torch.Tensor | Normed":
        """One layer call. ``pending`` is what the block before handed on: its residual update not
        yet added (a tensor, or None at the start), or a ``Normed`` when it already added it and
        applied this block's first norm. ``next_norm`` is the first norm of the block that runs
        next; where the feed-forward can carry the residual add and that norm in the tail of its
        last product, this block hands on a ``Normed``, else its own pending update.
        """
        if isinstance(pending, Normed) and pending.norm is self.mixer_norm:
            normed = pending.values if self.mixer.accepts_pending_norm else gemm.as_tensor(pending.values)
        else:
            if isinstance(pending, Normed):
                raise ValueError("the stream was normalised for another block than the one that runs next")
            normed = self.mixer_norm.add_norm(hidden, pending, ctx.dtype)
        follow = getattr(self.ff_norm, "add_norm_of_linear", None)
        if self.mixer.fuses_last_linear and follow is not None:
            chain = self.mixer.chains_last_linear
            normed = self.mixer.forward(normed, ctx, binding,
                                        finish=lambda x, w: follow(hidden, x, w, ctx.dtype, chain=chain))
        else:
            normed = self.ff_norm.add_norm(hidden, self.mixer.forward(normed, ctx, binding), ctx.dtype)
        if not self.feed_forward.accepts_pending_norm:
            normed = gemm.as_tensor(normed)
        follow = getattr(next_norm, "add_norm_of_linear", None)
        if self.feed_forward.fuses_last_linear and follow is not None:
            chain = self.feed_forward.chains_last_linear
            values = self.feed_forward.forward(
                normed, ctx, finish=lambda x, w: follow(hidden, x, w, ctx.dtype, chain=chain))
            return Normed(values, next_norm)
        return self.feed_forward.forward(normed, ctx)
