"""The two ends of a model: token ids to the residual stream, and normalised rows to logits."""

from __future__ import annotations

import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import gemm
from paged_kv_serving_b200.parts.base import ParamSpec, Part, StepContext

__all__ = ["LinearHead", "TokenEmbedding"]


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    """``hidden = table[ids]`` widened to float32
    (reference: src/paged_kv_serving/engine/model.py:266-267). ``forward(ctx)`` reads the step's
    token ids from ``ctx`` (and, for a token that was sampled on the device by the step before,
    from ``ctx.fed_back_ids``). An architecture whose embeddings are scaled, summed with others
    or looked up otherwise gives its layout another part with the same ``forward``."""

    graph_safe = True

    def __init__(self, vocab_size: int, width: int) -> None:
        self.vocab_size = int(vocab_size)
        self.width = int(width)
        self.table: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        return {"table": ParamSpec((self.vocab_size, self.width))}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        self.table = params["table"].contiguous()

    def forward(self, ctx: StepContext) -> torch.Tensor:
        fed_back_at = ctx.ints(ctx.TOKEN_FEEDBACK) if ctx.fed_back_ids is not None else None
        return ops.embedding_gather(self.table, ctx.ints(ctx.TOKEN_IDS), ctx.status, ctx.fed_back_ids, fed_back_at)


@register_part("head", "linear")
class LinearHead(Part):
    """``logits = normed @ weight^T`` in float32, ``weight [vocab, width]``; with ``tied`` the
    weight is that embedding part's table (reference: src/paged_kv_serving/engine/model.py:261-264,
    where the head is always tied). ``forward(normed, ctx)`` gets the rows the final norm left
    (only the wanted ones). A head with a scale, a soft cap or several outputs is another part
    with the same ``forward``."""

    graph_safe = True

    def __init__(self, vocab_size: int, width: int, tied: TokenEmbedding | None = None) -> None:
        self.vocab_size = int(vocab_size)
        self.width = int(width)
        self.tied = tied
        self._weight: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        return {} if self.tied is not None else {"weight": ParamSpec((self.vocab_size, self.width))}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        if "weight" in params:
            self._weight = params["weight"].contiguous()

    @property
    def weight(self) -> torch.Tensor:
        return self.tied.table if self.tied is not None else self._weight

    def forward(self, normed: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return gemm.linear(normed, self.weight, out_dtype=torch.float32, chain=True)
