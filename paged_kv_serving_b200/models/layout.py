"""What an architecture module hands to the framework: parts, layer order, tensor names."""

from __future__ import annotations

from dataclasses import dataclass, field

from paged_kv_serving_b200.parts.base import ParamSpec, Part

__all__ = ["LayerCall", "ModelLayout", "collect_param_specs"]


@dataclass(frozen=True, slots=True)
class LayerCall:
    """One entry of the run order. ``layer`` indexes ``ModelLayout.blocks``; the same layer may
    be named by several calls. ``cache`` is the number of the cache entry the call's mixer uses:
    by default a fresh one per call; a call that names an earlier call's entry with
    ``write=False`` reads that layer's keys and values without writing its own."""

    layer: int
    cache: int | None = None
    write: bool = True


@dataclass(slots=True)
class ModelLayout:
    """A model as data.

    ``names`` maps each tensor name of the model folder to ``(part, local name)``; the embedding
    table and an untied head are named separately because the framework itself applies them.
    """

    width: int
    vocab_size: int
    max_positions: int
    blocks: list[Part]
    order: list[LayerCall]
    final_norm: Part
    names: dict[str, tuple[Part, str]]
    embedding_name: str = "token_embedding"
    head_name: str | None = None          # None: the head is the embedding table (tied)
    notes: dict[str, str] = field(default_factory=dict)
    #: The part that turns the step's token ids into the residual stream (``forward(ctx)``) and
    #: the part that turns the final norm's rows into float32 logits (``forward(normed, ctx)``).
    #: Left ``None`` they are a plain table lookup named ``embedding_name`` and a linear head
    #: named ``head_name`` (tied to the table when that is ``None``). An architecture with
    #: another kind of embedding or head passes its own parts and names their tensors in ``names``.
    embedding: Part | None = None
    head: Part | None = None

    def __post_init__(self) -> None:
        from paged_kv_serving_b200.parts.io import LinearHead, TokenEmbedding

        if self.embedding is None:
            self.embedding = TokenEmbedding(self.vocab_size, self.width)
            self.names[self.embedding_name] = (self.embedding, "table")
        if self.head is None:
            tied = self.embedding if self.head_name is None and isinstance(self.embedding, TokenEmbedding) else None
            if self.head_name is None and tied is None:
                raise ValueError("a head tied to the embedding needs the plain embedding part, or a head of its own")
            self.head = LinearHead(self.vocab_size, self.width, tied=tied)
            if self.head_name is not None:
                self.names[self.head_name] = (self.head, "weight")

    def tensor_specs(self) -> dict[str, ParamSpec]:
        return {name: part.param_specs()[local] for name, (part, local) in self.names.items()}

    def parameter_count(self) -> int:
        """Number of parameters in the tensors of a model folder (a tied head counts once)."""
        total = 0
        for spec in self.tensor_specs().values():
            count = 1
            for size in spec.shape:
                count *= int(size)
            total += count
        return total

    def cache_entries(self) -> list[tuple[int, object]]:
        """``(entry number, request)`` of every distinct cache entry of the run order."""
        seen: dict[int, object] = {}
        next_free = 0
        for call in self.resolved_order():
            request = self.blocks[call.layer].cache_request()
            if request is None or call.cache is None:
                continue
            if call.cache in seen:
                if seen[call.cache] != request:
                    raise ValueError(f"layer calls sharing cache entry {call.cache} ask for different storage")
            else:
                seen[call.cache] = request
            next_free = max(next_free, call.cache + 1)
        return sorted(seen.items())

    def resolved_order(self) -> list[LayerCall]:
        """The run order with a cache entry number on every call whose mixer wants a cache."""
        explicit = [c.cache for c in self.order if c.cache is not None]
        next_free = max(explicit) + 1 if explicit else 0
        out = []
        for call in self.order:
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"layer call names layer {call.layer}, the model has {len(self.blocks)}")
            if call.cache is None and self.blocks[call.layer].cache_request() is not None:
                out.append(LayerCall(call.layer, next_free, call.write))
                next_free += 1
            else:
                out.append(call)
        return out


def collect_param_specs(prefix: str, part: Part, into: dict[str, tuple[Part, str]]) -> None:
    """Register ``prefix + local`` for every tensor of ``part`` and of its children
    (children's names are prefixed with ``child.``)."""
    for local in part.param_specs():
        into[prefix + local] = (part, local)
    for child_name, child in part.sub_parts().items():
        collect_param_specs(f"{prefix}{child_name}.", child, into)
