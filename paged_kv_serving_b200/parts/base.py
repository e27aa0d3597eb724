"""What every part of a layer has in common, and what a step hands to the parts.

A part (norm, position encoding, mixer, feed-forward, block) is built from explicit sizes and
constants, declares the tensors it needs (``param_specs``), receives them once (``load``) and
then transforms activations step by step. A part never looks at a model configuration and never
knows which model it is in. A mixer may ask the cache manager for paged key/value storage
(``PagedKVRequest``) or for a fixed-size state per running request (``StateRequest``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch

__all__ = [
    "Block", "CacheBinding", "GroupView", "IntArena", "Normed", "PagedKVRequest", "ParamSpec", "Part", "StateRequest",
    "StepContext",
]


@dataclass(frozen=True, slots=True)
class ParamSpec:
    """Shape and role of one tensor. ``matrix``: an operand of a matrix product, held in the
    engine's compute type; ``vector``: an element-wise parameter, held in float32;
    ``int_table``: an integer table, held in int32."""

    shape: tuple[int, ...]
    kind: str = "matrix"

    def __post_init__(self) -> None:
        if self.kind not in ("matrix", "vector", "int_table"):
            raise ValueError(f"unknown parameter kind {self.kind!r}")


@dataclass(frozen=True, slots=True)
class PagedKVRequest:
    """Paged keys and values for one layer call: ``window=None`` keeps every key, a number keeps
    only the last ``window`` positions (older pages are given back)."""

    n_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True, slots=True)
class StateRequest:
    """A fixed-size state per running request, e.g. ``shape=(heads, dim)``; zeroed when a request
    (re)starts from position zero."""

    shape: tuple[int, ...]
    dtype: str = "float32"


class Part:
    """Base class of all parts. Sub-classes override what they need."""

    def param_specs(self) -> dict[str, ParamSpec]:
        return {}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        """Receive the tensors named by ``param_specs`` (already on the device, already in the
        type their kind asks for). A part may re-lay them out for its kernels here."""
        for name, tensor in params.items():
            setattr(self, name, tensor)

    def sub_parts(self) -> dict[str, "Part"]:
        """Named children whose tensors are prefixed with their name."""
        return {}

    def cache_request(self) -> PagedKVRequest | StateRequest | None:
        return None

    #: True when ``forward`` only launches work on the current stream (no host reads of device
    #: data, no host-dependent control flow), so that a step may be captured in a CUDA graph.
    graph_safe = False

    #: True for a mixer or feed-forward whose ``forward`` ends in a matrix product and accepts
    #: ``finish``: a callable ``finish(x, w_nk)`` that stands for ``x @ w_nk^T`` followed by
    #: whatever the caller does with it next (the residual add and the following norm), so that
    #: one kernel can do both. ``forward`` then returns what ``finish`` returned.
    fuses_last_linear = False

    #: Whether that last product may be launched as a programmatic dependent of the part's kernel
    #: before it (see ``ops.gemm.linear``). False where that kernel leaves the SMs divided between
    #: L1 cache and shared memory in a way that slows the product down.
    chains_last_linear = True

    #: True for a mixer or feed-forward that hands its input straight to ``ops.gemm.linear`` or
    #: ``linear_silu_mul`` and so can take an ``ops.gemm.PendingNorm`` in place of a tensor.
    accepts_pending_norm = False

    def plan_step(self, ctx: "StepContext", binding: "CacheBinding | None") -> None:
        """Called once per layer call before a step's kernels run, on the host: a part that needs
        integer arrays on the device (work lists, tables) adds them to ``ctx.arena`` here, so that
        everything a step needs crosses to the device in one copy."""


@dataclass(slots=True)
class Normed:
    """What a block may hand on instead of a pending residual update: the stream has already
    taken the update, and ``values`` is the stream normalised by ``norm`` (the first norm of the
    block that comes next)."""

    values: torch.Tensor
    norm: object


class Block(Part):
    """The arrangement of the parts of one layer, and the interface the step function runs.

    The residual stream ``hidden`` is a float32 tensor ``[tokens, width]`` that blocks update in
    place. A residual add is never a kernel of its own: whoever produces an update hands it on as
    *pending*, and the norm that follows adds it while it normalises. Between blocks that means:

    * ``forward(hidden, pending, ctx, binding, next_norm=None)`` receives what the block before
      handed on: ``None`` (the first block: the stream holds the embeddings), a tensor (that
      block's last update, not yet added to ``hidden``), or a ``Normed`` (that block already added
      its update and applied ``first_norm`` of this block; ``Normed.norm`` says which norm it was,
      and a block that is handed a ``Normed`` made for another norm must refuse it).
    * It returns its own last update as a tensor, or, when ``next_norm`` was given (the
      ``first_norm`` of the block that runs next) and it could apply it in the tail of its last
      kernel, a ``Normed(values, next_norm)``. A block may always ignore ``next_norm`` and
      return a tensor.
    * ``first_norm`` is the norm the block applies to the stream it is given, or ``None`` when it
      has none that a predecessor could apply for it (the step function then never passes
      ``next_norm`` to the block before).

    The last block's update is added by the model's final norm. ``plan_step`` and
    ``cache_request`` are those of ``Part``; a block usually passes them on to its mixer.
    """

    @property
    def first_norm(self) -> "Part | None":
        return None

    def forward(self, hidden: torch.Tensor, pending: "torch.Tensor | Normed | None", ctx: "StepContext",
                binding: "CacheBinding | None", next_norm: "Part | None" = None) -> "torch.Tensor | Normed":
        raise NotImplementedError


class IntArena:
    """Collects the int32 arrays of one step on the host and uploads them in a single copy."""

    def __init__(self) -> None:
        self._arrays: dict[str, np.ndarray] = {}
        self._device: dict[str, torch.Tensor] = {}
        self._pinned: torch.Tensor | None = None      # kept alive until the copy has run
        self._offsets: dict[str, int] = {}
        self._total = 0
        self.uploaded = False
        self.bytes_uploaded = 0

    def __contains__(self, name: str) -> bool:
        return name in self._arrays

    def add(self, name: str, values: Any, shape: tuple[int, ...] | None = None) -> None:
        if self.uploaded:
            raise RuntimeError("the step's integer arrays were already uploaded")
        array = np.ascontiguousarray(np.asarray(values, dtype=np.int32))
        if shape is not None:
            array = array.reshape(shape)
        self._arrays[name] = array

    def signature(self) -> tuple:
        """Names and shapes in order: two arenas with equal signatures have the same layout."""
        return tuple((name, array.shape) for name, array in self._arrays.items())

    def total_ints(self) -> int:
        return max(4, sum((a.size + 3) // 4 * 4 for a in self._arrays.values()))

    def stage(self) -> None:
        """Pack every array into one pinned host buffer (each starts on a 16-byte boundary).
        A step prepared ahead of time stops here; ``patch`` may still change values."""
        names = list(self._arrays)
        sizes = [self._arrays[n].size for n in names]
        offsets, total = [], 0
        for size in sizes:
            offsets.append(total)
            total += (size + 3) // 4 * 4
        host = torch.empty((max(total, 4),), dtype=torch.int32, pin_memory=torch.cuda.is_available())
        view = host.numpy()
        for name, offset, size in zip(names, offsets, sizes):
            view[offset:offset + size] = self._arrays[name].reshape(-1)
        self._pinned, self._offsets, self._total = host, dict(zip(names, offsets)), total

    def patch(self, name: str, values: Any) -> None:
        """Overwrite a staged array (same size) before it is sent."""
        if self.uploaded or self._pinned is None:
            raise RuntimeError("only a staged, unsent arena can be patched")
        array = np.ascontiguousarray(np.asarray(values, dtype=np.int32)).reshape(self._arrays[name].shape)
        self._arrays[name] = array
        offset = self._offsets[name]
        self._pinned.numpy()[offset:offset + array.size] = array.reshape(-1)

    def upload(self, device: torch.device, into: torch.Tensor | None = None, views: bool = True) -> None:
        """Copy every array to the device in one transfer: into a fresh buffer, or into ``into``
        (an int32 device tensor of ``total_ints()`` elements that a captured graph reads).
        ``views=False`` skips the per-array device views (a graph replay reads ``into`` by the
        addresses it captured and asks for none)."""
        if self._pinned is None:
            self.stage()
        host = self._pinned
        if into is None:
            dev = host.to(device, non_blocking=True)
        else:
            if into.numel() < host.numel() or into.dtype != torch.int32:
                raise ValueError("the static integer buffer does not fit this step's arrays")
            dev = into
            dev[:host.numel()].copy_(host, non_blocking=True)
        if views:
            for name, offset in self._offsets.items():
                array = self._arrays[name]
                self._device[name] = dev[offset:offset + array.size].view(array.shape)
        self.uploaded = True
        self.bytes_uploaded = self._total * 4

    def __getitem__(self, name: str) -> torch.Tensor:
        return self._device[name]

    def host(self, name: str) -> np.ndarray:
        return self._arrays[name]


@dataclass(frozen=True, slots=True)
class CacheBinding:
    """Where one layer call finds its cache: ``group``/``index`` select a layer's pages inside a
    page group (or ``state`` a state tensor); ``write=False`` reads what another call wrote."""

    entry: int
    group: int | None = None
    index: int | None = None
    state: int | None = None
    write: bool = True


@dataclass(slots=True)
class GroupView:
    """One page group as a step sees it."""

    k_pool: torch.Tensor          # [layers of the group, pages, KV, page_size, hd]
    v_pool: torch.Tensor
    page_size: int
    window: int | None
    table_name: str               # arena names of this group's arrays
    slots_name: str


@dataclass(slots=True)
class StepContext:
    """Everything the parts may read during one step."""

    dtype: torch.dtype
    device: torch.device
    num_tokens: int
    num_seqs: int
    seq_lens: list[int]                # tokens of each entry in this step
    first_positions: list[int]         # absolute position of each entry's first token
    arena: IntArena
    groups: list[GroupView] = field(default_factory=list)
    states: list[torch.Tensor] = field(default_factory=list)   # [slots, *shape] per state entry
    scratch: dict[str, Any] = field(default_factory=dict)
    #: When set, parts plan launch shapes from this context length instead of the batch's own
    #: (a captured graph must keep its launch shapes from step to step).
    planning_context_len: int | None = None
    #: The device's status word (int32 [1]): kernels record a fault code there instead of trapping.
    status: torch.Tensor | None = None
    #: Where the sampler of the step before left its ids; a token whose ``TOKEN_FEEDBACK`` entry
    #: is not negative takes its id from there (see ``ModelRunner.sampled_ids``).
    fed_back_ids: torch.Tensor | None = None

    # the arrays every step has (names in the arena)
    TOKEN_IDS = "token_ids"
    POSITIONS = "positions"
    SEQ_STARTS = "seq_starts"
    FIRST_POS = "first_pos"
    CONTEXT_LENS = "context_lens"
    STATE_SLOTS = "state_slots"
    LOGITS_ROWS = "logits_rows"
    TOKEN_FEEDBACK = "token_feedback"   # per token: -1, or the place of its id in the sampler's output buffer

    def ints(self, name: str) -> torch.Tensor:
        return self.arena[name]
