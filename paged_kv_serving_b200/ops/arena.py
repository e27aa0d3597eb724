"""Activation memory of a step, handed out by bumping a pointer.

A step of a ragged batch allocates a hundred or so intermediate tensors whose sizes follow the
batch's token count, which changes from step to step. Through torch's caching allocator every
new size may end in ``cudaMalloc`` (measured: 110 us per ``torch.empty`` and 240 us per
``torch.mm`` in a serving run whose batches vary, most of the host's time), so the step function
gives its kernels' outputs memory of its own instead:

* a ``StepArena`` holds three *slots*, each a list of large blocks of device memory that grows
  when a step needs more and is never given back: the slot of the step (what lives as long as
  the step: the residual stream, the logits) and two slots that alternate from layer to layer
  (what a layer hands to the next one is still valid while that one runs, and dead one layer
  later);
* ``ops.empty`` carves tensors out of the active slot, or falls back to ``torch.empty`` when no
  arena is active (decode steps replayed as CUDA graphs keep torch's graph-private pool).

Memory handed out by an arena is valid until the slot is reset: the layer slots two layers on,
the step slot at the next step. Work is stream-ordered, so a later step's kernels never overwrite
what an earlier step's kernels still read.
"""

from __future__ import annotations

import torch

__all__ = ["StepArena", "active", "empty"]

_ALIGN = 256
_MIN_BLOCK = 64 << 20


class _Slot:
    """Blocks of device memory and a bump pointer into them."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.blocks: list[torch.Tensor] = []
        self.block = 0
        self.offset = 0

    def reset(self) -> None:
        self.block = 0
        self.offset = 0

    def take(self, nbytes: int) -> torch.Tensor:
        size = -(-max(nbytes, 1) // _ALIGN) * _ALIGN
        while self.block < len(self.blocks):
            block = self.blocks[self.block]
            if self.offset + size <= block.numel():
                piece = block[self.offset:self.offset + size]
                self.offset += size
                return piece
            self.block += 1
            self.offset = 0
        self.blocks.append(torch.empty((max(size, _MIN_BLOCK),), dtype=torch.uint8, device=self.device))
        self.block = len(self.blocks) - 1
        self.offset = size
        return self.blocks[-1][:size]

    @property
    def reserved_bytes(self) -> int:
        return sum(b.numel() for b in self.blocks)


class StepArena:
    """Three slots: the step's and two that alternate between layers."""

    def __init__(self, device: torch.device | str) -> None:
        self.device = torch.device(device)
        self.step_slot = _Slot(self.device)
        self.layer_slots = (_Slot(self.device), _Slot(self.device))
        self._current = self.step_slot
        self._layer = 0

    def begin_step(self) -> None:
        """Everything of the step before is dead: start over."""
        self.step_slot.reset()
        self.layer_slots[0].reset()
        self.layer_slots[1].reset()
        self._layer = 0
        self._current = self.step_slot

    def next_layer(self) -> None:
        """A layer begins: what the layer before the last one allocated is dead."""
        self._layer ^= 1
        self._current = self.layer_slots[self._layer]
        self._current.reset()

    def end_layers(self) -> None:
        """After the last layer: allocations live as long as the step again."""
        self._current = self.step_slot

    def empty(self, shape, dtype: torch.dtype) -> torch.Tensor:
        count = 1
        for s in shape:
            count *= int(s)
        itemsize = torch.empty((), dtype=dtype).element_size() if dtype not in _ITEMSIZE else _ITEMSIZE[dtype]
        return self._current.take(count * itemsize)[:count * itemsize].view(dtype).view(tuple(int(s) for s in shape))

    @property
    def reserved_bytes(self) -> int:
        return self.step_slot.reserved_bytes + sum(s.reserved_bytes for s in self.layer_slots)


_ITEMSIZE = {torch.float32: 4, torch.bfloat16: 2, torch.float16: 2, torch.int32: 4, torch.uint8: 1, torch.float64: 8,
             torch.int64: 8}
_ACTIVE: list[StepArena | None] = [None]


def active() -> StepArena | None:
    return _ACTIVE[0]


def activate(arena: StepArena | None) -> StepArena | None:
    """Make ``arena`` the one ``empty`` draws from (``None``: torch's allocator); returns the previous one."""
    before = _ACTIVE[0]
    _ACTIVE[0] = arena
    return before


def empty(shape, dtype: torch.dtype, device: torch.device | str) -> torch.Tensor:
    """An uninitialised tensor for a kernel's output: from the active arena when there is one on
    that device, else from torch's allocator."""
    arena = _ACTIVE[0]
    if arena is not None and arena.device == torch.device(device):
        return arena.empty(shape, dtype)
    return torch.empty(tuple(shape), dtype=dtype, device=device)
