"""Sampling above the device kernel: per-sequence generators on the host, ids from the GPU.

Each sequence carries its own NumPy generator seeded from ``(seed, sample index)``
(src/paged_kv_serving/engine/sequence.py:165-170 of the reference); exactly one uniform number
is drawn per sampled token and none for a greedy one (src/paged_kv_serving/engine/sampling.py:3-10,
56-74), so output never depends on batching or preemption. The kernel receives the draw and
returns the token id.
"""

from __future__ import annotations

import numpy as np
import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.engine.sequence import GREEDY_TEMPERATURE, SamplingParams

__all__ = ["Sampler"]


class Sampler:
    """Turns logits rows into token ids on the device."""

    def __init__(self, device: torch.device | str = "cuda") -> None:
        self.device = torch.device(device)
        self._probs: torch.Tensor | None = None
        self._greedy: dict[int, tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}
        # pinned staging buffers for the draws and parameters of a step, used in turn: the host may
        # run a step ahead of the GPU, so a buffer is written again only once its copy has run
        self._staging: list[tuple[torch.Tensor, torch.cuda.Event]] = []
        self._turn = 0

    def _stage(self, nbytes: int) -> tuple[torch.Tensor, "torch.cuda.Event"]:
        if len(self._staging) < 4:
            size = max(nbytes, 4096)
            self._staging.append((torch.empty((size,), dtype=torch.uint8, pin_memory=torch.cuda.is_available()),
                                  torch.cuda.Event()))
            return self._staging[-1]
        self._turn = (self._turn + 1) % 4
        buffer, event = self._staging[self._turn]
        event.synchronize()
        if buffer.numel() < nbytes:
            buffer = torch.empty((nbytes,), dtype=torch.uint8, pin_memory=torch.cuda.is_available())
            self._staging[self._turn] = (buffer, event)
        return buffer, event

    def sample(self, logits: torch.Tensor, params: list[SamplingParams],
               generators: list[np.random.Generator]) -> list[int]:
        """One token per row of ``logits [R, V]`` (float32, on the device), read back to the host."""
        return [int(t) for t in self.sample_on_device(logits, params, generators).cpu().tolist()]

    def sample_on_device(self, logits: torch.Tensor, params: list[SamplingParams],
                         generators: list[np.random.Generator], status: torch.Tensor | None = None,
                         out: torch.Tensor | None = None) -> torch.Tensor:
        """The same ids as an int32 tensor on the device: nothing waits for the GPU. With
        ``status`` (the device's status word) one more element follows the ids: the word's value
        once the step's kernels have finished, so that one copy brings back ids and faults. ``out``
        (an int32 device buffer) receives the ids where the next step's embedding lookup can read them."""
        rows, vocab = logits.shape
        if rows != len(params) or rows != len(generators):
            raise ValueError("one SamplingParams and one generator per logits row are required")
        if all(p.greedy for p in params):
            # nothing to send: no draw is made for a greedy row (cached zeros and ones per row count)
            cached = self._greedy.get(rows)
            if cached is None:
                cached = self._greedy[rows] = (torch.zeros(rows, dtype=torch.float32, device=self.device),
                                               torch.ones(rows, dtype=torch.float32, device=self.device),
                                               torch.zeros(rows, dtype=torch.float64, device=self.device))
            temperature, top_p, uniform = cached
        else:
            # one pinned buffer, one copy: [rows] float64 draws, then [rows] float32 temperatures and top-p
            buffer, copied = self._stage(rows * 16)
            staged = buffer[:rows * 16]
            draws = staged[:rows * 8].view(torch.float64).numpy()
            floats = staged[rows * 8:].view(torch.float32).numpy()
            floats[:rows] = [p.temperature for p in params]
            floats[rows:] = [p.top_p for p in params]
            draws[:] = [0.0 if p.greedy else rng.random() for p, rng in zip(params, generators)]
            dev = staged.to(self.device, non_blocking=True)
            copied.record()
            uniform = dev[:rows * 8].view(torch.float64)
            temperature = dev[rows * 8:rows * 12].view(torch.float32)
            top_p = dev[rows * 12:].view(torch.float32)
        if self._probs is None or self._probs.numel() < rows * vocab:
            self._probs = torch.empty((rows * vocab,), dtype=torch.float32, device=self.device)
        return ops.sample(logits, temperature, top_p, uniform, GREEDY_TEMPERATURE, self._probs, status, out)
