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

    def sample(self, logits: torch.Tensor, params: list[SamplingParams],
               generators: list[np.random.Generator]) -> list[int]:
        """One token per row of ``logits [R, V]`` (float32, on the device)."""
        rows, vocab = logits.shape
        if rows != len(params) or rows != len(generators):
            raise ValueError("one SamplingParams and one generator per logits row are required")
        host = np.zeros((rows, 4), dtype=np.float64)
        for i, (p, rng) in enumerate(zip(params, generators)):
            host[i, 0] = p.temperature
            host[i, 1] = p.top_p
            host[i, 2] = 0.0 if p.greedy else float(rng.random())
        staged = torch.from_numpy(host)
        if torch.cuda.is_available():
            staged = staged.pin_memory()
        dev = staged.to(self.device, non_blocking=True)
        temperature = dev[:, 0].to(torch.float32).contiguous()
        top_p = dev[:, 1].to(torch.float32).contiguous()
        uniform = dev[:, 2].contiguous()
        if self._probs is None or self._probs.numel() < rows * vocab:
            self._probs = torch.empty((rows * vocab,), dtype=torch.float32, device=self.device)
        ids = ops.sample(logits, temperature, top_p, uniform, GREEDY_TEMPERATURE, self._probs)
        return [int(t) for t in ids.cpu().tolist()]
