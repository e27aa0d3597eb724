"""Trace replay: feed given token ids through a model step by step and write the logits.

Nothing is sampled. A ``ReplaySession`` drives the framework's own model, step function, cache
manager and kernels: the ones generation uses. Each request of a trace is a sequence whose
tokens arrive a few at a time; pages are reserved through the cache manager as the tokens come
and given back when the trace ends the request, so that a small pool reuses pages.
The reference's nearest pieces are ``paged_chunked_logits`` and ``RecordingExecutor``
(src/paged_kv_serving/engine/equivalence.py:49-139).

Input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` holds the float32 logits
``[wanted, vocab]`` in the order of the entries and of ``want``; ``done <step>`` is printed and
flushed after every step.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.cache.manager import KVCacheManager
from paged_kv_serving_b200.engine.batch import BatchEntry, ExecutionBatch
from paged_kv_serving_b200.engine.sequence import PageTable, Request, SamplingParams, Sequence

__all__ = ["ReplaySession", "main"]

#: A request's token count is rounded up to a multiple of this when the pool is sized.
TOKEN_ROUNDING = 64


class ReplaySession:
    """A model, a page pool sized for ``max_tokens`` live tokens, and the live requests."""

    def __init__(self, model, *, max_tokens: int, block_size: int = 16, max_live: int = 64) -> None:
        from paged_kv_serving_b200.engine.runner import ModelRunner

        if block_size < 1 or max_tokens < 1:
            raise ValueError("max_tokens and block_size must be >= 1")
        rounding = max(TOKEN_ROUNDING, block_size)
        capacity = -(-max_tokens // rounding) * rounding
        self.block_size = block_size
        self.num_blocks = -(-capacity // block_size)
        self.model = model
        self.runner = ModelRunner(model, num_blocks=self.num_blocks, block_size=block_size, max_running_seqs=max_live)
        self.cache = KVCacheManager(self.runner.groups, num_blocks=self.num_blocks, block_size=block_size,
                                    store=self.runner, enable_prefix_cache=False,
                                    num_state_slots=self.runner.num_state_slots)
        self.live: dict[str, Sequence] = {}

    def _sequence(self, name: str, first_tokens: list[int]) -> Sequence:
        sequence = self.live.get(name)
        if sequence is None:
            request = Request(request_id=name, prompt_token_ids=tuple(first_tokens),
                              sampling=SamplingParams(max_new_tokens=1))
            sequence = Sequence.from_request(request, 0, num_groups=self.cache.num_groups)
            sequence.token_ids = []
            self.cache.acquire_state_slot(sequence)
            self.live[name] = sequence
        return sequence

    def step(self, entries: list[dict], end: list[str] | tuple[str, ...] = ()) -> np.ndarray | None:
        """Run one step of a trace; returns the wanted logits ``[wanted, vocab]`` or ``None``."""
        batch_entries = []
        advanced = []
        for item in entries:
            name, tokens = str(item["id"]), [int(t) for t in item["tokens"]]
            want = tuple(int(w) for w in item.get("want", ()))
            if not tokens:
                raise ValueError(f"request {name}: an entry must bring at least one token")
            sequence = self._sequence(name, tokens)
            start = sequence.num_computed_tokens
            sequence.token_ids.extend(tokens)
            self.cache.reserve(sequence, start + len(tokens))
            batch_entries.append(BatchEntry(
                seq_id=name, token_ids=tuple(tokens), first_position=start,
                block_tables=tuple(table.snapshot() if isinstance(table, PageTable) else tuple(table)
                                   for table in sequence.block_tables),
                logits_at=want, state_slot=sequence.state_slot))
            advanced.append((sequence, len(tokens)))
        clear = self.cache.state_slots.take_slots_to_clear() if self.cache.state_slots is not None else None
        result = self.runner.step(ExecutionBatch(tuple(batch_entries)), clear_state_slots=clear)
        for sequence, count in advanced:
            sequence.num_computed_tokens += count
            self.cache.release_behind_window(sequence)
        for name in end:
            sequence = self.live.pop(str(name), None)
            if sequence is not None:
                self.cache.free(sequence)
        # the wanted logits and the device's status word cross to the host behind one
        # synchronisation; a fault that a kernel recorded raises instead of writing wrong logits
        status = torch.empty((1,), dtype=torch.int32, pin_memory=True)
        status.copy_(self.runner.status, non_blocking=True)
        host = None
        if result.logits is not None:
            host = torch.empty(result.logits.shape, dtype=torch.float32, pin_memory=True)
            host.copy_(result.logits, non_blocking=True)
        torch.cuda.current_stream(self.model.device).synchronize()
        ops.raise_for_status(int(status[0]), self.model.device)
        return None if host is None else host.numpy().copy()

    def check_invariants(self) -> None:
        self.cache.check_invariants()


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description="replay token ids step by step, write logits")
    parser.add_argument("--model", required=True, type=Path, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    parser.add_argument("--out", required=True, type=Path, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", required=True, type=int,
                        help="most tokens live requests hold at any time (each rounded up to 64)")
    parser.add_argument("--block-size", type=int, default=16, help="tokens per page of the cache (default 16)")
    args = parser.parse_args(argv)

    print("[trace_run] loading the model", file=sys.stderr, flush=True)
    from paged_kv_serving_b200.models.decoder import DecoderModel

    model = DecoderModel.from_folder(args.model, dtype=args.dtype, device="cuda")
    session = ReplaySession(model, max_tokens=args.max_tokens, block_size=args.block_size)
    args.out.mkdir(parents=True, exist_ok=True)
    print("[trace_run] ready", file=sys.stderr, flush=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        logits = session.step(record.get("entries", []), record.get("end", []))
        if logits is not None:
            np.ascontiguousarray(logits, dtype="<f4").tofile(args.out / f"{step}.f32")
        print(f"done {step}", flush=True)
    return 0
