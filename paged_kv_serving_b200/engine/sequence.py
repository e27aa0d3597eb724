"""Requests, sampling parameters and the per-sample state the scheduler moves around.

One rule covers prefill, portions of a prompt, decoding and recomputation after preemption
(reference: src/paged_kv_serving/engine/sequence.py:1-13): ``token_ids`` is the prompt followed
by everything sampled so far, ``num_computed_tokens`` counts the leading tokens whose keys and
values are in the cache, a step runs ``token_ids[computed : computed + n]`` at those positions,
and it yields logits exactly when the portion reaches the end of ``token_ids``.
Names and defaults of ``SamplingParams`` and ``Request`` are the reference's
(src/paged_kv_serving/engine/sequence.py:64-126).
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from enum import Enum

import numpy as np

__all__ = [
    "GREEDY_TEMPERATURE", "FinishReason", "Request", "SamplingParams", "Sequence", "SequenceStatus",
    "SloClass", "finish_reason_for", "new_sequence_id",
]

#: Below this temperature a request is decoded greedily
#: (reference: src/paged_kv_serving/engine/sequence.py:42).
GREEDY_TEMPERATURE = 1e-5

_ORDER = itertools.count()


class SloClass(Enum):
    """Service class; a lower rank is scheduled first
    (reference: src/paged_kv_serving/engine/config.py:17-32)."""

    INTERACTIVE = ("interactive", 0)
    BATCH = ("batch", 1)

    def __init__(self, label: str, rank: int) -> None:
        self.label = label
        self.rank = rank

    @classmethod
    def parse(cls, value: str) -> "SloClass":
        for member in cls:
            if member.label == value:
                return member
        raise ValueError(f"unknown SLO class {value!r}")


class SequenceStatus(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED = "finished"
    ABORTED = "aborted"


class FinishReason(Enum):
    LENGTH = "length"
    STOP = "stop"
    CONTEXT_LIMIT = "context_limit"
    ABORTED = "aborted"


@dataclass(frozen=True, slots=True)
class SamplingParams:
    max_new_tokens: int = 32
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0
    ignore_eos: bool = False

    def __post_init__(self) -> None:
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        if self.temperature < 0.0:
            raise ValueError("temperature must be >= 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.seed < 0:
            raise ValueError("seed must be >= 0")

    @property
    def greedy(self) -> bool:
        return self.temperature < GREEDY_TEMPERATURE


@dataclass(frozen=True, slots=True)
class Request:
    """A submitted request; its ``n`` samples share the prompt's pages."""

    request_id: str
    prompt_token_ids: tuple[int, ...]
    sampling: SamplingParams = SamplingParams()
    n: int = 1
    slo_class: SloClass = SloClass.INTERACTIVE
    deadline_seconds: float | None = None
    key_id: str = "anonymous"
    arrival_time: float = 0.0

    def __post_init__(self) -> None:
        if not self.prompt_token_ids:
            raise ValueError("the prompt must contain at least one token")
        if self.n < 1:
            raise ValueError("n must be >= 1")
        if self.deadline_seconds is not None and self.deadline_seconds <= 0:
            raise ValueError("deadline_seconds must be > 0")

    @property
    def prompt_len(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def deadline(self) -> float | None:
        return None if self.deadline_seconds is None else self.arrival_time + self.deadline_seconds


def new_sequence_id(request_id: str, index: int) -> str:
    return f"{request_id}#{index}"


@dataclass(slots=True)
class Sequence:
    """One sample of a request."""

    seq_id: str
    request: Request
    sample_index: int = 0
    token_ids: list[int] = field(default_factory=list)
    block_tables: list[list[int]] = field(default_factory=lambda: [[]])   # one table per page group
    num_computed_tokens: int = 0
    status: SequenceStatus = SequenceStatus.WAITING
    finish_reason: FinishReason | None = None
    cached_prefix_blocks: int = 0
    fork_slots: int = 0
    block_hashes: list[bytes] = field(default_factory=list)
    state_slot: int | None = None
    preemption_count: int = 0
    first_token_time: float | None = None
    finish_time: float | None = None
    admission_order: int = field(default_factory=lambda: next(_ORDER))
    rng: np.random.Generator | None = None

    @classmethod
    def from_request(cls, request: Request, sample_index: int, num_groups: int = 1) -> "Sequence":
        sequence = cls(
            seq_id=new_sequence_id(request.request_id, sample_index),
            request=request,
            sample_index=sample_index,
            token_ids=list(request.prompt_token_ids),
            block_tables=[[] for _ in range(max(1, num_groups))],
        )
        # One generator per sample: output depends on (seed, sample index) only
        # (reference: src/paged_kv_serving/engine/sequence.py:165-170).
        sequence.rng = np.random.default_rng(
            np.random.SeedSequence(entropy=request.sampling.seed, spawn_key=(sample_index,)))
        return sequence

    # --- lengths -------------------------------------------------------------------------

    @property
    def block_table(self) -> list[int]:
        """The table of the first page group (the only one of an attention-only model)."""
        return self.block_tables[0]

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def num_output_tokens(self) -> int:
        return len(self.token_ids) - self.request.prompt_len

    @property
    def num_uncomputed_tokens(self) -> int:
        return len(self.token_ids) - self.num_computed_tokens

    @property
    def output_token_ids(self) -> list[int]:
        return self.token_ids[self.request.prompt_len:]

    @property
    def is_decoding(self) -> bool:
        return self.num_computed_tokens > 0 and self.num_uncomputed_tokens == 1

    @property
    def is_finished(self) -> bool:
        return self.status in (SequenceStatus.FINISHED, SequenceStatus.ABORTED)

    @property
    def holds_pages(self) -> bool:
        return any(self.block_tables)

    # --- transitions ---------------------------------------------------------------------

    def append_token(self, token_id: int) -> None:
        self.token_ids.append(int(token_id))

    def reset_for_recompute(self) -> None:
        """Forget what is cached; sampled tokens stay and are recomputed with the prompt
        (reference: src/paged_kv_serving/engine/sequence.py:210-221)."""
        self.num_computed_tokens = 0
        for table in self.block_tables:
            table.clear()
        self.block_hashes.clear()
        self.cached_prefix_blocks = 0
        self.status = SequenceStatus.PREEMPTED
        self.preemption_count += 1

    def finish(self, reason: FinishReason, now: float) -> None:
        self.status = SequenceStatus.ABORTED if reason is FinishReason.ABORTED else SequenceStatus.FINISHED
        self.finish_reason = reason
        self.finish_time = now

    def priority_key(self) -> tuple[int, float, int]:
        """Class, then earliest deadline, then arrival
        (reference: src/paged_kv_serving/engine/sequence.py:230-241)."""
        deadline = self.request.deadline
        return (self.request.slo_class.rank, float("inf") if deadline is None else deadline, self.admission_order)


def finish_reason_for(sequence: Sequence, token: int, *, eos_token_id: int | None,
                      max_context_tokens: int) -> FinishReason | None:
    """Why a sequence is done after sampling ``token``, or ``None``
    (reference: src/paged_kv_serving/engine/sequence.py:244-262; a stop token wins over the
    length cap, the context cap is checked last)."""
    sampling = sequence.request.sampling
    if eos_token_id is not None and token == eos_token_id and not sampling.ignore_eos:
        return FinishReason.STOP
    if sequence.num_output_tokens >= sampling.max_new_tokens:
        return FinishReason.LENGTH
    if sequence.num_tokens >= max_context_tokens:
        return FinishReason.CONTEXT_LIMIT
    return None
