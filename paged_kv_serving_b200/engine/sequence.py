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
import math
from dataclasses import dataclass, field
from enum import Enum

import numpy as np

__all__ = [
    "GREEDY_TEMPERATURE", "FinishReason", "PageTable", "Request", "SamplingParams", "Sequence", "SequenceStatus",
    "SloClass", "TableSnapshot", "finish_reason_for", "new_sequence_id",
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
    """How a request's tokens are chosen; the field names and defaults are the reference's
    (src/paged_kv_serving/engine/sequence.py:64-87)."""

    max_new_tokens: int = 32
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0
    ignore_eos: bool = False

    def __post_init__(self) -> None:
        problems = []
        if self.max_new_tokens < 1:
            problems.append(f"max_new_tokens is {self.max_new_tokens}: a request generates one token or more")
        if self.temperature < 0.0:
            problems.append(f"temperature is {self.temperature}: it cannot be negative (0 decodes greedily)")
        if not 0.0 < self.top_p <= 1.0:
            problems.append(f"top_p is {self.top_p}: the nucleus mass lies in (0, 1]")
        if self.seed < 0:
            problems.append(f"seed is {self.seed}: seeds are non-negative integers")
        if problems:
            raise ValueError("; ".join(problems))

    @property
    def greedy(self) -> bool:
        return self.temperature < GREEDY_TEMPERATURE


@dataclass(frozen=True, slots=True)
class Request:
    """A submitted request; its ``n`` samples share the prompt's pages
    (fields as in the reference, src/paged_kv_serving/engine/sequence.py:90-126)."""

    request_id: str
    prompt_token_ids: tuple[int, ...]
    sampling: SamplingParams = SamplingParams()
    n: int = 1
    slo_class: SloClass = SloClass.INTERACTIVE
    deadline_seconds: float | None = None
    key_id: str = "anonymous"
    arrival_time: float = 0.0

    def __post_init__(self) -> None:
        if len(self.prompt_token_ids) == 0:
            raise ValueError(f"request {self.request_id}: an empty prompt has no position to predict from")
        if self.n < 1:
            raise ValueError(f"request {self.request_id}: n is {self.n}, at least one sample is generated")
        if self.deadline_seconds is not None and not self.deadline_seconds > 0:
            raise ValueError(f"request {self.request_id}: a deadline lies after the arrival (deadline_seconds > 0)")

    @property
    def prompt_len(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def deadline(self) -> float | None:
        return None if self.deadline_seconds is None else self.arrival_time + self.deadline_seconds


def new_sequence_id(request_id: str, index: int) -> str:
    return f"{request_id}#{index}"


class TableSnapshot(tuple):
    """The page numbers of a ``PageTable`` at one moment: a tuple (what a batch entry holds) that
    also gives them as an int32 array, made once."""

    @property
    def array(self) -> np.ndarray:
        made = self.__dict__.get("_array")
        if made is None:
            made = self.__dict__["_array"] = np.asarray(self, dtype=np.int32)
            made.flags.writeable = False
        return made


class PageTable(list):
    """A sequence's pages in one page group, in logical order: a list that keeps an immutable
    copy of itself until it is changed. A decode step of hundreds of sequences changes a few
    tables (a page is added every ``block_size`` tokens); the others hand the step the tuple and
    the array they made before."""

    __slots__ = ("_snapshot",)

    def __init__(self, *args) -> None:
        super().__init__(*args)
        self._snapshot = None

    def snapshot(self) -> TableSnapshot:
        made = self._snapshot
        if made is None:
            made = self._snapshot = TableSnapshot(self)
        return made

    def _changed(method):  # noqa: N805 - wraps the list methods that change the content
        def wrapper(self, *args, **kwargs):
            self._snapshot = None
            return method(self, *args, **kwargs)
        wrapper.__name__ = method.__name__
        return wrapper

    append = _changed(list.append)
    extend = _changed(list.extend)
    insert = _changed(list.insert)
    pop = _changed(list.pop)
    remove = _changed(list.remove)
    clear = _changed(list.clear)
    reverse = _changed(list.reverse)
    sort = _changed(list.sort)
    __setitem__ = _changed(list.__setitem__)
    __delitem__ = _changed(list.__delitem__)
    __iadd__ = _changed(list.__iadd__)
    __imul__ = _changed(list.__imul__)
    del _changed


@dataclass(slots=True)
class Sequence:
    """One sample of a request."""

    seq_id: str
    request: Request
    sample_index: int = 0
    token_ids: list[int] = field(default_factory=list)
    block_tables: list[list[int]] = field(default_factory=lambda: [PageTable()])   # one table per page group
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
    #: Tokens at the end of ``token_ids`` that stand in for ids sampled on the device and not
    #: read back yet (the engine's overlapped steps); their values mean nothing until settled.
    num_unsettled_tokens: int = 0

    @classmethod
    def from_request(cls, request: Request, sample_index: int, num_groups: int = 1) -> "Sequence":
        """Sample ``sample_index`` of ``request``, with nothing computed and nothing held. Its
        generator is seeded by (the request's seed, the sample's index) alone, so what it draws
        depends on nothing else (reference: src/paged_kv_serving/engine/sequence.py:165-170)."""
        seed = np.random.SeedSequence(entropy=request.sampling.seed, spawn_key=(sample_index,))
        return cls(seq_id=new_sequence_id(request.request_id, sample_index), request=request,
                   sample_index=sample_index, token_ids=[int(t) for t in request.prompt_token_ids],
                   block_tables=[PageTable() for _ in range(max(1, num_groups))], rng=np.random.default_rng(seed))

    # --- lengths -------------------------------------------------------------------------

    @property
    def block_table(self) -> list[int]:
        """The table of the first page group (the only one of an attention-only model)."""
        return self.block_tables[0]

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def num_settled_tokens(self) -> int:
        """Leading tokens whose ids are final."""
        return len(self.token_ids) - self.num_unsettled_tokens

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
        """After preemption: the cache holds nothing of this sequence any more. Its tokens, the
        sampled ones included, all stay and will be run again like a prompt, which draws no random
        number (reference: src/paged_kv_serving/engine/sequence.py:210-221)."""
        self.status = SequenceStatus.PREEMPTED
        self.preemption_count += 1
        self.num_computed_tokens = self.cached_prefix_blocks = 0
        self.block_hashes = []
        self.block_tables = [PageTable() for _ in self.block_tables]

    def finish(self, reason: FinishReason, now: float) -> None:
        aborted = reason is FinishReason.ABORTED
        self.finish_reason, self.finish_time = reason, now
        self.status = SequenceStatus.ABORTED if aborted else SequenceStatus.FINISHED

    def priority_key(self) -> tuple[int, float, int]:
        """Sort key of the scheduler: service class first, then the earlier deadline (none sorts
        last), then the order of admission (reference: src/paged_kv_serving/engine/sequence.py:230-241)."""
        request = self.request
        return (request.slo_class.rank, math.inf if request.deadline is None else request.deadline, self.admission_order)


def finish_reason_for(sequence: Sequence, token: int | None, *, eos_token_id: int | None, max_context_tokens: int,
                      num_output_tokens: int | None = None) -> FinishReason | None:
    """Why a sequence is done once it has ``num_output_tokens`` sampled tokens (default: all it
    holds now), the newest being ``token``; ``None`` if it goes on. A stop token counts before the
    caps, the cap on new tokens before the cap on the context
    (reference: src/paged_kv_serving/engine/sequence.py:244-262). With ``token=None`` only the
    caps are looked at: whether the sequence is complete whatever its newest token is."""
    sampling = sequence.request.sampling
    produced = sequence.num_output_tokens if num_output_tokens is None else num_output_tokens
    stops = token is not None and eos_token_id is not None and not sampling.ignore_eos and token == eos_token_id
    if stops:
        return FinishReason.STOP
    if produced >= sampling.max_new_tokens:
        return FinishReason.LENGTH
    if sequence.request.prompt_len + produced >= max_context_tokens:
        return FinishReason.CONTEXT_LIMIT
    return None
