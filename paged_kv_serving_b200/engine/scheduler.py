"""Continuous batching with chunked prefill and preemption by recomputation.

Every step the batch is decided anew under a token budget (``max_batched_tokens``):

1. *Decode first.* Each running sequence whose prompt is computed gets one token, in priority
   order, so a long prompt never delays sequences that are already generating.
2. *Then prompts.* Running sequences with an unfinished prompt and waiting sequences are walked
   in one priority order (class, deadline, arrival). A running one takes its next portion; a
   waiting one is admitted with its first portion while running slots, pages and the watermark
   allow. A portion is cut by the remaining budget, by what the pools can hold and, for classes
   below the highest one with work, by the lower-class allowance.

When pages run out, the lowest-priority sequence that has not been scheduled yet in this step
is preempted: its pages are given back, its computed count returns to zero, it keeps all its
tokens (prompt and output) and waits to be recomputed. Nothing new is admitted in a step that
preempted. No step is empty while work is queued: a sequence that cannot get a page preempts
somebody behind it, a waiter that is not admitted holds nothing, and the watermark is ignored
when nothing runs.

These are the decisions of the reference's scheduler (src/paged_kv_serving/engine/scheduler.py:
114-425; preemption: docs/adr/0002-preemption-by-recomputation.md of the reference), restated
over a cache manager with several page groups and state slots. ``max_prefill_chunk`` is this
engine's addition.
"""

from __future__ import annotations

from dataclasses import dataclass

from paged_kv_serving_b200.cache.manager import KVCacheManager
from paged_kv_serving_b200.cache.pages import OutOfPages
from paged_kv_serving_b200.config.engine_config import EngineConfig
from paged_kv_serving_b200.engine.batch import BatchEntry, ExecutionBatch
from paged_kv_serving_b200.engine.sequence import PageTable, Sequence, SequenceStatus

__all__ = ["ScheduledSequence", "Scheduler", "SchedulerOutput", "SchedulerStats"]


@dataclass(frozen=True, slots=True)
class ScheduledSequence:
    """A sequence and how many of its tokens this step computes. ``produces_token`` is fixed
    here, while ``num_computed_tokens`` still describes the state the batch was built from."""

    sequence: Sequence
    num_tokens: int
    is_prefill: bool
    produces_token: bool


@dataclass(frozen=True, slots=True)
class SchedulerOutput:
    batch: ExecutionBatch
    scheduled: tuple[ScheduledSequence, ...] = ()
    preempted: tuple[str, ...] = ()
    admitted: tuple[str, ...] = ()

    @property
    def is_empty(self) -> bool:
        return not self.scheduled

    @property
    def num_batched_tokens(self) -> int:
        return self.batch.num_tokens


@dataclass(slots=True)
class SchedulerStats:
    iterations: int = 0
    preemptions: int = 0
    batched_tokens: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0

    @property
    def mean_batch_size(self) -> float:
        return self.batched_tokens / self.iterations if self.iterations else 0.0


class _StepPlan:
    """Mutable state of one call of ``schedule``."""

    def __init__(self, budget: int, top_rank: int, lower_allowance: int) -> None:
        self.budget = budget
        self.top_rank = top_rank
        self.lower_left = lower_allowance
        self.scheduled: list[ScheduledSequence] = []
        self.preempted: list[str] = []
        self.admitted: list[str] = []

    def allowed(self, sequence: Sequence, tokens: int) -> int:
        """Cut a portion to the lower-class allowance (higher classes are never cut)."""
        if sequence.request.slo_class.rank <= self.top_rank:
            return tokens
        return min(tokens, self.lower_left)

    def spend(self, sequence: Sequence, tokens: int, *, prefill: bool, produces: bool) -> None:
        self.scheduled.append(ScheduledSequence(sequence, tokens, is_prefill=prefill, produces_token=produces))
        self.budget -= tokens
        if prefill and sequence.request.slo_class.rank > self.top_rank:
            self.lower_left -= tokens


class Scheduler:
    """Waiting and running queues over one cache manager."""

    def __init__(self, config: EngineConfig, cache: KVCacheManager) -> None:
        self.config = config
        self.cache = cache
        self._waiting: list[Sequence] = []
        self._running: list[Sequence] = []
        self.stats = SchedulerStats()

    # --- queues --------------------------------------------------------------------------

    @property
    def waiting(self) -> tuple[Sequence, ...]:
        return tuple(self._waiting)

    @property
    def running(self) -> tuple[Sequence, ...]:
        return tuple(self._running)

    @property
    def queue_depth(self) -> int:
        return len(self._waiting)

    @property
    def num_running(self) -> int:
        return len(self._running)

    @property
    def has_work(self) -> bool:
        return bool(self._waiting or self._running)

    @property
    def slots_in_use(self) -> int:
        """Running sequences plus the forks they have yet to create."""
        return sum(1 + s.fork_slots for s in self._running)

    def add(self, sequence: Sequence) -> None:
        sequence.status = SequenceStatus.WAITING
        self._waiting.append(sequence)

    def add_running(self, sequence: Sequence) -> None:
        """Insert a fork whose keys and values are already in the cache."""
        sequence.status = SequenceStatus.RUNNING
        self._running.append(sequence)

    def remove(self, sequence: Sequence) -> None:
        if sequence in self._running:
            self._running.remove(sequence)
        elif sequence in self._waiting:
            self._waiting.remove(sequence)
        self.cache.free(sequence)

    def drop_finished(self) -> list[Sequence]:
        done = [s for s in self._running if s.is_finished]
        for sequence in done:
            self._running.remove(sequence)
            self.cache.free(sequence)
        return done

    # --- one step ------------------------------------------------------------------------

    def schedule(self) -> SchedulerOutput:
        """Choose this step's batch. An empty batch means nothing can run."""
        everyone = (*self._running, *self._waiting)
        plan = _StepPlan(
            budget=self.config.max_batched_tokens,
            top_rank=min((s.request.slo_class.rank for s in everyone), default=0),
            lower_allowance=self.config.lower_class_prefill_tokens,
        )
        self._decode_phase(plan)
        self._prompt_phase(plan)
        self._waiting.sort(key=Sequence.priority_key)
        output = SchedulerOutput(
            batch=ExecutionBatch(tuple(self._entry(item) for item in plan.scheduled)),
            scheduled=tuple(plan.scheduled),
            preempted=tuple(plan.preempted),
            admitted=tuple(plan.admitted),
        )
        if plan.scheduled:
            self.stats.iterations += 1
            self.stats.batched_tokens += output.num_batched_tokens
            self.stats.prefill_tokens += sum(i.num_tokens for i in plan.scheduled if i.is_prefill)
            self.stats.decode_tokens += sum(i.num_tokens for i in plan.scheduled if not i.is_prefill)
        return output

    def _preempt(self, victim: Sequence, plan: _StepPlan) -> None:
        self._running.remove(victim)
        self.cache.free(victim)
        victim.reset_for_recompute()
        self._waiting.append(victim)
        self.stats.preemptions += 1
        plan.preempted.append(victim.seq_id)

    def _decode_phase(self, plan: _StepPlan) -> None:
        pending = sorted((s for s in self._running if s.is_decoding), key=Sequence.priority_key)
        at = 0                                   # pending[at:] are still to be scheduled
        while at < len(pending) and plan.budget > 0:
            sequence = pending[at]
            try:
                self.cache.reserve(sequence, sequence.num_tokens)
            except OutOfPages:
                # The weakest sequence not yet scheduled pays: the last pending decoder or a
                # sequence still in its prompt, whichever ranks lower. With nobody else left the
                # sequence preempts itself, which still frees its pages for the next step.
                in_prompt = [s for s in self._running if not s.is_decoding]
                victim = max([*in_prompt, pending[-1]], key=Sequence.priority_key)
                if victim is pending[-1]:
                    pending.pop()
                self._preempt(victim, plan)
                continue
            at += 1
            plan.spend(sequence, 1, prefill=False, produces=True)

    def _prompt_phase(self, plan: _StepPlan) -> None:
        self._waiting.sort(key=Sequence.priority_key)
        order = sorted([*(s for s in self._running if not s.is_decoding), *self._waiting], key=Sequence.priority_key)
        admitting = not plan.preempted
        for at, sequence in enumerate(order):
            if plan.budget <= 0:
                break
            if sequence.status is SequenceStatus.RUNNING:
                before = len(plan.preempted)
                self._continue_prompt(sequence, order[at + 1:], plan)
                admitting = admitting and len(plan.preempted) == before
            elif admitting:
                admitting = self._admit(sequence, plan)

    def _portion(self, sequence: Sequence, plan: _StepPlan) -> int:
        tokens = min(plan.budget, sequence.num_uncomputed_tokens)
        if self.config.max_prefill_chunk:
            tokens = min(tokens, self.config.max_prefill_chunk)
        return tokens

    def _continue_prompt(self, sequence: Sequence, behind: list[Sequence], plan: _StepPlan) -> None:
        wanted = plan.allowed(sequence, self._portion(sequence, plan))
        if wanted <= 0:
            return
        tokens = min(wanted, self.cache.coverable_tokens(sequence, enough=wanted))
        while tokens <= 0:
            # Two long prompts can hold the whole pool between them with no decoder left to
            # trigger a preemption; the one in front takes pages from the weakest one behind it.
            victims = [s for s in behind if s.status is SequenceStatus.RUNNING and s.holds_pages]
            if not victims:
                return
            self._preempt(victims[-1], plan)
            tokens = min(wanted, self.cache.coverable_tokens(sequence, enough=wanted))
        try:
            self.cache.reserve(sequence, sequence.num_computed_tokens + tokens)
        except OutOfPages:  # pragma: no cover - coverable_tokens bounds the portion
            return
        plan.spend(sequence, tokens, prefill=True,
                   produces=sequence.num_computed_tokens + tokens == sequence.num_tokens)

    def _admit(self, sequence: Sequence, plan: _StepPlan) -> bool:
        """Admit one waiting sequence with its first portion; False closes admission for the step."""
        if self.slots_in_use + 1 + sequence.fork_slots > self.config.max_running_seqs:
            return False
        reuse = self.cache.attach_prefix(sequence, record=False)
        # The watermark keeps room for the decode steps of running sequences; with nothing
        # running it protects nobody and could refuse the only request forever.
        keep_free = int(self.config.watermark * self.cache.num_blocks) if self._running else 0
        portion = self._portion(sequence, plan)
        tokens = min(portion, self.cache.coverable_tokens(sequence, keep_free, enough=portion))
        tokens = plan.allowed(sequence, tokens)
        if tokens <= 0:
            self.cache.detach_prefix(sequence)
            return False
        try:
            self.cache.reserve(sequence, sequence.num_computed_tokens + tokens)
        except OutOfPages:  # pragma: no cover - coverable_tokens bounds the portion
            self.cache.detach_prefix(sequence)
            return False
        self.cache.record_prefix(reuse)
        self.cache.acquire_state_slot(sequence)
        self._waiting.remove(sequence)
        sequence.status = SequenceStatus.RUNNING
        self._running.append(sequence)
        plan.admitted.append(sequence.seq_id)
        plan.spend(sequence, tokens, prefill=True,
                   produces=sequence.num_computed_tokens + tokens == sequence.num_tokens)
        return True

    @staticmethod
    def _entry(item: ScheduledSequence) -> BatchEntry:
        sequence = item.sequence
        start = sequence.num_computed_tokens
        return BatchEntry(
            seq_id=sequence.seq_id,
            token_ids=tuple(sequence.token_ids[start:start + item.num_tokens]),
            first_position=start,
            block_tables=tuple(table.snapshot() if isinstance(table, PageTable) else tuple(table)
                               for table in sequence.block_tables),
            logits_at=(item.num_tokens - 1,) if item.produces_token else (),
            state_slot=sequence.state_slot,
        )
