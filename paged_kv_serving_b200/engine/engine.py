"""The generation loop: one synchronous ``step()`` per scheduled batch.

A step (reference: src/paged_kv_serving/engine/engine.py:413-465): the scheduler picks a ragged
batch and reserves its pages, preempting if it must; the step function runs it; every entry
that reached the end of its sequence samples one token with the sequence's own generator, newly
filled pages are offered to the prefix cache, windowed pages that fell out of reach are given
back, the remaining samples of an n-way request fork from the prompt's final logits and share
its pages, and finished sequences return what they hold.

The public surface keeps the reference's names (``submit``, ``step``, ``run_until_idle``,
``generate``, ``abort``, ``snapshot``, ``check_invariants``, ``StepOutput``, ``RequestOutput`` ...).
Deadline admission control, entitlements and metrics exporters of the reference are not part
of this engine; the hard request limits are (src/paged_kv_serving/engine/engine.py:306-319).
"""

from __future__ import annotations

import time
from collections.abc import Callable, Iterable
from dataclasses import dataclass, field
from enum import Enum
from pathlib import Path
from typing import Protocol

import numpy as np

from paged_kv_serving_b200.cache.manager import GroupSpec, KVCacheManager, plan_groups
from paged_kv_serving_b200.config.engine_config import EngineConfig
from paged_kv_serving_b200.engine.batch import ExecutionBatch
from paged_kv_serving_b200.engine.scheduler import Scheduler, SchedulerOutput
from paged_kv_serving_b200.engine.sequence import (
    FinishReason, Request, Sequence, SequenceStatus, SloClass, finish_reason_for,
)

__all__ = [
    "AdmissionDecision", "Engine", "EngineExecutor", "RejectionReason", "RequestOutput", "SampleOutput",
    "StepOutput", "TokenEvent",
]


class EngineExecutor(Protocol):
    """What the engine needs from a step function; ``ModelRunner`` implements it. Tests put a
    fake in its place to drive the scheduler without a GPU
    (reference: src/paged_kv_serving/engine/engine.py:64-73)."""

    def execute(self, batch: ExecutionBatch) -> dict[str, np.ndarray]: ...


class RejectionReason(Enum):
    PROMPT_TOO_LONG = "prompt_too_long"
    CONTEXT_TOO_LONG = "context_too_long"
    TOO_MANY_SAMPLES = "too_many_samples"


@dataclass(frozen=True, slots=True)
class AdmissionDecision:
    admitted: bool
    reason: RejectionReason | None = None
    retry_after_seconds: float = 0.0


@dataclass(frozen=True, slots=True)
class TokenEvent:
    request_id: str
    sample_index: int
    token_id: int
    index: int
    finished: bool
    finish_reason: FinishReason | None = None


@dataclass(frozen=True, slots=True)
class SampleOutput:
    sample_index: int
    token_ids: tuple[int, ...]
    finish_reason: FinishReason
    preemptions: int


@dataclass(frozen=True, slots=True)
class RequestOutput:
    request_id: str
    key_id: str
    slo_class: SloClass
    samples: tuple[SampleOutput, ...]
    prompt_tokens: int
    cached_prompt_tokens: int
    arrival_time: float
    first_token_time: float
    finish_time: float
    deadline: float | None = None

    @property
    def ttft(self) -> float:
        return self.first_token_time - self.arrival_time

    @property
    def latency(self) -> float:
        return self.finish_time - self.arrival_time

    @property
    def output_tokens(self) -> int:
        return sum(len(s.token_ids) for s in self.samples)

    @property
    def tpot(self) -> float:
        extra = self.output_tokens - len(self.samples)
        return (self.finish_time - self.first_token_time) / extra if extra > 0 else 0.0

    @property
    def preemptions(self) -> int:
        return sum(s.preemptions for s in self.samples)

    @property
    def met_deadline(self) -> bool | None:
        return None if self.deadline is None else self.finish_time <= self.deadline


@dataclass(frozen=True, slots=True)
class StepOutput:
    iteration: int
    duration: float
    num_batched_tokens: int
    num_prefill_tokens: int
    num_decode_tokens: int
    num_running: int
    queue_depth: int
    tokens: tuple[TokenEvent, ...] = ()
    finished: tuple[RequestOutput, ...] = ()
    preempted: tuple[str, ...] = ()

    @property
    def is_empty(self) -> bool:
        return self.num_batched_tokens == 0


@dataclass(slots=True)
class _RequestState:
    request: Request
    sequences: dict[int, Sequence] = field(default_factory=dict)
    pending_forks: list[Sequence] = field(default_factory=list)
    finished: dict[int, SampleOutput] = field(default_factory=dict)
    first_token_time: float | None = None
    cached_prompt_tokens: int = 0

    @property
    def complete(self) -> bool:
        return len(self.finished) == self.request.n


class Engine:
    """Continuous-batching engine over the paged cache.

    ``model`` is a loaded ``DecoderModel`` or a model folder (loaded in ``config.dtype``). With an
    ``executor`` of its own (a stand-in step function, for tests of the scheduling logic) no GPU
    is touched and ``model`` may be ``None``; token ids then come from ``host_sampler(row, params,
    generator)`` if given, else from the argmax of the rows the executor returns.
    """

    def __init__(self, model=None, config: EngineConfig | None = None, *, executor: EngineExecutor | None = None,
                 clock: Callable[[], float] = time.perf_counter, eos_token_id: int | None = None,
                 prefix_cache_scope: str = "per_key", groups: list[GroupSpec] | None = None,
                 host_sampler: Callable[..., int] | None = None) -> None:
        self.config = config or EngineConfig()
        self.clock = clock
        self.eos_token_id = eos_token_id
        self.host_sampler = host_sampler
        self.runner = None
        self.sampler = None
        store = None
        num_state_slots = 0
        if isinstance(model, (str, Path)):
            from paged_kv_serving_b200.models.decoder import DecoderModel

            model = DecoderModel.from_folder(model, dtype=self.config.dtype)
        self.model = model
        if model is not None and self.config.max_context_tokens > model.layout.max_positions:
            raise ValueError("max_context_tokens exceeds the model's max_seq_len")
        if executor is None:
            if model is None:
                raise ValueError("an engine needs a model or an executor")
            from paged_kv_serving_b200.engine.runner import ModelRunner
            from paged_kv_serving_b200.sampling.sampler import Sampler

            self.runner = ModelRunner(model, num_blocks=self.config.num_blocks, block_size=self.config.block_size,
                                      max_running_seqs=self.config.max_running_seqs)
            self.sampler = Sampler(model.device)
            executor = self.runner
            store = self.runner
            groups = self.runner.groups
            num_state_slots = self.runner.num_state_slots
        elif groups is None:
            if model is not None:
                groups, states = plan_groups(model.layout.cache_entries())
                num_state_slots = self.config.max_running_seqs if states else 0
            else:
                groups = [GroupSpec((0,), 1, 2, None)]
        self.executor: EngineExecutor = executor
        self.cache = KVCacheManager(groups, num_blocks=self.config.num_blocks, block_size=self.config.block_size,
                                    store=store, enable_prefix_cache=self.config.enable_prefix_cache,
                                    prefix_scope=prefix_cache_scope, num_state_slots=num_state_slots)
        self.prefix_cache = self.cache.prefix_cache
        self.scheduler = Scheduler(self.config, self.cache)
        self._requests: dict[str, _RequestState] = {}
        self._iteration = 0
        self.aborted_requests = 0
        self.rejections: dict[str, int] = {}
        self.h2d_bytes_last_step = 0
        self.d2h_bytes_last_step = 0

    # --- introspection -------------------------------------------------------------------

    @property
    def iteration(self) -> int:
        return self._iteration

    @property
    def has_work(self) -> bool:
        return self.scheduler.has_work or any(s.pending_forks for s in self._requests.values())

    @property
    def active_requests(self) -> int:
        return len(self._requests)

    def snapshot(self) -> dict[str, float]:
        return {
            "iteration": float(self._iteration),
            "queue_depth": float(self.scheduler.queue_depth),
            "running": float(self.scheduler.num_running),
            "kv_blocks_used_ratio": self.cache.utilization,
            "prefix_cache_hit_ratio": self.prefix_cache.stats.hit_ratio,
            "preemptions_total": float(self.scheduler.stats.preemptions),
            "aborted_requests_total": float(self.aborted_requests),
        }

    # --- admission -----------------------------------------------------------------------

    def _limit_violation(self, request: Request) -> RejectionReason | None:
        sampling = request.sampling
        if request.prompt_len > self.config.max_prompt_tokens:
            return RejectionReason.PROMPT_TOO_LONG
        if (sampling.max_new_tokens > self.config.max_new_tokens
                or request.prompt_len + sampling.max_new_tokens > self.config.max_context_tokens):
            return RejectionReason.CONTEXT_TOO_LONG
        if request.n > self.config.max_running_seqs:
            return RejectionReason.TOO_MANY_SAMPLES
        return None

    def submit(self, request: Request) -> AdmissionDecision:
        """Check the hard limits and queue the request; refused before any page is taken."""
        if request.request_id in self._requests:
            raise ValueError(f"request {request.request_id} is already in flight")
        violation = self._limit_violation(request)
        if violation is not None:
            self.rejections[violation.value] = self.rejections.get(violation.value, 0) + 1
            return AdmissionDecision(False, violation)
        state = _RequestState(request=request)
        primary = Sequence.from_request(request, 0, num_groups=self.cache.num_groups)
        primary.fork_slots = request.n - 1
        state.sequences[0] = primary
        for index in range(1, request.n):
            child = Sequence.from_request(request, index, num_groups=self.cache.num_groups)
            state.sequences[index] = child
            state.pending_forks.append(child)
        self._requests[request.request_id] = state
        self.scheduler.add(primary)
        return AdmissionDecision(True)

    def abort(self, request_id: str) -> int:
        """Cancel a request and give back everything it holds; returns sequences removed."""
        state = self._requests.pop(request_id, None)
        if state is None:
            return 0
        removed = 0
        now = self.clock()
        for sequence in state.sequences.values():
            if sequence.sample_index in state.finished:
                continue
            self.scheduler.remove(sequence)
            sequence.finish(FinishReason.ABORTED, now)
            removed += 1
        state.pending_forks.clear()
        self.aborted_requests += 1
        return removed

    # --- the loop ------------------------------------------------------------------------

    def step(self) -> StepOutput:
        plan = self.scheduler.schedule()
        if plan.is_empty:
            return StepOutput(self._iteration, 0.0, 0, 0, 0, self.scheduler.num_running, self.scheduler.queue_depth,
                              preempted=plan.preempted)
        self._iteration += 1
        started = self.clock()
        device_logits, host_rows, row_of = self._run(plan)
        events: list[TokenEvent] = []
        producers: list[Sequence] = []
        for item in plan.scheduled:
            sequence = item.sequence
            state = self._requests.get(sequence.request.request_id)
            if state is not None:  # noted while the sequence still holds its pages
                state.cached_prompt_tokens = max(state.cached_prompt_tokens,
                                                 sequence.cached_prefix_blocks * self.config.block_size)
            sequence.num_computed_tokens += item.num_tokens
            self.cache.publish_full_blocks(sequence)
            self.cache.release_behind_window(sequence)
            if item.produces_token:
                producers.append(sequence)
        # forks are created before anything is sampled: every sample of a request draws from the
        # prompt's final logits with its own generator
        samplers: list[tuple[Sequence, int]] = []
        for sequence in producers:
            row = row_of[sequence.seq_id]
            for child in self._fork_pending(sequence):
                samplers.append((child, row))
            samplers.append((sequence, row))
        tokens = self._sample(device_logits, host_rows, samplers)
        now = self.clock()
        duration = now - started
        for (sequence, _), token in zip(samplers, tokens):
            self._emit(sequence, token, now, events)
        finished = self._collect_finished(now)
        return StepOutput(
            iteration=self._iteration,
            duration=duration,
            num_batched_tokens=plan.num_batched_tokens,
            num_prefill_tokens=sum(i.num_tokens for i in plan.scheduled if i.is_prefill),
            num_decode_tokens=sum(i.num_tokens for i in plan.scheduled if not i.is_prefill),
            num_running=self.scheduler.num_running,
            queue_depth=self.scheduler.queue_depth,
            tokens=tuple(events),
            finished=finished,
            preempted=plan.preempted,
        )

    def _run(self, plan: SchedulerOutput):
        """Run the batch; returns ``(device logits or None, host rows or None, seq_id -> row)``."""
        if self.runner is not None and self.executor is self.runner:
            clear = self.cache.state_slots.take_slots_to_clear() if self.cache.state_slots is not None else None
            result = self.runner.step(plan.batch, clear_state_slots=clear)
            self.h2d_bytes_last_step = result.h2d_bytes
            return result.logits, None, {seq_id: i for i, (seq_id, _) in enumerate(result.rows)}
        rows = self.executor.execute(plan.batch)
        names = list(rows)
        return None, [rows[name] for name in names], {name: i for i, name in enumerate(names)}

    def _sample(self, device_logits, host_rows, samplers: list[tuple[Sequence, int]]) -> list[int]:
        if not samplers:
            return []
        params = [s.request.sampling for s, _ in samplers]
        generators = [s.rng for s, _ in samplers]
        if device_logits is not None:
            index = [row for _, row in samplers]
            logits = device_logits
            if index != list(range(device_logits.shape[0])):
                import torch

                logits = device_logits.index_select(0, torch.tensor(index, device=device_logits.device))
            self.h2d_bytes_last_step += 32 * len(samplers)
            ids = self.sampler.sample_on_device(logits, params, generators, status=self.runner.status)
            # the GPU is busy with this step: the host gets the arrays of the next one ready
            self.runner.prepare_next()
            # one copy brings the ids and, behind them, the device's status word: a kernel that
            # recorded a fault (a wait it gave up, an id outside the table) stops generation here
            # instead of letting wrong tokens through
            values = ids.cpu().tolist()
            self.d2h_bytes_last_step = 4 * len(values)
            from paged_kv_serving_b200 import ops

            ops.raise_for_status(values.pop(), self.runner.model.device)
            return [int(t) for t in values]
        # rows of a stand-in executor (tests without a GPU): the caller's sampler, else the argmax
        if self.host_sampler is not None:
            return [int(self.host_sampler(np.asarray(host_rows[row]), p, g))
                    for (_, row), p, g in zip(samplers, params, generators)]
        return [int(np.argmax(host_rows[row])) for _, row in samplers]

    def _fork_pending(self, sequence: Sequence) -> list[Sequence]:
        """The other samples of an n-way request, created when its first sample ends its prompt."""
        state = self._requests.get(sequence.request.request_id)
        if state is None or sequence.sample_index != 0 or sequence.num_output_tokens or not state.pending_forks:
            return []
        children = list(state.pending_forks)
        for child in children:
            self.cache.fork(sequence, child)
            self.scheduler.add_running(child)
        state.pending_forks.clear()
        sequence.fork_slots = 0
        return children

    def _emit(self, sequence: Sequence, token: int, now: float, events: list[TokenEvent]) -> None:
        sequence.append_token(token)
        if sequence.first_token_time is None:
            sequence.first_token_time = now
            state = self._requests.get(sequence.request.request_id)
            if state is not None and state.first_token_time is None:
                state.first_token_time = now
        reason = finish_reason_for(sequence, token, eos_token_id=self.eos_token_id,
                                   max_context_tokens=self.config.max_context_tokens)
        if reason is not None:
            sequence.finish(reason, now)
        events.append(TokenEvent(sequence.request.request_id, sequence.sample_index, token,
                                 sequence.num_output_tokens - 1, reason is not None, reason))

    def _collect_finished(self, now: float) -> tuple[RequestOutput, ...]:
        completed = []
        for sequence in self.scheduler.drop_finished():
            state = self._requests.get(sequence.request.request_id)
            if state is None:  # pragma: no cover - aborted between scheduling and collection
                continue
            state.finished[sequence.sample_index] = SampleOutput(
                sequence.sample_index, tuple(sequence.output_token_ids),
                sequence.finish_reason or FinishReason.LENGTH, sequence.preemption_count)
            if state.complete:
                request = state.request
                del self._requests[request.request_id]
                completed.append(RequestOutput(
                    request_id=request.request_id, key_id=request.key_id, slo_class=request.slo_class,
                    samples=tuple(state.finished[i] for i in sorted(state.finished)),
                    prompt_tokens=request.prompt_len, cached_prompt_tokens=state.cached_prompt_tokens,
                    arrival_time=request.arrival_time,
                    first_token_time=state.first_token_time if state.first_token_time is not None else now,
                    finish_time=now, deadline=request.deadline))
        return tuple(completed)

    # --- convenience ---------------------------------------------------------------------

    def run_until_idle(self, max_iterations: int = 100_000) -> list[RequestOutput]:
        """Step until nothing is left. An empty batch while work is queued is a bug, not a state
        to wait out, and is raised (reference: src/paged_kv_serving/engine/engine.py:579-599)."""
        outputs: list[RequestOutput] = []
        for _ in range(max_iterations):
            if not self.has_work:
                return outputs
            step = self.step()
            outputs.extend(step.finished)
            if step.is_empty:
                if not self.scheduler.has_work:
                    return outputs
                raise RuntimeError(f"the scheduler produced an empty batch with {self.scheduler.num_running} "
                                   f"running and {self.scheduler.queue_depth} waiting sequences")
        raise RuntimeError(f"engine did not drain within {max_iterations} iterations")

    def generate(self, requests: Iterable[Request]) -> list[RequestOutput]:
        """Submit every request, then drain; refused requests do not appear in the result."""
        for request in requests:
            self.submit(request)
        return self.run_until_idle()

    def flush_prefix_cache(self) -> int:
        return self.prefix_cache.flush()

    def check_invariants(self) -> None:
        self.cache.check_invariants()

    def live_sequences(self) -> tuple[Sequence, ...]:
        return (*self.scheduler.running, *self.scheduler.waiting)

    def sequence_status(self, request_id: str, sample_index: int = 0) -> SequenceStatus | None:
        state = self._requests.get(request_id)
        if state is None:
            return None
        sequence = state.sequences.get(sample_index)
        return sequence.status if sequence is not None else None
