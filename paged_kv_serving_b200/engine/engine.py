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


#: What stands in a sequence's tokens for a token that was sampled on the device and has not been
#: read back yet. Any valid id would do: the step that runs it reads the real id on the device.
STAND_IN_TOKEN = 0


@dataclass(slots=True)
class _Flight:
    """A step that has been launched: what it ran, who sampled from it, and where its tokens
    will be found. ``drawn`` is ``(sequence, place of the stand-in in its tokens)`` per sampled
    token, in the order of the sampler's rows."""

    iteration: int
    started: float
    plan: SchedulerOutput
    drawn: list[tuple[Sequence, int]]
    tokens: list[int] | None = None          # known at once (a stand-in executor on the host)
    host_ids: object = None                  # pinned int32 buffer the device ids are copied into
    ready: object = None                     # CUDA event recorded behind that copy


class Engine:
    """Continuous-batching engine over the paged cache.

    ``model`` is a loaded ``DecoderModel`` or a model folder (loaded in ``config.dtype``). With an
    ``executor`` of its own (a stand-in step function, for tests of the scheduling logic) no GPU
    is touched and ``model`` may be ``None``; token ids then come from ``host_sampler(row, params,
    generator)`` if given, else from the argmax of the rows the executor returns.

    A step has two halves. *Launch*: the scheduler's batch goes to the step function, the rows
    that end a sequence's tokens are sampled, and each sampled token takes its place in the
    sequence as a stand-in. *Settle*: the sampled ids arrive, replace the stand-ins, and stop
    tokens, finished requests and outputs are dealt with. With ``overlap`` (the default on the
    GPU) ``step()`` launches step k and then settles step k-1, so that the host's share of a step
    (scheduling, bookkeeping, reading ids back) runs while the GPU computes: a decoded token
    enters the next step on the device (``ModelRunner.sampled_ids``), a sequence that is complete
    by its token count leaves the batch at launch, and a stop token is noticed one step late
    (the one token computed in vain is dropped). ``StepOutput.tokens`` of a call are then the
    tokens of the step launched by the call before. Without ``overlap`` both halves of a step
    happen in the same call.
    """

    def __init__(self, model=None, config: EngineConfig | None = None, *, executor: EngineExecutor | None = None,
                 clock: Callable[[], float] = time.perf_counter, eos_token_id: int | None = None,
                 prefix_cache_scope: str = "per_key", groups: list[GroupSpec] | None = None,
                 host_sampler: Callable[..., int] | None = None, overlap: bool | None = None) -> None:
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
        on_device = self.runner is not None and self.executor is self.runner
        if overlap and not on_device:
            raise ValueError("steps overlap only with the engine's own step function on the GPU")
        self.overlap = on_device if overlap is None else bool(overlap)
        self.cache = KVCacheManager(groups, num_blocks=self.config.num_blocks, block_size=self.config.block_size,
                                    store=store, enable_prefix_cache=self.config.enable_prefix_cache,
                                    prefix_scope=prefix_cache_scope, num_state_slots=num_state_slots)
        self.prefix_cache = self.cache.prefix_cache
        self.scheduler = Scheduler(self.config, self.cache)
        self._requests: dict[str, _RequestState] = {}
        self._iteration = 0
        self._flight: _Flight | None = None
        self._fed_back: dict[str, int] = {}      # sequence id -> place of its newest id in the runner's buffer
        self._host_ids: list = []                # two pinned buffers, used in turn
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
        return (self.scheduler.has_work or self._flight is not None
                or any(s.pending_forks for s in self._requests.values()))

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
        """The hard limits of the reference (src/paged_kv_serving/engine/engine.py:306-319)."""
        limits = self.config
        wanted = request.sampling.max_new_tokens
        if request.prompt_len > limits.max_prompt_tokens:
            return RejectionReason.PROMPT_TOO_LONG
        if wanted > limits.max_new_tokens or request.prompt_len + wanted > limits.max_context_tokens:
            return RejectionReason.CONTEXT_TOO_LONG
        if request.n > limits.max_running_seqs:
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
        samples = [Sequence.from_request(request, index, num_groups=self.cache.num_groups) for index in range(request.n)]
        first, others = samples[0], samples[1:]
        first.fork_slots = len(others)           # running slots kept for the samples still to fork
        self._requests[request.request_id] = _RequestState(
            request=request, sequences={s.sample_index: s for s in samples}, pending_forks=list(others))
        self.scheduler.add(first)
        return AdmissionDecision(True)

    def abort(self, request_id: str) -> int:
        """Cancel a request; everything it holds goes back. Returns how many of its samples were
        still unfinished."""
        state = self._requests.pop(request_id, None)
        if state is None:
            return 0
        when = self.clock()
        live = [s for index, s in state.sequences.items() if index not in state.finished]
        for sequence in live:
            self.scheduler.remove(sequence)           # running, waiting, or not yet forked: all the same
            sequence.finish(FinishReason.ABORTED, when)
            self._fed_back.pop(sequence.seq_id, None)
        state.pending_forks.clear()
        self.aborted_requests += 1
        return len(live)

    # --- the loop ------------------------------------------------------------------------

    def step(self) -> StepOutput:
        """Launch the next step and settle one: the same step, or with ``overlap`` the one the
        previous call launched."""
        plan = self.scheduler.schedule()
        launched = self._launch(plan) if not plan.is_empty else None
        if self.overlap:
            settling, self._flight = self._flight, launched
        else:
            settling = launched
        events: list[TokenEvent] = []
        finished: tuple[RequestOutput, ...] = ()
        duration = 0.0
        if settling is not None:
            finished = self._settle(settling, events)
            duration = self.clock() - settling.started
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

    def _launch(self, plan: SchedulerOutput) -> _Flight:
        """First half of a step: run the batch, sample, and give every sampled token its place."""
        self._iteration += 1
        flight = _Flight(self._iteration, self.clock(), plan, [])
        device_logits, host_rows, row_of = self._run(plan)
        enders: list[Sequence] = []
        block_size = self.config.block_size
        for item in plan.scheduled:
            sequence = item.sequence
            state = self._requests.get(sequence.request.request_id)
            if state is not None:  # noted while the sequence still holds its pages
                state.cached_prompt_tokens = max(state.cached_prompt_tokens,
                                                 sequence.cached_prefix_blocks * self.config.block_size)
            sequence.num_computed_tokens += item.num_tokens
            if sequence.num_computed_tokens // block_size > len(sequence.block_hashes):
                self.cache.publish_full_blocks(sequence)      # a page was filled
            self.cache.release_behind_window(sequence)
            if item.produces_token:
                enders.append(sequence)
        # forks are created before anything is sampled: every sample of a request draws from the
        # prompt's final logits with its own generator
        samplers: list[tuple[Sequence, int]] = []
        for sequence in enders:
            row = row_of[sequence.seq_id]
            samplers.extend((child, row) for child in self._fork_pending(sequence))
            samplers.append((sequence, row))
        self._sample(flight, device_logits, host_rows, samplers)
        self._fed_back = {}
        for place, (sequence, _) in enumerate(samplers):
            sequence.append_token(STAND_IN_TOKEN)
            sequence.num_unsettled_tokens += 1
            flight.drawn.append((sequence, sequence.num_tokens - 1))
            if flight.tokens is None:
                self._fed_back[sequence.seq_id] = place
            # a sequence that this token completes, whatever it turns out to be, runs no further
            # step: it leaves the batch now and its pages go back (work already launched is
            # ordered before anything that takes them)
            if self._length_reason(sequence) is not None:
                self.scheduler.remove(sequence)
        return flight

    def _run(self, plan: SchedulerOutput):
        """Run the batch; returns ``(device logits or None, host rows or None, seq_id -> row)``."""
        if self.runner is not None and self.executor is self.runner:
            clear = self.cache.state_slots.take_slots_to_clear() if self.cache.state_slots is not None else None
            result = self.runner.step(plan.batch, clear_state_slots=clear, feedback=self._fed_back or None)
            self.h2d_bytes_last_step = result.h2d_bytes
            return result.logits, None, {seq_id: i for i, (seq_id, _) in enumerate(result.rows)}
        rows = self.executor.execute(plan.batch)
        names = list(rows)
        return None, [rows[name] for name in names], {name: i for i, name in enumerate(names)}

    def _sample(self, flight: _Flight, device_logits, host_rows, samplers: list[tuple[Sequence, int]]) -> None:
        """Sample one token per entry of ``samplers``: on the device (the ids stay there for the
        next step and are copied to pinned host memory behind an event) or, for a stand-in
        executor's host rows, here and now."""
        if not samplers:
            flight.tokens = []
            return
        params = [s.request.sampling for s, _ in samplers]
        generators = [s.rng for s, _ in samplers]
        if device_logits is None:
            # rows of a stand-in executor (tests without a GPU): the caller's sampler, else the argmax
            if self.host_sampler is not None:
                flight.tokens = [int(self.host_sampler(np.asarray(host_rows[row]), p, g))
                                 for (_, row), p, g in zip(samplers, params, generators)]
            else:
                flight.tokens = [int(np.argmax(host_rows[row])) for _, row in samplers]
            return
        import torch

        index = [row for _, row in samplers]
        logits = device_logits
        if index != list(range(device_logits.shape[0])):
            logits = device_logits.index_select(0, torch.tensor(index, device=device_logits.device))
        self.h2d_bytes_last_step += 32 * len(samplers)
        # the ids land in the runner's buffer, where the next step's embedding lookup reads them,
        # with the device's status word behind them
        ids = self.sampler.sample_on_device(logits, params, generators, status=self.runner.status,
                                            out=self.runner.sampled_ids)
        if not self._host_ids:
            size = self.runner.sampled_ids.numel()
            self._host_ids = [torch.empty((size,), dtype=torch.int32, pin_memory=True) for _ in range(2)]
        flight.host_ids = self._host_ids[flight.iteration % 2][:ids.numel()]
        flight.host_ids.copy_(ids, non_blocking=True)
        flight.ready = torch.cuda.Event()
        flight.ready.record()
        self.d2h_bytes_last_step = 4 * ids.numel()
        # the GPU is busy with this step: the host gets the arrays of the next one ready
        self.runner.prepare_next()

    def _settle(self, flight: _Flight, events: list[TokenEvent]) -> tuple[RequestOutput, ...]:
        """Second half of a step: the sampled ids replace their stand-ins; stop tokens, finished
        samples and complete requests are dealt with."""
        tokens = flight.tokens
        if tokens is None:
            from paged_kv_serving_b200 import ops

            flight.ready.synchronize()
            values = flight.host_ids.tolist()
            # behind the ids: the device's status word. A kernel that recorded a fault (a wait it
            # gave up, an id outside the table) stops generation here instead of letting wrong
            # tokens through: the requests with tokens in this step, and in the step launched
            # after it, are aborted (nothing they computed since can be trusted), the rest of
            # the engine stays as it is, and the fault is raised.
            if values[-1]:
                suspects = [sequence for sequence, _ in flight.drawn]
                if self._flight is not None and self._flight is not flight:
                    suspects += [sequence for sequence, _ in self._flight.drawn]
                    self._flight = None
                for request_id in {sequence.request.request_id for sequence in suspects}:
                    self.abort(request_id)
            ops.raise_for_status(values.pop(), self.runner.model.device)
            tokens = values
        now = self.clock()
        completed: list[RequestOutput] = []
        for (sequence, place), token in zip(flight.drawn, tokens):
            if sequence.is_finished:       # aborted, or stopped by a token of the step before
                continue
            sequence.token_ids[place] = int(token)
            sequence.num_unsettled_tokens -= 1
            state = self._requests.get(sequence.request.request_id)
            if sequence.first_token_time is None:
                sequence.first_token_time = now
                if state is not None and state.first_token_time is None:
                    state.first_token_time = now
            produced = place - sequence.request.prompt_len + 1
            reason = finish_reason_for(sequence, int(token), eos_token_id=self.eos_token_id,
                                       max_context_tokens=self.config.max_context_tokens, num_output_tokens=produced)
            events.append(TokenEvent(sequence.request.request_id, sequence.sample_index, int(token), produced - 1,
                                     reason is not None, reason))
            if reason is None:
                continue
            # a stop token may come while the sequence already runs its next step: what that step
            # samples is dropped with the stand-in that waits for it
            del sequence.token_ids[place + 1:]
            sequence.num_unsettled_tokens = 0
            self._fed_back.pop(sequence.seq_id, None)
            self.scheduler.remove(sequence)
            sequence.finish(reason, now)
            output = self._record_finished(sequence, state, now)
            if output is not None:
                completed.append(output)
        return tuple(completed)

    def _length_reason(self, sequence: Sequence) -> FinishReason | None:
        """Why the sequence is complete by its counts alone (no token needed), or ``None``."""
        return finish_reason_for(sequence, None, eos_token_id=None, max_context_tokens=self.config.max_context_tokens)

    def _record_finished(self, sequence: Sequence, state: _RequestState | None, now: float) -> RequestOutput | None:
        """Note a finished sample; the request's output once every sample is in."""
        if state is None:                   # the request was aborted meanwhile
            return None
        state.finished[sequence.sample_index] = SampleOutput(
            sequence.sample_index, tuple(sequence.output_token_ids),
            sequence.finish_reason or FinishReason.LENGTH, sequence.preemption_count)
        if not state.complete:
            return None
        request = state.request
        del self._requests[request.request_id]
        return RequestOutput(
            request_id=request.request_id, key_id=request.key_id, slo_class=request.slo_class,
            samples=tuple(state.finished[i] for i in sorted(state.finished)),
            prompt_tokens=request.prompt_len, cached_prompt_tokens=state.cached_prompt_tokens,
            arrival_time=request.arrival_time,
            first_token_time=state.first_token_time if state.first_token_time is not None else now,
            finish_time=now, deadline=request.deadline)

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

    # --- convenience ---------------------------------------------------------------------

    def run_until_idle(self, max_iterations: int = 100_000) -> list[RequestOutput]:
        """Call ``step`` until no work is left; returns the outputs in the order they completed.
        A call that neither ran nor settled anything while sequences are still queued means the
        scheduler is stuck, which is a fault to report, not a state to wait out
        (reference: src/paged_kv_serving/engine/engine.py:579-599)."""
        outputs: list[RequestOutput] = []
        calls = 0
        while self.has_work:
            if calls == max_iterations:
                raise RuntimeError(f"the engine still has work after {max_iterations} steps")
            calls += 1
            step = self.step()
            outputs += step.finished
            if step.is_empty and not step.tokens and self.scheduler.has_work:
                raise RuntimeError(f"nothing could be scheduled although {self.scheduler.num_running} sequences "
                                   f"run and {self.scheduler.queue_depth} wait")
        return outputs

    def generate(self, requests: Iterable[Request]) -> list[RequestOutput]:
        """Queue the requests and run to the end. A request beyond the hard limits is left out of
        the result (``submit`` says why when called directly)."""
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
