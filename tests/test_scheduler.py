"""The scheduler's decisions and the generation loop, driven by a stand-in step function (no GPU).

The stand-in returns one-hot logits that depend only on a sequence's last token and its context
length, so a run's tokens are a pure function of the prompts: whatever the scheduler does
(portions, mixing, preemption, prefix reuse, forks) must leave them unchanged.
"""

from __future__ import annotations

import numpy as np
import pytest

import plain_model
from paged_kv_serving_b200.cache import GroupSpec, KVCacheManager, RecordingPageStore
from paged_kv_serving_b200.config import EngineConfig
from paged_kv_serving_b200.engine.engine import Engine, RejectionReason
from paged_kv_serving_b200.engine.scheduler import Scheduler
from paged_kv_serving_b200.engine.sequence import (
    FinishReason, Request, SamplingParams, Sequence, SequenceStatus, SloClass,
)

VOCAB = 50


class StandInExecutor:
    def __init__(self):
        self.batches = []

    def execute(self, batch):
        self.batches.append(batch)
        rows = {}
        for entry in batch.entries:
            for table in entry.block_tables:
                assert len(table) * BLOCK >= entry.context_len
            if entry.logits_at:
                place = entry.logits_at[-1]
                row = np.zeros(VOCAB, dtype=np.float32)
                row[(entry.token_ids[place] * 7 + entry.first_position + place + 1) % VOCAB] = 1.0
                rows[entry.seq_id] = row
        return rows


BLOCK = 4


def expected_tokens(prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append((tokens[-1] * 7 + len(tokens)) % VOCAB)
    return tokens[len(prompt):]


def make_config(**overrides):
    base = dict(block_size=BLOCK, num_blocks=32, max_batched_tokens=8, max_running_seqs=4, max_prompt_tokens=64,
                max_new_tokens=16, max_context_tokens=80, enable_prefix_cache=True, watermark=0.0)
    base.update(overrides)
    return EngineConfig(**base)


def make_scheduler(**overrides):
    config = make_config(**overrides)
    cache = KVCacheManager([GroupSpec((0,), 1, 2, None)], num_blocks=config.num_blocks, block_size=config.block_size,
                           store=RecordingPageStore(), enable_prefix_cache=config.enable_prefix_cache)
    return Scheduler(config, cache), cache


def seq(name, prompt_len, max_new=4, slo=SloClass.INTERACTIVE, deadline=None, base=0, n=1):
    request = Request(request_id=name, prompt_token_ids=tuple((base + i) % VOCAB for i in range(prompt_len)),
                      sampling=SamplingParams(max_new_tokens=max_new), slo_class=slo, deadline_seconds=deadline, n=n)
    return Sequence.from_request(request, 0)


def advance(scheduler, output, token=1):
    """What the engine does after a step, without a model."""
    for item in output.scheduled:
        item.sequence.num_computed_tokens += item.num_tokens
        scheduler.cache.publish_full_blocks(item.sequence)
        if item.produces_token:
            item.sequence.append_token(token)


def test_a_prompt_is_cut_into_portions_and_only_the_last_produces():
    scheduler, _ = make_scheduler()
    s = seq("a", 20)
    scheduler.add(s)
    sizes, produces = [], []
    for _ in range(3):
        out = scheduler.schedule()
        sizes.append(out.scheduled[0].num_tokens)
        produces.append(out.scheduled[0].produces_token)
        assert out.batch.entries[0].logits_at == ((sizes[-1] - 1,) if produces[-1] else ())
        advance(scheduler, out)
    assert sizes == [8, 8, 4] and produces == [False, False, True]
    out = scheduler.schedule()
    assert [(i.num_tokens, i.is_prefill) for i in out.scheduled] == [(1, False)]
    assert out.batch.entries[0].first_position == 20


def test_a_one_token_prompt_is_a_prefill_of_one():
    scheduler, _ = make_scheduler()
    scheduler.add(seq("a", 1))
    out = scheduler.schedule()
    assert [(i.num_tokens, i.is_prefill, i.produces_token) for i in out.scheduled] == [(1, True, True)]


def test_decoding_sequences_go_first_and_prompts_share_what_is_left():
    scheduler, _ = make_scheduler()
    a, b = seq("a", 3), seq("b", 3, base=10)
    scheduler.add(a); scheduler.add(b)
    advance(scheduler, scheduler.schedule())
    scheduler.add(seq("long", 30, base=20))
    out = scheduler.schedule()
    assert [(i.sequence.seq_id, i.num_tokens, i.is_prefill) for i in out.scheduled] == \
        [("a#0", 1, False), ("b#0", 1, False), ("long#0", 6, True)]
    assert scheduler.stats.decode_tokens == 2 and scheduler.stats.prefill_tokens == 12


def test_order_is_class_then_deadline_then_arrival():
    scheduler, _ = make_scheduler(max_batched_tokens=64, max_running_seqs=8)
    batch = seq("batch", 4, slo=SloClass.BATCH)
    late = seq("late", 4, deadline=9.0)
    none = seq("none", 4)
    soon = seq("soon", 4, deadline=1.0)
    for s in (batch, late, none, soon):
        scheduler.add(s)
    out = scheduler.schedule()
    assert [i.sequence.seq_id for i in out.scheduled] == ["soon#0", "late#0", "none#0", "batch#0"]


def test_running_cap_counts_fork_slots_and_closes_admission():
    scheduler, _ = make_scheduler(max_batched_tokens=64, max_running_seqs=3)
    wide = seq("wide", 4, n=3)
    wide.fork_slots = 2
    other = seq("other", 4)
    scheduler.add(wide); scheduler.add(other)
    out = scheduler.schedule()
    assert out.admitted == ("wide#0",) and scheduler.queue_depth == 1 and scheduler.slots_in_use == 3


def test_lower_class_prefill_allowance():
    scheduler, _ = make_scheduler(max_batched_tokens=16, lower_class_prefill_share=0.25)
    scheduler.add(seq("interactive", 6))
    scheduler.add(seq("batch", 30, slo=SloClass.BATCH))
    out = scheduler.schedule()
    assert [(i.sequence.seq_id, i.num_tokens) for i in out.scheduled] == [("interactive#0", 6), ("batch#0", 4)]


def test_max_prefill_chunk_caps_one_sequence_portion():
    scheduler, _ = make_scheduler(max_batched_tokens=32, max_prefill_chunk=5)
    scheduler.add(seq("a", 12)); scheduler.add(seq("b", 3, base=9))
    out = scheduler.schedule()
    assert [(i.sequence.seq_id, i.num_tokens) for i in out.scheduled] == [("a#0", 5), ("b#0", 3)]


def test_watermark_holds_back_admission_only_while_something_runs():
    scheduler, cache = make_scheduler(num_blocks=20, max_batched_tokens=64, watermark=0.5, max_context_tokens=80)
    scheduler.add(seq("first", 60))
    out = scheduler.schedule()
    assert out.scheduled[0].num_tokens == 60            # nothing runs: the watermark protects nobody
    advance(scheduler, out)
    scheduler.add(seq("second", 30, base=5))
    out = scheduler.schedule()
    assert out.admitted == () and scheduler.queue_depth == 1
    assert not scheduler.waiting[0].holds_pages          # a refused waiter keeps nothing


def test_decoder_without_a_page_preempts_the_weakest_and_admits_nobody():
    scheduler, cache = make_scheduler(num_blocks=4, max_batched_tokens=16, max_context_tokens=16,
                                      max_prompt_tokens=8, max_new_tokens=8)
    strong, weak = seq("strong", 8), seq("weak", 8, base=20)
    scheduler.add(strong); scheduler.add(weak)
    advance(scheduler, scheduler.schedule())              # both prompts computed: the pool is full
    scheduler.add(seq("newcomer", 2, base=40))
    out = scheduler.schedule()
    assert out.preempted == ("weak#0",) and out.admitted == ()
    assert [i.sequence.seq_id for i in out.scheduled] == ["strong#0"]
    assert weak.status is SequenceStatus.PREEMPTED and weak.num_computed_tokens == 0 and not weak.holds_pages
    assert weak.num_tokens == 9 and weak.preemption_count == 1     # its sampled token is kept
    cache.check_invariants()


def test_a_lone_decoder_preempts_itself_and_restarts():
    scheduler, cache = make_scheduler(num_blocks=2, max_batched_tokens=16, max_context_tokens=8,
                                      max_prompt_tokens=6, max_new_tokens=2, enable_prefix_cache=False)
    s = seq("solo", 8)
    other = seq("other", 4, base=30)
    scheduler.add(s)
    advance(scheduler, scheduler.schedule())
    hog = cache.allocators[0]
    assert hog.num_free == 0
    out = scheduler.schedule()                            # needs a third page, nobody else to take it from
    assert out.preempted == ("solo#0",) and out.is_empty
    out = scheduler.schedule()                            # next step recomputes it from position zero
    assert out.scheduled and out.scheduled[0].sequence is s and out.batch.entries[0].first_position == 0
    del other


def test_prefill_that_cannot_get_a_page_preempts_a_prefill_behind_it():
    scheduler, cache = make_scheduler(num_blocks=8, max_batched_tokens=16, max_context_tokens=32,
                                      max_prompt_tokens=28, max_new_tokens=4, enable_prefix_cache=False)
    front, back = seq("front", 28), seq("back", 28, base=7)
    scheduler.add(front); scheduler.add(back)
    advance(scheduler, scheduler.schedule())              # 16 tokens of front
    advance(scheduler, scheduler.schedule())              # 12 of front... and back gets what is left
    while front.num_uncomputed_tokens > 1 and not scheduler.stats.preemptions:
        advance(scheduler, scheduler.schedule())
    cache.check_invariants()
    assert front.num_computed_tokens > 0


def test_engine_tokens_do_not_depend_on_scheduling(tmp_path):
    prompts = [[(3 * i + j) % VOCAB for j in range(n)] for i, n in enumerate([5, 9, 17, 1, 30, 12])]

    def run(**overrides):
        executor = StandInExecutor()
        engine = Engine(None, make_config(**overrides), executor=executor)
        outputs = engine.generate(
            Request(f"r{i}", tuple(p), SamplingParams(max_new_tokens=6)) for i, p in enumerate(prompts))
        engine.check_invariants()
        engine.flush_prefix_cache()
        assert engine.cache.num_free_blocks == engine.config.num_blocks
        return {o.request_id: o for o in outputs}, engine

    want = {f"r{i}": tuple(expected_tokens(p, 6)) for i, p in enumerate(prompts)}
    roomy, _ = run(num_blocks=64, max_batched_tokens=64)
    cramped, engine = run(num_blocks=12, max_batched_tokens=8, max_prompt_tokens=32, max_new_tokens=8,
                          max_context_tokens=40)
    for outputs in (roomy, cramped):
        assert {k: v.samples[0].token_ids for k, v in outputs.items()} == want
        assert all(v.samples[0].finish_reason is FinishReason.LENGTH for v in outputs.values())
    assert engine.scheduler.stats.preemptions > 0, "the cramped scenario must preempt"
    assert sum(o.preemptions for o in cramped.values()) == engine.scheduler.stats.preemptions


def test_engine_never_steps_empty_while_work_is_queued():
    rng = np.random.default_rng(0)
    for trial in range(150):
        config = make_config(num_blocks=int(rng.integers(10, 20)), max_batched_tokens=int(rng.integers(2, 24)),
                             max_running_seqs=int(rng.integers(1, 6)), max_prompt_tokens=30, max_new_tokens=10,
                             max_context_tokens=40, watermark=float(rng.choice([0.0, 0.1, 0.3])),
                             enable_prefix_cache=bool(rng.integers(0, 2)))
        engine = Engine(None, config, executor=StandInExecutor())
        requests = []
        for i in range(int(rng.integers(1, 8))):
            shared = [1, 2, 3, 4, 5, 6, 7, 8] if rng.integers(0, 2) else []
            prompt = shared + [int(t) for t in rng.integers(0, VOCAB, size=int(rng.integers(1, 20)))]
            requests.append(Request(f"t{trial}r{i}", tuple(prompt), SamplingParams(max_new_tokens=int(rng.integers(1, 10))),
                                    n=int(rng.choice([1, 1, 2])) if config.max_running_seqs >= 2 else 1))
        for request in requests:
            assert engine.submit(request).admitted
        outputs = []
        for _ in range(2000):
            if not engine.has_work:
                break
            step = engine.step()
            assert not step.is_empty or step.preempted, "an empty step while work is queued"
            outputs.extend(step.finished)
            engine.check_invariants()
        assert not engine.has_work and len(outputs) == len(requests)
        for output, request in zip(sorted(outputs, key=lambda o: o.request_id), sorted(requests, key=lambda r: r.request_id)):
            for sample in output.samples:
                assert sample.token_ids == tuple(expected_tokens(request.prompt_token_ids, request.sampling.max_new_tokens))


def test_prefix_cache_hit_is_counted_and_saves_prefill():
    executor = StandInExecutor()
    engine = Engine(None, make_config(max_batched_tokens=64), executor=executor)
    shared = list(range(16))
    engine.generate([Request("first", tuple(shared + [20, 21]), SamplingParams(max_new_tokens=2))])
    before = engine.scheduler.stats.prefill_tokens
    out = engine.generate([Request("second", tuple(shared + [30, 31, 32]), SamplingParams(max_new_tokens=2))])
    assert out[0].cached_prompt_tokens == 16
    assert engine.scheduler.stats.prefill_tokens - before == 3
    assert engine.prefix_cache.stats.hit_blocks == 4
    other_key = engine.generate([Request("third", tuple(shared + [1]), SamplingParams(max_new_tokens=1), key_id="b")])
    assert other_key[0].cached_prompt_tokens == 0


def test_n_way_request_forks_from_the_prompt_and_shares_pages():
    executor = StandInExecutor()
    engine = Engine(None, make_config(max_batched_tokens=64), executor=executor,
                    host_sampler=lambda row, params, rng: plain_model.sample_token(row * 3, params.temperature,
                                                                                   params.top_p, float(rng.random())))
    request = Request("multi", tuple(range(10)), SamplingParams(max_new_tokens=5, temperature=1.0, seed=4), n=3)
    engine.submit(request)
    engine.step()
    assert engine.scheduler.num_running == 3
    tables = [s.block_table for s in engine.scheduler.running]
    assert tables[0][:2] == tables[1][:2] == tables[2][:2]
    outputs = engine.run_until_idle()
    assert len(outputs) == 1 and len(outputs[0].samples) == 3
    again = Engine(None, make_config(max_batched_tokens=7, num_blocks=21), executor=StandInExecutor(),
                   host_sampler=engine.host_sampler).generate([request])
    assert [s.token_ids for s in again[0].samples] == [s.token_ids for s in outputs[0].samples]
    engine.check_invariants()


def test_hard_limits_and_finish_reasons():
    engine = Engine(None, make_config(), executor=StandInExecutor(), eos_token_id=expected_tokens([3, 4], 2)[1])
    assert engine.submit(Request("long", tuple(range(65)))).reason is RejectionReason.PROMPT_TOO_LONG
    assert engine.submit(Request("new", (1,), SamplingParams(max_new_tokens=17))).reason is RejectionReason.CONTEXT_TOO_LONG
    assert engine.submit(Request("n", (1,), SamplingParams(max_new_tokens=2), n=5)).reason is RejectionReason.TOO_MANY_SAMPLES
    assert engine.rejections == {"prompt_too_long": 1, "context_too_long": 1, "too_many_samples": 1}
    outputs = engine.generate([Request("stop", (3, 4), SamplingParams(max_new_tokens=8)),
                               Request("go-on", (3, 4), SamplingParams(max_new_tokens=3, ignore_eos=True), key_id="k2")])
    by_id = {o.request_id: o.samples[0] for o in outputs}
    assert by_id["stop"].finish_reason is FinishReason.STOP and len(by_id["stop"].token_ids) == 2
    assert by_id["go-on"].finish_reason is FinishReason.LENGTH and len(by_id["go-on"].token_ids) == 3
    small = SamplingParams(max_new_tokens=2)
    assert engine.submit(Request("dup", (1,), small)).admitted
    with pytest.raises(ValueError, match="already in flight"):
        engine.submit(Request("dup", (1,), small))


def test_abort_gives_everything_back():
    engine = Engine(None, make_config(), executor=StandInExecutor())
    engine.submit(Request("a", tuple(range(20)), SamplingParams(max_new_tokens=8)))
    engine.submit(Request("b", tuple(range(5, 15)), SamplingParams(max_new_tokens=8)))
    engine.step(); engine.step()
    assert engine.abort("a") == 1 and engine.abort("a") == 0
    outputs = engine.run_until_idle()
    assert [o.request_id for o in outputs] == ["b"]
    engine.flush_prefix_cache()
    engine.check_invariants()
    assert engine.cache.num_free_blocks == engine.config.num_blocks


def test_step_arrays_are_packed_once_and_can_be_patched_before_they_are_sent():
    """The integer arrays of a step: every array starts on a 16-byte boundary of one buffer; a
    step prepared ahead is staged, its token ids patched when they are known, then sent."""
    import torch

    from paged_kv_serving_b200.parts.base import IntArena

    arena = IntArena()
    arena.add("token_ids", [0, 0, 0])
    arena.add("positions", [7, 8, 9])
    arena.add("table", np.arange(10).reshape(2, 5))
    assert arena.signature() == (("token_ids", (3,)), ("positions", (3,)), ("table", (2, 5)))
    assert arena.total_ints() == 4 + 4 + 12
    arena.stage()
    arena.patch("token_ids", [5, 6, 7])
    with pytest.raises(ValueError):
        arena.patch("token_ids", [1, 2])
    target = torch.full((arena.total_ints(),), -1, dtype=torch.int32)
    arena.upload(torch.device("cpu"), into=target)
    assert target[:3].tolist() == [5, 6, 7] and target[4:7].tolist() == [7, 8, 9]
    assert arena["table"].tolist() == np.arange(10).reshape(2, 5).tolist()
    assert arena.host("token_ids").tolist() == [5, 6, 7] and arena.bytes_uploaded == 80
    with pytest.raises(RuntimeError):
        arena.patch("token_ids", [1, 2, 3])     # already sent
    with pytest.raises(RuntimeError):
        arena.add("more", [1])


def test_even_shares_decode_kernel_is_chosen_only_when_a_round_of_blocks_would_be_nearly_empty():
    import torch

    from paged_kv_serving_b200.parts import attention
    from paged_kv_serving_b200.parts.position import RotaryEncoding

    def part(n_kv):
        return attention.PagedAttention(width=64 * n_kv, n_heads=n_kv, n_kv_heads=n_kv, head_dim=64,
                                        position=RotaryEncoding(64, 10000.0, 128))

    saved = attention._sm_count
    attention._sm_count = lambda device: 148
    try:
        cpu = torch.device("cpu")
        assert not part(8)._flat_pays(8, cpu)        # 64 pairs on 296 places: one round
        assert not part(8)._flat_pays(64, cpu)       # 512 pairs: 1.7 rounds, the second one well filled
        assert part(40)._flat_pays(8, cpu)           # 320 pairs: the second round holds 24 blocks
        assert not part(40)._flat_pays(64, cpu)      # 2,560 pairs: 8.6 rounds
        forced = part(8)
        forced.FLAT_DECODE = "always"
        assert forced._flat_pays(1, cpu)
        forced.FLAT_DECODE = "never"
        assert not forced._flat_pays(1000, cpu)
    finally:
        attention._sm_count = saved


def test_a_prepared_step_is_used_only_for_the_batch_it_was_prepared_for():
    from paged_kv_serving_b200.engine.batch import BatchEntry, ExecutionBatch
    from paged_kv_serving_b200.engine.runner import ModelRunner

    def batch(*entries):
        return ExecutionBatch(tuple(entries))

    expected = batch(BatchEntry("a", (0,), 40, ((3, 4, 5),), (0,), None), BatchEntry("b", (0,), 17, ((9, 8),), (0,), None))
    same = batch(BatchEntry("a", (123,), 40, ((3, 4, 5),), (0,), None), BatchEntry("b", (7,), 17, ((9, 8),), (0,), None))
    assert ModelRunner._as_expected(same, expected)
    others = [
        batch(same.entries[0]),                                                                   # a request left
        batch(same.entries[1], same.entries[0]),                                                  # another order
        batch(BatchEntry("a", (1,), 41, ((3, 4, 5),), (0,), None), same.entries[1]),               # another position
        batch(BatchEntry("a", (1,), 40, ((3, 4, 6),), (0,), None), same.entries[1]),               # a page copied on write
        batch(BatchEntry("a", (1,), 40, ((3, 4, 5, 6),), (0,), None), same.entries[1]),            # a page more
        batch(BatchEntry("c", (1,), 40, ((3, 4, 5),), (0,), None), same.entries[1]),               # another request
        batch(BatchEntry("a", (1, 2), 40, ((3, 4, 5),), (1,), None), same.entries[1]),             # a portion of a prompt
        batch(BatchEntry("a", (1,), 40, ((3, 4, 5),), (), None), same.entries[1]),                 # no logits wanted
        batch(BatchEntry("a", (1,), 40, ((3, 4, 5),), (0,), 2), same.entries[1]),                  # another state slot
    ]
    for other in others:
        assert not ModelRunner._as_expected(other, expected)
