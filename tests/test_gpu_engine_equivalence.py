"""Every logits row the engine samples from, against the plain implementation (``-m gpu``).

The scheduler-driven path as a whole: seeded draws of engine limits (a pool within two pages of
one sequence up to three times that, token budgets of 4 to 160, 1 to 8 running sequences, prefix
cache on and off, a watermark) and of workloads (1 to 6 requests, shared prefixes, prompts of 1
to 300 tokens, greedy and temperature 0.8, 1, 2 or 4 samples a request) run through ``Engine``.
A recorder around the step function keeps every row of logits that a token was sampled from,
with its sequence and context length; each is compared with the plain implementation's logits
at that place of the sequence's final tokens. The cache's invariants are checked after every
step, no step is empty while work is queued, and the scenarios of one model together must have
preempted, hit the prefix cache and forked, so that the comparison cannot go vacuous.

Both ways of stepping are driven: a step's two halves in one call, and overlapped (a step is
launched before the one before it is settled, decoded tokens enter the next step on the device).

On the head-64 model in bfloat16 this drives the tcgen05 prefill attention above cached keys
(recomputed and prefix-attached portions), TMA reads of pages that forked samples share, and
mixed steps alternating with graph-replayed decode steps prepared ahead.

The reference does the same with its ``RecordingExecutor``
(src/paged_kv_serving/engine/equivalence.py:111-187, tests/property/test_engine_equivalence.py:51-190
of rouviere-german/paged-kv-serving).
"""

from __future__ import annotations

import numpy as np
import pytest

import helpers
import plain_model

pytestmark = pytest.mark.gpu


class Recorder:
    """Stands around ``ModelRunner.step``: keeps ``(sequence id, context length, logits row)`` of
    every row a step returns."""

    def __init__(self, runner) -> None:
        self.inner = runner.step
        self.records: list[tuple[str, int, np.ndarray]] = []
        self.graph_steps = 0
        self.mixed_steps = 0
        self._runner = runner

    def __call__(self, batch, **options):
        result = self.inner(batch, **options)
        lens = [e.num_tokens for e in batch.entries]
        if lens and max(lens) > 1 and min(lens) == 1:
            self.mixed_steps += 1
        if self._runner._last_graph_step is not None:
            self.graph_steps += 1
        if result.logits is not None:
            host = result.logits.float().cpu().numpy().copy()
            first = {e.seq_id: e.first_position for e in batch.entries}
            for i, (seq_id, place) in enumerate(result.rows):
                self.records.append((seq_id, first[seq_id] + place + 1, host[i]))
        return result


def _draw_scenario(rng: np.random.Generator, config: dict, block: int, longest: int, scenario: int):
    """One workload and engine limits that admit it. Whether the prefix cache is on and whether
    the pool is cramped alternate with the scenario's number, the rest is drawn."""
    from paged_kv_serving_b200.config import EngineConfig
    from paged_kv_serving_b200.engine.sequence import Request, SamplingParams

    vocab = config["vocab_size"]
    count = int(rng.integers(1, 7))
    shared = [int(t) for t in rng.integers(0, vocab, size=block * int(rng.integers(1, 5)))]
    long_prompts = bool(rng.integers(0, 2))
    requests = []
    for i in range(count):
        length = int(rng.integers(40, longest + 1)) if long_prompts else int(rng.integers(1, 17))
        own = [int(t) for t in rng.integers(0, vocab, size=length)]
        prompt = (shared + own if rng.random() < 0.6 else own)[:longest]
        temperature = 0.8 if rng.random() < 0.5 else 0.0
        n = int(rng.choice([1, 1, 2, 4]))
        requests.append(Request(
            request_id=f"q{i}", prompt_token_ids=tuple(prompt), n=n, key_id="same-key",
            sampling=SamplingParams(max_new_tokens=int(rng.integers(3, 21)), temperature=temperature,
                                    top_p=0.9 if temperature and rng.random() < 0.5 else 1.0, seed=int(rng.integers(0, 1000)))))
    max_prompt = max(r.prompt_len for r in requests)
    max_new = max(r.sampling.max_new_tokens for r in requests)
    one_sequence = -(-(max_prompt + max_new) // block)
    cramped = scenario % 4 < 2
    num_blocks = one_sequence + int(rng.integers(0, 3)) if cramped else int(one_sequence * rng.uniform(1.5, 3.0)) + 1
    engine_config = EngineConfig(
        block_size=block, num_blocks=num_blocks, max_batched_tokens=int(rng.integers(4, 161)),
        max_running_seqs=max(int(rng.integers(1, 9)), max(r.n for r in requests)), max_prompt_tokens=max_prompt,
        max_new_tokens=max_new, max_context_tokens=max_prompt + max_new, enable_prefix_cache=scenario % 2 == 0,
        watermark=float(rng.choice([0.0, 0.05])), dtype="bfloat16")
    return requests, engine_config


@pytest.mark.parametrize("overlap", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, longest, scenarios", [("D", 300, 14), ("B", 150, 10)])
def test_every_sampled_row_matches_the_plain_implementation(name, longest, scenarios, dtype, overlap):
    from dataclasses import replace

    from paged_kv_serving_b200.engine.engine import Engine

    config = helpers.CONFIGS[name]
    tensors = helpers.tensors_for(name, dtype)
    model = helpers.build_model(config, tensors, dtype)
    rng = np.random.default_rng(1000 + len(name) + (7 if dtype == "bfloat16" else 0))
    totals = {"preemptions": 0, "hit_blocks": 0, "forks": 0, "rows": 0, "graph_steps": 0, "mixed_steps": 0}
    for scenario in range(scenarios):
        requests, engine_config = _draw_scenario(rng, config, helpers.PAGE_SIZE[name], longest, scenario)
        engine = Engine(model, replace(engine_config, dtype=dtype), overlap=overlap)
        recorder = Recorder(engine.runner)
        engine.runner.step = recorder
        for request in requests:
            assert engine.submit(request).admitted
        outputs = {}
        for _ in range(20_000):
            if not engine.has_work:
                break
            step = engine.step()
            # (with overlapped steps the last call only settles the step launched before it)
            assert not step.is_empty or step.tokens, "no step may be empty while work is queued"
            engine.check_invariants()
            outputs.update({o.request_id: o for o in step.finished})
        assert not engine.has_work and set(outputs) == {r.request_id for r in requests}
        engine.runner.check_status()

        # the final tokens of every sample, and the plain logits at every place of them
        final: dict[str, list[int]] = {}
        for request in requests:
            samples = outputs[request.request_id].samples
            assert len(samples) == request.n
            for sample in samples:
                assert len(sample.token_ids) == request.sampling.max_new_tokens
                final[f"{request.request_id}#{sample.sample_index}"] = list(request.prompt_token_ids) + list(sample.token_ids)
        plain = {seq_id: plain_model.forward(config, tensors, tokens[:-1]) for seq_id, tokens in final.items()}
        for seq_id, context_len, row in recorder.records:
            want = plain[seq_id][context_len - 1]
            helpers.assert_close(row[None], want[None], dtype,
                                 f"tiny {name} {dtype} scenario {scenario}: {seq_id} at context {context_len} "
                                 f"({engine_config})")
        # every token was sampled from a recorded row: prompts end once per request (forks share
        # that row), every later token has a row of its own; recomputation adds rows, never drops any
        sampled = sum(r.n * r.sampling.max_new_tokens for r in requests)
        assert len(recorder.records) >= sampled - sum(r.n - 1 for r in requests)
        totals["preemptions"] += engine.scheduler.stats.preemptions
        totals["hit_blocks"] += engine.prefix_cache.stats.hit_blocks
        totals["forks"] += sum(r.n - 1 for r in requests)
        totals["rows"] += len(recorder.records)
        totals["graph_steps"] += recorder.graph_steps
        totals["mixed_steps"] += recorder.mixed_steps
        engine.flush_prefix_cache()
        engine.check_invariants()
        assert engine.cache.num_free_blocks == engine_config.num_blocks, "the pool is whole after the flush"
    print(f"\n[tiny {name} {dtype}] {totals}")
    assert totals["preemptions"] > 0, "the scenarios must preempt"
    assert totals["hit_blocks"] > 0, "the scenarios must hit the prefix cache"
    assert totals["forks"] > 0, "the scenarios must fork"
    assert totals["mixed_steps"] > 0, "portions must have run beside decoded tokens"
    if dtype == "bfloat16":
        assert totals["graph_steps"] > 0, "decode steps must have been replayed as graphs"


@pytest.mark.parametrize("overlap", [True, False])
def test_requests_aborted_between_steps_leave_the_others_right_and_the_pool_whole(overlap):
    """Drawn scenarios on tiny D in bfloat16 in which requests are aborted at random moments (with
    overlapped steps: while a step that holds their tokens is in flight). Every other request
    finishes with all its tokens, every row sampled for it is the plain implementation's, the
    books balance after every call and the pool is whole at the end."""
    from dataclasses import replace

    from paged_kv_serving_b200.engine.engine import Engine

    name, dtype = "D", "bfloat16"
    config = helpers.CONFIGS[name]
    tensors = helpers.tensors_for(name, dtype)
    model = helpers.build_model(config, tensors, dtype)
    rng = np.random.default_rng(50_001)
    aborts = 0
    for scenario in range(16):
        requests, engine_config = _draw_scenario(rng, config, helpers.PAGE_SIZE[name], 300, scenario)
        engine = Engine(model, replace(engine_config, dtype=dtype), overlap=overlap)
        recorder = Recorder(engine.runner)
        engine.runner.step = recorder
        for request in requests:
            assert engine.submit(request).admitted
        outputs, gone = {}, set()
        for _ in range(20_000):
            if not engine.has_work:
                break
            if rng.random() < 0.1:
                victim = requests[int(rng.integers(0, len(requests)))].request_id
                if victim not in gone and victim not in outputs:
                    engine.abort(victim)
                    gone.add(victim)
                    aborts += 1
                    engine.check_invariants()
            step = engine.step()
            engine.check_invariants()
            outputs.update({o.request_id: o for o in step.finished})
        assert not engine.has_work
        engine.runner.check_status()
        final = {}
        for request in requests:
            if request.request_id in gone:
                continue
            assert request.request_id in outputs, "a request that was not aborted must finish"
            for sample in outputs[request.request_id].samples:
                assert len(sample.token_ids) == request.sampling.max_new_tokens
                final[f"{request.request_id}#{sample.sample_index}"] = list(request.prompt_token_ids) + list(sample.token_ids)
        plain = {seq_id: plain_model.forward(config, tensors, tokens[:-1]) for seq_id, tokens in final.items()}
        for seq_id, context_len, row in recorder.records:
            if seq_id in plain:
                helpers.assert_close(row[None], plain[seq_id][context_len - 1][None], dtype, f"scenario {scenario}: {seq_id} at {context_len}")
        engine.flush_prefix_cache()
        engine.check_invariants()
        assert engine.cache.num_free_blocks == engine_config.num_blocks, "the pool is whole after the flush"
    assert aborts >= 5, "the scenarios must abort requests"
