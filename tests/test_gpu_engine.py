"""Generation through the Python entry point, the command line and ``bin/trace_run`` (``-m gpu``)."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers
import plain_model

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _folder(tmp_path, name, dtype):
    from paged_kv_serving_b200.config import ModelConfig
    from paged_kv_serving_b200.weights.random_init import write_model_folder

    tensors = helpers.tensors_for(name, dtype)
    stored = {k: torch.from_numpy(v).to(torch.bfloat16 if dtype == "bfloat16" and v.ndim == 2 else torch.float32)
              for k, v in tensors.items()}
    write_model_folder(tmp_path, ModelConfig.from_dict(helpers.CONFIGS[name]), stored)
    return tensors


def test_decode_steps_prepared_ahead_are_the_steps_built_afresh():
    """While the GPU runs a decode step the runner builds the integer arrays of the next one.
    They must be the arrays it would build when the step arrives, it must use them only when the
    batch is the expected one, and a page boundary or another batch must make it build afresh."""
    from paged_kv_serving_b200.engine.batch import BatchEntry, ExecutionBatch
    from paged_kv_serving_b200.engine.runner import ModelRunner
    from paged_kv_serving_b200.parts.base import StepContext

    config = helpers.TINY_D
    tensors = helpers.tensors_for("D", "bfloat16")
    model = helpers.build_model(config, tensors, "bfloat16")
    prompts = [helpers.random_tokens(config, n, seed=300 + n) for n in (60, 37)]
    pages = 6
    tables = [tuple(range(i * pages, (i + 1) * pages)) for i in range(2)]
    outputs = {}
    for ahead in (True, False):
        runner = ModelRunner(model, num_blocks=2 * pages, block_size=16, max_running_seqs=2)
        for i, p in enumerate(prompts):
            runner.step(ExecutionBatch((BatchEntry(f"s{i}", tuple(p[:30]), 0, (tables[i],), ()),)))
        rows, used = [], 0
        for k in range(30, 37):
            batch = ExecutionBatch(tuple(BatchEntry(f"s{i}", (p[k],), k, (tables[i],), (0,)) for i, p in enumerate(prompts)))
            was_ready = runner._ahead is not None
            result = runner.step(batch)
            used += was_ready and runner._ahead is None
            if ahead:
                runner.prepare_next()
                if k == 31:     # position 32 starts a new page of this table: it is there, so the step is prepared
                    assert runner._ahead is not None
                    fresh, _ = runner._context(runner._ahead["batch"], table_width=32, pad_to=2)
                    for name, shape in fresh.arena.signature():
                        if name != StepContext.TOKEN_IDS:
                            assert np.array_equal(fresh.arena.host(name), runner._ahead["ctx"].arena.host(name)), name
            rows.append(result.logits.float().cpu().numpy())
        # another batch than the expected one: one request alone
        runner.prepare_next() if ahead else None
        alone = runner.step(ExecutionBatch((BatchEntry("s0", (prompts[0][37],), 37, (tables[0],), (0,)),)))
        rows.append(alone.logits.float().cpu().numpy())
        outputs[ahead] = np.concatenate(rows)
        assert (used > 0) == ahead
    assert np.array_equal(outputs[True], outputs[False])
    want = plain_model.forward(config, tensors, prompts[0][:38])
    helpers.assert_close(outputs[True][-1:], want[37:38], "bfloat16", "prepared-ahead decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    from paged_kv_serving_b200.api import generate

    config = helpers.CONFIGS[name]
    tensors = _folder(tmp_path, name, dtype)
    prompts = [helpers.random_tokens(config, n, seed=20 + n) for n in (5, 9, 17)]
    got = generate(tmp_path, prompts, max_new_tokens=8, dtype=dtype, block_size=helpers.PAGE_SIZE[name],
                   max_batched_tokens=16)
    for i, (prompt, samples) in enumerate(zip(prompts, got)):
        assert len(samples[0]) == 8
        helpers.assert_greedy_tokens(config, tensors, prompt, samples[0], dtype, f"tiny {name} prompt {i}")


def test_generation_is_the_same_cramped_and_roomy_and_hits_the_prefix_cache(tmp_path):
    """Tiny B in float32: prompts of 1, 7, 30 and 64 tokens, the last two sharing 16 tokens;
    temperature 0.8 with per-request seeds; a pool with few pages forces preemption."""
    from paged_kv_serving_b200.config import EngineConfig
    from paged_kv_serving_b200.engine.engine import Engine
    from paged_kv_serving_b200.engine.sequence import Request, SamplingParams
    from paged_kv_serving_b200.models.decoder import DecoderModel

    config = helpers.TINY_B
    tensors = _folder(tmp_path, "B", "float32")
    rng = np.random.default_rng(3)
    shared = [int(t) for t in rng.integers(0, config["vocab_size"], size=16)]
    prompts = [[int(t) for t in rng.integers(0, config["vocab_size"], size=n)] for n in (1, 7)]
    prompts += [shared + [int(t) for t in rng.integers(0, config["vocab_size"], size=n)] for n in (14, 48)]
    model = DecoderModel.from_folder(tmp_path, dtype="float32")

    def run(num_blocks, budget):
        engine = Engine(model, EngineConfig(block_size=8, num_blocks=num_blocks, max_batched_tokens=budget,
                                            max_running_seqs=4, max_prompt_tokens=64, max_new_tokens=12,
                                            max_context_tokens=76, dtype="float32", watermark=0.0))
        requests = [Request(f"r{i}", tuple(p), SamplingParams(max_new_tokens=12, temperature=0.8, seed=40 + i))
                    for i, p in enumerate(prompts)]
        outputs = {o.request_id: o for o in engine.generate(requests)}
        engine.check_invariants()
        return engine, [list(outputs[f"r{i}"].samples[0].token_ids) for i in range(len(prompts))], outputs

    roomy, roomy_tokens, outputs = run(64, 16)
    cramped, cramped_tokens, _ = run(13, 16)
    assert roomy_tokens == cramped_tokens
    assert cramped.scheduler.stats.preemptions > 0, "the cramped pool must preempt"
    assert roomy.prefix_cache.stats.hit_blocks >= 2 and outputs["r3"].cached_prompt_tokens == 16
    for i, prompt in enumerate(prompts):
        want = plain_model.generate(config, tensors, prompt, 12, temperature=0.8, seed=40 + i)
        assert roomy_tokens[i] == want, f"request {i}"


def test_overlapped_steps_give_the_tokens_of_steps_in_order():
    """Launching step k before step k-1 is settled changes when the host learns a token, not the
    token: the same requests (greedy and sampled, 1 to 3 samples each, a stop token that ends
    some of them early, a pool so small that sequences are preempted, shared prefixes) give the
    same outputs, finish reasons and counts both ways, and the pool is whole afterwards. In
    float32, where a recomputed sequence's logits do not depend on which kernels recomputed them
    beyond 1e-6 (the two ways preempt at different moments); the bfloat16 logits of overlapped
    steps are compared row by row in test_gpu_engine_equivalence.py."""
    dtype = "float32"
    from paged_kv_serving_b200.config import EngineConfig
    from paged_kv_serving_b200.engine.engine import Engine
    from paged_kv_serving_b200.engine.sequence import FinishReason, Request, SamplingParams

    config = helpers.TINY_D
    model = helpers.build_model(config, helpers.tensors_for("D", dtype), dtype)
    rng = np.random.default_rng(12)
    shared = [int(t) for t in rng.integers(0, config["vocab_size"], size=32)]
    prompts = [shared + [int(t) for t in rng.integers(0, config["vocab_size"], size=n)] for n in (3, 40, 9, 70, 1, 25)]

    def run(overlap, eos):
        engine = Engine(model, EngineConfig(block_size=16, num_blocks=10, max_batched_tokens=48, max_running_seqs=6,
                                            max_prompt_tokens=104, max_new_tokens=24, max_context_tokens=128,
                                            dtype=dtype, watermark=0.0), eos_token_id=eos, overlap=overlap)
        requests = [Request(f"r{i}", tuple(p), SamplingParams(max_new_tokens=10 + 2 * i, temperature=0.0 if i % 2 else 0.9,
                                                              top_p=0.95, seed=70 + i), n=1 + i % 3)
                    for i, p in enumerate(prompts)]
        outputs = {o.request_id: o for o in engine.generate(requests)}
        engine.check_invariants()
        engine.flush_prefix_cache()
        assert engine.cache.num_free_blocks == 10 and not engine.has_work
        return engine, {name: [(s.sample_index, s.token_ids, s.finish_reason) for s in o.samples]
                        for name, o in outputs.items()}

    _, free_running = run(False, None)
    # a stop token that some samples meet early: the most frequent token of the free-running outputs
    counts = np.bincount([t for samples in free_running.values() for _, tokens, _ in samples for t in tokens[2:]])
    eos = int(counts.argmax())
    in_order_engine, in_order = run(False, eos)
    overlapped_engine, overlapped = run(True, eos)
    assert overlapped == in_order
    reasons = [reason for samples in in_order.values() for _, _, reason in samples]
    assert FinishReason.STOP in reasons and FinishReason.LENGTH in reasons
    assert in_order_engine.scheduler.stats.preemptions > 0 and overlapped_engine.scheduler.stats.preemptions > 0
    assert overlapped_engine.prefix_cache.stats.hit_blocks > 0


def test_n_way_sampling_shares_the_prompt_and_reproduces(tmp_path):
    from paged_kv_serving_b200.api import generate

    config = helpers.TINY_A
    tensors = _folder(tmp_path, "A", "float32")
    prompt = helpers.random_tokens(config, 11, seed=8)
    got = generate(tmp_path, [prompt], max_new_tokens=6, temperature=1.0, top_p=0.9, seed=5, n=3, dtype="float32",
                   block_size=4)
    assert len(got[0]) == 3
    for index, sample in enumerate(got[0]):
        want = plain_model.generate(config, tensors, prompt, 6, temperature=1.0, top_p=0.9, seed=5, sample_index=index)
        assert sample == want
    assert len({tuple(s) for s in got[0]}) > 1


def test_command_line_build_and_generate(tmp_path):
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    build = subprocess.run([sys.executable, "-m", "paged_kv_serving_b200", "build-checkpoint", "--out", str(tmp_path),
                            "--preset", "tiny-a", "--seed", "7", "--dtype", "float32", "--std", "0.08"],
                           capture_output=True, text=True, env=env, check=True)
    assert json.loads(build.stdout)["parameters"] == 123712
    run = subprocess.run([sys.executable, "-m", "paged_kv_serving_b200", "generate", "--model", str(tmp_path),
                          "--prompt-ids", "5,17,3,200", "--prompt-ids", "9 8 7", "--max-new-tokens", "5",
                          "--dtype", "float32", "--block-size", "4"], capture_output=True, text=True, env=env, check=True)
    lines = [json.loads(line) for line in run.stdout.splitlines() if line.startswith("{")]
    assert [line["prompt_token_ids"] for line in lines] == [[5, 17, 3, 200], [9, 8, 7]]
    from paged_kv_serving_b200.weights import read_model_folder

    config, stored = read_model_folder(tmp_path)
    tensors = {k: v.float().numpy() for k, v in stored.items()}
    for line in lines:
        want = plain_model.generate(config.to_dict(), tensors, line["prompt_token_ids"], 5)
        assert line["samples"][0] == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    """``bin/trace_run`` as a user runs it: a process, JSON lines in, ``done`` lines and files out."""
    name = "B"
    config = helpers.CONFIGS[name]
    model_dir, out_dir = tmp_path / "model", tmp_path / "out"
    tensors = _folder(model_dir, name, dtype)
    a = helpers.random_tokens(config, 70, seed=31)
    b = helpers.random_tokens(config, 40, seed=32)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:50], "want": [0, 49]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[:38], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[50:52], "want": [1]}, {"id": "b", "tokens": b[38:39], "want": [0]}], "end": []},
        {"step": 3, "entries": [{"id": "b", "tokens": b[39:], "want": [0]}], "end": ["b"]},
        {"step": 4, "entries": [{"id": "a", "tokens": a[52:], "want": [17]}], "end": ["a"]},
    ]
    process = subprocess.Popen([str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
                                "--out", str(out_dir), "--max-tokens", "128", "--block-size", "8"],
                               stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for record in steps:
        process.stdin.write(json.dumps(record) + "\n")
        process.stdin.flush()
        assert process.stdout.readline().strip() == f"done {record['step']}"
    process.stdin.close()
    assert process.wait(timeout=120) == 0
    ref_a = plain_model.forward(config, tensors, a)
    ref_b = plain_model.forward(config, tensors, b)
    vocab = config["vocab_size"]
    read = lambda step: np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(-1, vocab)
    assert not (out_dir / "1.f32").exists()
    helpers.assert_close(read(0), ref_a[[0, 49]], dtype, "step 0")
    helpers.assert_close(read(2), np.stack([ref_a[51], ref_b[38]]), dtype, "step 2")
    helpers.assert_close(read(3), ref_b[39:40], dtype, "step 3")
    helpers.assert_close(read(4), ref_a[69:70], dtype, "step 4")
