"""The device's status word and the bounded waits behind it (``-m gpu``).

The kernels that wait on mbarriers give up after a limit, record code 2 in the device's status
word and return in order; an embedding lookup of an id outside the table records code 1. The
host reads the word in the copy that brings a step's results back and raises. Nothing here
faults, traps or hangs the GPU: the one wait that runs out is a probe that waits, for about a
millisecond, on a barrier nothing arrives at, and returns by itself.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def test_a_bounded_wait_gives_up_records_its_code_and_leaves_the_context_usable():
    from paged_kv_serving_b200 import ops

    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    started, ended = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    started.record()
    gave_up = ops.wait_probe(status, 2_000_000)       # about a millisecond of SM clock cycles
    ended.record()
    torch.cuda.synchronize()
    assert int(gave_up.item()) == 1 and int(status.item()) == 2
    assert 0.2 < started.elapsed_time(ended) < 100.0, "the wait ran for its limit, not for the kernels' second"
    # the context is as usable as before: an ordinary kernel runs and is right
    x = torch.arange(1000, device="cuda", dtype=torch.float32)
    assert float(x.sum().item()) == 499500.0
    with pytest.raises(RuntimeError, match="gave up a bounded wait"):
        ops.raise_for_status(int(status.item()), "cuda")
    with pytest.raises(ValueError):
        ops.wait_probe(status, 10 ** 10)                 # limits beyond a tenth of a second are refused


def _engine(dtype="bfloat16"):
    from paged_kv_serving_b200.config import EngineConfig
    from paged_kv_serving_b200.engine.engine import Engine

    model = helpers.build_model(helpers.TINY_D, helpers.tensors_for("D", dtype), dtype)
    config = EngineConfig(block_size=16, num_blocks=32, max_batched_tokens=64, max_running_seqs=4, max_prompt_tokens=64,
                          max_new_tokens=8, max_context_tokens=96, dtype=dtype)
    return Engine(model, config)


def test_engine_step_raises_on_a_recorded_fault_and_recovers():
    """A wait that gave up anywhere in a step reaches the host with the sampled ids: the step
    raises, the word and the shared workspaces are cleared, and the next request runs clean."""
    from paged_kv_serving_b200 import ops
    from paged_kv_serving_b200.engine.sequence import Request, SamplingParams

    engine = _engine()
    prompt = tuple(helpers.random_tokens(helpers.TINY_D, 20, seed=1))
    clean = engine.generate([Request("clean", prompt, SamplingParams(max_new_tokens=4))])[0].samples[0].token_ids
    engine.submit(Request("r", prompt, SamplingParams(max_new_tokens=6)))
    engine.step()                                                   # the prompt and the first token
    ops.wait_probe(engine.runner.status, 2_000_000)                 # what a real kernel's give-up leaves behind
    with pytest.raises(RuntimeError, match="gave up a bounded wait"):
        # the word travels with the ids of the next step that is settled: with overlapped steps
        # that is the call after the one that launches it
        engine.step()
        engine.step()
    assert int(engine.runner.status.item()) == 0, "the word is cleared once its fault has been raised"
    assert engine.active_requests == 0 and not engine.has_work, "the request whose step failed was aborted"
    engine.check_invariants()
    again = engine.generate([Request("again", prompt, SamplingParams(max_new_tokens=4))])[0].samples[0].token_ids
    assert again == clean


def test_replay_step_raises_on_a_recorded_fault():
    from paged_kv_serving_b200 import ops
    from paged_kv_serving_b200.engine.replay import ReplaySession

    model = helpers.build_model(helpers.TINY_D, helpers.tensors_for("D", "bfloat16"), "bfloat16")
    session = ReplaySession(model, max_tokens=128, block_size=16)
    tokens = helpers.random_tokens(helpers.TINY_D, 40, seed=2)
    first = session.step([{"id": "a", "tokens": tokens[:30], "want": [29]}])
    ops.wait_probe(session.runner.status, 2_000_000)
    with pytest.raises(RuntimeError, match="gave up a bounded wait"):
        session.step([{"id": "a", "tokens": tokens[30:32], "want": [1]}])
    # afterwards the session answers as before
    session.step([], end=["a"])
    again = session.step([{"id": "b", "tokens": tokens[:30], "want": [29]}])
    assert np.array_equal(first, again)


def test_status_stays_zero_through_ordinary_steps():
    engine = _engine()
    from paged_kv_serving_b200.engine.sequence import Request, SamplingParams

    prompts = [tuple(helpers.random_tokens(helpers.TINY_D, n, seed=n)) for n in (5, 33, 64)]
    engine.generate([Request(f"r{i}", p, SamplingParams(max_new_tokens=8)) for i, p in enumerate(prompts)])
    engine.runner.check_status()                                    # raises if any kernel recorded anything
    assert int(engine.runner.status.item()) == 0


def test_sampling_a_draw_at_the_very_top_lands_on_a_kept_token():
    """u = 1 - 2^-53 with a nucleus filter: the draw sits at (or rounds up to) the total mass, where
    no share of the cumulative sum claims it. The id must be one the filter kept, never the
    vocabulary's last id, which the filter zeroed."""
    from paged_kv_serving_b200 import ops
    import plain_model

    rng = np.random.default_rng(11)
    top = float(np.nextafter(1.0, 0.0))
    for vocab, top_p in ((1237, 0.5), (50021, 0.3), (4096, 0.9)):
        logits = (rng.standard_normal((4, vocab)) * 3).astype(np.float32)
        logits[:, vocab - 1] = -40.0                                 # the last id is never inside the nucleus
        temperature = np.full(4, 0.9, dtype=np.float32)
        tp = np.full(4, top_p, dtype=np.float32)
        u = np.array([top, top, 0.999999999, 1.0 - 2.0 ** -40])
        ids = ops.sample(torch.from_numpy(logits).cuda(), torch.from_numpy(temperature).cuda(), torch.from_numpy(tp).cuda(),
                         torch.from_numpy(u).cuda(), 1e-5).cpu().numpy()
        for row in range(4):
            p = plain_model.sample_distribution(logits[row], 0.9, top_p)
            assert p[ids[row]] > 0.0, (vocab, row, int(ids[row]))
            assert ids[row] == int(np.nonzero(p)[0].max()), "the top of the distribution is the last kept id"
