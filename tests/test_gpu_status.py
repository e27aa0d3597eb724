"""The device's status word and the bounded waits behind it (``-m gpu``).

The kernels that wait on mbarriers give up after a limit, record code 2 in the device's status
word and return in order; an embedding lookup of an id outside the table records code 1; a
page, a cache slot or a position outside its range records code 3 and is not used (the bad
index never becomes an address: the store is skipped, the page reads as zeros). The host reads
the word in the copy that brings a step's results back and raises. Nothing here
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


@pytest.fixture
def device_status():
    """The device's own status word (the kernels without a status argument record there), zero
    before and after."""
    from paged_kv_serving_b200 import ops

    word = ops.status_word("cuda")
    word.zero_()
    yield word
    word.zero_()


@pytest.mark.parametrize("value", [10 ** 6, -5])
@pytest.mark.parametrize("kernel", ["generic", "mma", "mma-prefill", "tma", "flat", "tcgen05"])
def test_a_table_entry_that_is_no_page_is_recorded_and_read_as_zeros(kernel, value, device_status):
    """A block-table entry beyond the pool (or negative and not -1) in the middle of a sequence:
    every attention kernel records code 3 and reads that page's keys and values as zeros, as it
    reads -1; the answer is the plain one with those keys and values zeroed."""
    import test_gpu_kernels as kernels

    rng = np.random.default_rng(len(kernel) + abs(value) % 7)
    common = dict(heads=8, kv=2, hd=64, page=16, window=None, dtype="bfloat16", spike=False, corrupt=(1, 2, value))
    if kernel == "generic":
        got, want = kernels._attention_case(rng, contexts=[40, 100, 17], queries=[1, 3, 17], **common)
    elif kernel == "mma":
        got, want = kernels._attention_case(rng, contexts=[40, 100, 17], queries=[1, 2, 1], fast=True, splits=2, **common)
    elif kernel == "mma-prefill":
        got, want = kernels._attention_case(rng, contexts=[40, 100, 70], queries=[40, 100, 70], fast=True, **common)
    elif kernel == "tma":
        got, want = kernels._attention_case(rng, contexts=[40, 100, 17], queries=[1, 2, 1], fast=True, tcgen05=True, splits=2,
                                            expect_status=3, **common)
    elif kernel == "flat":
        got, want = kernels._attention_case(rng, contexts=[40, 100, 17], queries=[1, 2, 1], fast=True, tcgen05=True,
                                            flat_blocks=5, expect_status=3, **common)
    else:
        got, want = kernels._attention_case(rng, contexts=[40, 200, 70], queries=[40, 200, 70], fast=True, tcgen05=True,
                                            expect_status=3, **common)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 2e-2 * max(1.0, np.abs(want).max())
    if kernel in ("generic", "mma", "mma-prefill"):
        assert int(device_status.item()) == 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hd", [20, 64])
def test_a_slot_or_position_out_of_range_is_recorded_and_not_used(hd, dtype, device_status):
    """The rotation and cache-write kernel (both of its forms): a slot beyond the pools is not
    written to, a position beyond the tables is not looked up; both are recorded as code 3 and
    every other token is treated as always."""
    from paged_kv_serving_b200 import ops
    import plain_model
    import test_gpu_kernels as kernels

    rng = np.random.default_rng(hd)
    heads, kv, page, pages, tokens = 4, 2, 4, 6, 7
    torch_dtype = kernels.DTYPES[dtype]
    cos, sin = plain_model.rope_tables(32, hd, 10000.0)
    qkv = rng.standard_normal((tokens, (heads + 2 * kv) * hd)).astype(np.float32)
    positions = rng.integers(0, 32, size=tokens).astype(np.int32)
    slots = rng.permutation(pages * page)[:tokens].astype(np.int32)
    for bad_slot, bad_position in ((pages * page + 3, None), (-9, None), (None, 32), (None, -1)):
        device_status.zero_()
        s, p = slots.copy(), positions.copy()
        if bad_slot is not None:
            s[2] = bad_slot
        if bad_position is not None:
            p[4] = bad_position
        qkv_d = kernels.dev(qkv, torch_dtype)
        seen = kernels.as_np(qkv_d).copy()
        k_pool = torch.full((pages, kv, page, hd), float("nan"), dtype=torch_dtype, device="cuda")
        v_pool = torch.full((pages, kv, page, hd), float("nan"), dtype=torch_dtype, device="cuda")
        ops.rope_kv_store(qkv_d, kernels.dev(p), kernels.dev(cos), kernels.dev(sin), k_pool, v_pool, kernels.dev(s),
                          heads, kv, hd, page)
        assert int(device_status.item()) == 3
        kp, vp = kernels.as_np(k_pool), kernels.as_np(v_pool)
        k = seen[:, heads * hd:(heads + kv) * hd].reshape(tokens, kv, hd)
        v = seen[:, (heads + kv) * hd:].reshape(tokens, kv, hd)
        used = np.where((p >= 0) & (p < 32), p, 0)
        k_rot = plain_model.apply_rope(k, used, cos, sin)
        written = np.zeros((pages, page), dtype=bool)
        for t in range(tokens):
            if not 0 <= s[t] < pages * page:
                continue
            at, offset = divmod(int(s[t]), page)
            written[at, offset] = True
            assert np.abs(kp[at, :, offset] - k_rot[t]).max() <= kernels.tol(dtype, 4)
            assert np.abs(vp[at, :, offset] - v[t]).max() <= kernels.tol(dtype, 1e-3)
        untouched = np.broadcast_to(~written[:, None, :], (pages, kv, page))
        assert np.isnan(kp[untouched]).all() and np.isnan(vp[untouched]).all()


def test_the_fused_projection_checks_slots_and_positions_too(device_status):
    """The decode projection with rotation and cache write in its epilogue: the same two checks."""
    from paged_kv_serving_b200 import ops
    import plain_model
    import test_gpu_kernels as kernels

    rng = np.random.default_rng(5)
    heads, kv, hd, page, pages, rows, width = 4, 2, 64, 16, 3, 5, 256
    cos, sin = plain_model.rope_tables(64, hd, 10000.0)
    x = kernels.dev(rng.standard_normal((rows, width)).astype(np.float32), torch.bfloat16)
    w = kernels.dev((rng.standard_normal(((heads + 2 * kv) * hd, width)) * 0.05).astype(np.float32), torch.bfloat16)
    positions = np.asarray([3, 9, 64, 1, 0], dtype=np.int32)                  # one beyond the tables
    slots = np.asarray([0, 17, 5, pages * page, 40], dtype=np.int32)          # one beyond the pools
    k_pool = torch.full((pages, kv, page, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    v_pool = torch.full((pages, kv, page, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    out = ops.gemm_small_m(x, w, "rope_kv", rope_kv=(kernels.dev(positions), kernels.dev(cos), kernels.dev(sin), k_pool,
                                                      v_pool, kernels.dev(slots), heads, kv, hd, page))
    assert int(device_status.item()) == 3
    assert torch.isfinite(out[:, :heads * hd].float()).all()
    written = torch.isfinite(k_pool.float()).any(dim=(1, 3))                  # [pages, page]
    expect = torch.zeros_like(written)
    for slot in (0, 17, 5, 40):
        expect[slot // page, slot % page] = True
    assert torch.equal(written, expect)
