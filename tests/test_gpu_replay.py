"""The engine against the plain implementation, through the replay session (``-m gpu``).

Every request is replayed whole, with the last 32 tokens decoded one by one, in portions of
changing size down to two tokens, and mixed with other requests in a pool so small that pages
are used again; in float32 and in bfloat16; on tiny configurations that differ in every size.
"""

from __future__ import annotations

import numpy as np
import pytest

import helpers
import plain_model

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")
LENGTHS = {"A": 100, "B": 150, "C": 300, "D": 450}


def _session(name, dtype, max_tokens):
    from paged_kv_serving_b200.engine.replay import ReplaySession

    tensors = helpers.tensors_for(name, dtype)
    model = helpers.build_model(helpers.CONFIGS[name], tensors, dtype)
    session = ReplaySession(model, max_tokens=max_tokens, block_size=helpers.PAGE_SIZE[name])
    session.runner.storage.fill(float("nan"))   # stale pages must never be read
    return session, tensors


def _reference(name, tensors, tokens):
    return plain_model.forward(helpers.CONFIGS[name], tensors, tokens)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ("A", "B", "C", "D"))
def test_whole_prompt_every_position(name, dtype):
    session, tensors = _session(name, dtype, 512)
    tokens = helpers.random_tokens(helpers.CONFIGS[name], LENGTHS[name], seed=11)
    got = session.step([{"id": "r", "tokens": tokens, "want": list(range(len(tokens)))}], end=["r"])
    helpers.assert_close(got, _reference(name, tensors, tokens), dtype, f"{name} whole")
    session.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ("A", "B", "C", "D"))
def test_bulk_then_last_32_one_by_one(name, dtype):
    session, tensors = _session(name, dtype, 512)
    tokens = helpers.random_tokens(helpers.CONFIGS[name], LENGTHS[name], seed=12)
    want = _reference(name, tensors, tokens)
    bulk = len(tokens) - 32
    got = [session.step([{"id": "r", "tokens": tokens[:bulk], "want": [bulk - 1]}])]
    for i in range(bulk, len(tokens)):
        got.append(session.step([{"id": "r", "tokens": [tokens[i]], "want": [0]}]))
    helpers.assert_close(np.concatenate(got), want[bulk - 1:], dtype, f"{name} bulk+decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ("A", "B", "C", "D"))
def test_portions_of_changing_size(name, dtype):
    session, tensors = _session(name, dtype, 512)
    tokens = helpers.random_tokens(helpers.CONFIGS[name], LENGTHS[name], seed=13)
    want = _reference(name, tensors, tokens)
    # config D also takes portions of 130 and 150 tokens: enough rows for the tensor-core product
    sizes, cycle, at = [], [7, 3, 11, 2, 5, 2, 13, 1, 4] if name != "D" else [7, 150, 2, 130, 3, 1, 60, 2], 0
    while sum(sizes) < len(tokens):
        sizes.append(min(cycle[at % len(cycle)], len(tokens) - sum(sizes)))
        at += 1
    start, rows, got = 0, [], []
    for size in sizes:
        out = session.step([{"id": "r", "tokens": tokens[start:start + size], "want": [0, size - 1] if size > 1 else [0]}])
        rows += [start, start + size - 1] if size > 1 else [start]
        got.append(out)
        start += size
    helpers.assert_close(np.concatenate(got), want[rows], dtype, f"{name} portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ("A", "B", "D"))
def test_mixed_requests_with_page_reuse(name, dtype):
    """Up to four live requests; portions of some beside decoded tokens of others; the pool
    (256 tokens) is smaller than what all requests need together, so pages are used again."""
    config = helpers.CONFIGS[name]
    session, tensors = _session(name, dtype, 256)
    lengths = [60, 50, 64, 40, 64, 30, 55, 48]
    prompts = [helpers.random_tokens(config, n, seed=100 + i) for i, n in enumerate(lengths)]
    wants = [_reference(name, tensors, p) for p in prompts]
    rng = np.random.default_rng(7)
    progress = [0] * len(prompts)
    waiting = list(range(len(prompts)))
    live: list[int] = []
    owners: dict[int, set[str]] = {}      # page -> the requests that have held it
    step = 0
    while waiting or live:
        while waiting and len(live) < 4 and sum(-(-lengths[i] // 64) * 64 for i in live) + 64 <= 256:
            live.append(waiting.pop(0))
        entries, finished, checks = [], [], []
        for i in live:
            remaining = lengths[i] - progress[i]
            decode_phase = remaining <= 8
            size = 1 if decode_phase else int(min(remaining - 8, rng.integers(2, 14)))
            chunk = prompts[i][progress[i]:progress[i] + size]
            want = [size - 1]
            entries.append({"id": f"q{i}", "tokens": chunk, "want": want})
            checks.append((i, progress[i] + size - 1))
            progress[i] += size
            if progress[i] == lengths[i]:
                finished.append(i)
        got = session.step(entries, end=[f"q{i}" for i in finished])
        for row, (i, position) in enumerate(checks):
            helpers.assert_close(got[row:row + 1], wants[i][position:position + 1], dtype,
                                 f"{name} mixed step {step} request {i} position {position}")
        for request, sequence in session.live.items():
            for page in sequence.block_table:
                owners.setdefault(page, set()).add(request)
        for i in finished:
            live.remove(i)
        session.check_invariants()
        step += 1
    total_pages_needed = sum(-(-n // helpers.PAGE_SIZE[name]) for n in lengths)
    assert total_pages_needed > session.num_blocks, "the scenario must need more pages than the pool has"
    assert session.cache.num_free_blocks == session.num_blocks
    assert sum(len(requests) > 1 for requests in owners.values()) >= session.num_blocks // 2, \
        "pages must have passed from finished requests to later ones"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, d_ff, vocab, n_kv", [("A", 173, 257, 2), ("B", 75, 1001, 1), ("D", 333, 515, 2)])
def test_odd_feed_forward_and_vocabulary_sizes(name, d_ff, vocab, n_kv, dtype):
    """Inner sizes and vocabularies that are odd numbers (no multiple of 8, so no 16-byte rows):
    a prompt, a portion of two tokens and decoding, against the plain implementation."""
    from paged_kv_serving_b200.engine.replay import ReplaySession

    config = dict(helpers.CONFIGS[name], d_ff=d_ff, vocab_size=vocab, n_kv_heads=n_kv)
    tensors = plain_model.random_tensors(config, seed=3, std=0.06)
    if dtype == "bfloat16":
        tensors = {k: (plain_model.round_to_bfloat16(v) if v.ndim == 2 else v) for k, v in tensors.items()}
    model = helpers.build_model(config, tensors, dtype)
    tokens = helpers.random_tokens(config, 70, seed=5)
    want = plain_model.forward(config, tensors, np.asarray(tokens))
    session = ReplaySession(model, max_tokens=128, block_size=helpers.PAGE_SIZE[name])
    got = [session.step([{"id": "a", "tokens": tokens[:37], "want": list(range(37))}])]
    got.append(session.step([{"id": "a", "tokens": tokens[37:39], "want": [0, 1]}]))
    got += [session.step([{"id": "a", "tokens": [t], "want": [0]}]) for t in tokens[39:]]
    helpers.assert_close(np.concatenate(got), want, dtype, f"odd sizes {name}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd, heads, kv, page", [(16, 5, 5, 32), (48, 4, 2, 16), (80, 2, 1, 8), (96, 3, 3, 16), (112, 2, 2, 4),
                                                   (144, 2, 1, 16), (128, 4, 1, 128), (64, 6, 3, 64)])
def test_head_sizes_head_counts_and_page_sizes_through_the_engine(hd, heads, kv, page, dtype):
    """Head sizes in steps of 16 (and one beyond 128), head counts and groupings that are no
    power of two, pages of 4 to 128 keys: whichever attention kernel the engine picks for them, a
    prompt in two portions beside a second request, then both decoding, against the plain
    implementation."""
    from paged_kv_serving_b200.engine.replay import ReplaySession

    config = dict(helpers.TINY_A, d_model=heads * hd, n_heads=heads, n_kv_heads=kv, head_dim=hd, d_ff=96, vocab_size=300,
                  n_layers=2, max_seq_len=256)
    tensors = plain_model.random_tensors(config, seed=hd, std=0.05)
    if dtype == "bfloat16":
        tensors = {k: (plain_model.round_to_bfloat16(v) if v.ndim == 2 else v) for k, v in tensors.items()}
    model = helpers.build_model(config, tensors, dtype)
    rng = np.random.default_rng(hd)
    a = [int(t) for t in rng.integers(0, 300, size=170)]
    b = [int(t) for t in rng.integers(0, 300, size=80)]
    want_a, want_b = plain_model.forward(config, tensors, np.asarray(a)), plain_model.forward(config, tensors, np.asarray(b))
    session = ReplaySession(model, max_tokens=320, block_size=page)
    got = session.step([{"id": "a", "tokens": a[:150], "want": [0, 77, 149]}])
    helpers.assert_close(got, want_a[[0, 77, 149]], dtype, f"head size {hd}: first portion")
    got = session.step([{"id": "a", "tokens": a[150:152], "want": [1]}, {"id": "b", "tokens": b[:60], "want": [59]}])
    helpers.assert_close(got, np.stack([want_a[151], want_b[59]]), dtype, f"head size {hd}: two tokens beside a prompt")
    for i in range(152, 170):
        entries = [{"id": "a", "tokens": [a[i]], "want": [0]}, {"id": "b", "tokens": [b[i - 92]], "want": [0]}]
        got = session.step(entries)
        helpers.assert_close(got, np.stack([want_a[i], want_b[i - 92]]), dtype, f"head size {hd}: decoding at {i}")
    session.runner.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_single_token_prompt(dtype):
    session, tensors = _session("B", dtype, 256)
    tokens = helpers.random_tokens(helpers.TINY_B, 5, seed=14)
    want = _reference("B", tensors, tokens)
    got = [session.step([{"id": "one", "tokens": tokens[:1], "want": [0]}])]
    got.append(session.step([{"id": "one", "tokens": tokens[1:3], "want": [0, 1]}]))
    got.append(session.step([{"id": "one", "tokens": tokens[3:], "want": [0, 1]}], end=["one"]))
    helpers.assert_close(np.concatenate(got), want, dtype, "first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    """A short prompt, then 400 tokens decoded one by one, in config C (pages of 16)."""
    session, tensors = _session("C", dtype, 512)
    tokens = helpers.random_tokens(helpers.TINY_C, 420, seed=15)
    want = _reference("C", tensors, tokens)
    got = [session.step([{"id": "r", "tokens": tokens[:20], "want": [19]}])]
    for i in range(20, len(tokens)):
        got.append(session.step([{"id": "r", "tokens": [tokens[i]], "want": [0]}]))
    helpers.assert_close(np.concatenate(got), want[19:], dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_prompt_of_2500_tokens_in_two_portions_then_decoding(dtype):
    """Config D with room for longer sequences: 1,300 tokens, then 1,190 above them (the second
    portion's query blocks start over 1,300 cached keys, 40 key tiles deep at the end), then ten
    tokens one by one; every 97th position and the last ones against the plain implementation."""
    from paged_kv_serving_b200.engine.replay import ReplaySession

    config = dict(helpers.TINY_D, max_seq_len=4096)
    tensors = plain_model.random_tensors(config, seed=21, std=0.05)
    if dtype == "bfloat16":
        tensors = {k: (plain_model.round_to_bfloat16(v) if v.ndim == 2 else v) for k, v in tensors.items()}
    model = helpers.build_model(config, tensors, dtype)
    tokens = helpers.random_tokens(config, 2500, seed=22)
    want = plain_model.forward(config, tensors, np.asarray(tokens))
    session = ReplaySession(model, max_tokens=2560, block_size=16)
    first = list(range(0, 1300, 97)) + [1299]
    got = session.step([{"id": "r", "tokens": tokens[:1300], "want": first}])
    helpers.assert_close(got, want[first], dtype, "first 1,300 tokens")
    second = list(range(5, 1190, 97)) + [1188, 1189]
    got = session.step([{"id": "r", "tokens": tokens[1300:2490], "want": second}])
    helpers.assert_close(got, want[[1300 + i for i in second]], dtype, "1,190 tokens above 1,300 cached ones")
    got = [session.step([{"id": "r", "tokens": [t], "want": [0]}]) for t in tokens[2490:]]
    helpers.assert_close(np.concatenate(got), want[2490:], dtype, "decoding at 2,490 tokens of context")
    session.runner.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_captured_decode_steps_equal_eager_ones(dtype):
    """Decode-only steps replay CUDA graphs; the same steps without graphs give the same logits,
    also when the number of live requests changes from step to step."""
    from paged_kv_serving_b200.engine.replay import ReplaySession

    tensors = helpers.tensors_for("C", dtype)
    model = helpers.build_model(helpers.TINY_C, tensors, dtype)
    prompts = [helpers.random_tokens(helpers.TINY_C, n, seed=70 + n) for n in (40, 75, 23)]
    outputs = []
    for use_graphs in (True, False):
        session = ReplaySession(model, max_tokens=512, block_size=16)
        session.runner.use_graphs = use_graphs
        got = []
        for i, p in enumerate(prompts):
            session.step([{"id": f"s{i}", "tokens": p[:20], "want": []}])
        for k in range(20, 75):
            entries = [{"id": f"s{i}", "tokens": [p[k]], "want": [0]} for i, p in enumerate(prompts) if k < len(p)]
            got.append(session.step(entries))
        if use_graphs:
            assert len(session.runner._graphs) >= 3        # batches of 3, 2 and 1 requests
        outputs.append(np.concatenate(got))
    want = plain_model.forward(helpers.TINY_C, tensors, prompts[1])
    helpers.assert_close(outputs[0][-1:], want[74:75], dtype, "graph decode against plain")
    assert np.abs(outputs[0] - outputs[1]).max() <= (1e-5 if dtype == "float32" else helpers.bf16_atol(outputs[1]))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ("B", "D"))
def test_random_traces(name, dtype):
    """Seeded random traces: up to four live requests of 2 to 300 tokens, each step a random subset
    of them with portions of random size (half of them a single token), wanted places anywhere,
    a pool that only just holds four requests, so pages pass from request to request."""
    from paged_kv_serving_b200.engine.replay import ReplaySession

    config = helpers.CONFIGS[name]
    longest = min(300, config["max_seq_len"])
    tensors = helpers.tensors_for(name, dtype)
    model = helpers.build_model(config, tensors, dtype)
    for seed in range(12):
        rng = np.random.default_rng(10_000 + seed)
        session = ReplaySession(model, max_tokens=4 * (-(-longest // 64) * 64), block_size=helpers.PAGE_SIZE[name])
        todo = [helpers.random_tokens(config, int(rng.integers(2, longest + 1)), seed=int(rng.integers(0, 10 ** 6)))
                for _ in range(int(rng.integers(3, 9)))]
        wants, live, started, steps = {}, {}, 0, 0
        while todo or live:
            while todo and len(live) < 4 and (not live or rng.random() < 0.5):
                tokens = todo.pop()
                live[f"r{started}"] = [tokens, 0]
                wants[f"r{started}"] = plain_model.forward(config, tensors, np.asarray(tokens))
                started += 1
            entries, expect, ended = [], [], []
            for request, state in live.items():
                if len(live) > 1 and rng.random() < 0.25:
                    continue                                  # left out of this step
                tokens, done = state
                left = len(tokens) - done
                size = 1 if rng.random() < 0.4 else int(rng.integers(1, 1 + min(left, 160)))
                want = sorted({int(x) for x in rng.integers(0, size, size=int(rng.integers(0, 4)))})
                if done + size == len(tokens) and size - 1 not in want:
                    want.append(size - 1)
                entries.append({"id": request, "tokens": tokens[done:done + size], "want": want})
                expect += [wants[request][done + i] for i in want]
                state[1] = done + size
                if state[1] == len(tokens):
                    ended.append(request)
            if not entries:
                continue
            got = session.step(entries, end=ended)
            for request in ended:
                del live[request]
            steps += 1
            if expect:
                helpers.assert_close(got, np.stack(expect), dtype, f"random trace {seed} of {name}, step {steps}: "
                                     f"{[(e['id'], len(e['tokens']), e['want']) for e in entries]}")
        session.check_invariants()
        session.runner.check_status()


def test_only_so_many_captured_graphs_are_kept():
    """A runner keeps a bounded number of captured graphs and drops the one replayed longest ago;
    a size class whose graph was dropped is captured again and gives the right logits."""
    from paged_kv_serving_b200.engine.replay import ReplaySession

    dtype = "bfloat16"
    tensors = helpers.tensors_for("C", dtype)
    model = helpers.build_model(helpers.TINY_C, tensors, dtype)
    prompts = {name: helpers.random_tokens(helpers.TINY_C, 60, seed=170 + i) for i, name in enumerate("abcde")}
    wants = {name: plain_model.forward(helpers.TINY_C, tensors, p) for name, p in prompts.items()}
    session = ReplaySession(model, max_tokens=512, block_size=16)
    session.runner.MAX_GRAPHS = 2
    at = {}

    def start(names):
        session.step([{"id": n, "tokens": prompts[n][:20], "want": []} for n in names])
        at.update({n: 20 for n in names})

    def decode(names, steps, end=()):
        for step in range(steps):
            got = session.step([{"id": n, "tokens": [prompts[n][at[n]]], "want": [0]} for n in names],
                               end=list(end) if step == steps - 1 else [])
            helpers.assert_close(got, np.stack([wants[n][at[n]] for n in names]), dtype, f"{names} at {at[names[0]]}")
            for n in names:
                at[n] += 1
            assert len(session.runner._graphs) <= 2

    start("abc")
    decode("abc", 3, end="c")          # three rows: the four-row class
    decode("ab", 3, end="b")           # the two-row class
    classes = set(session.runner._graphs)
    decode("a", 3)                     # the one-row class: the four-row graph goes
    assert len(session.runner._graphs) == 2 and set(session.runner._graphs) != classes
    start("de")
    decode("ade", 3)                   # three rows again: captured again, the two-row graph goes
    session.runner.check_status()


@pytest.mark.parametrize("use_graphs", [True, False])
def test_even_shares_decode_attention_in_the_engine(monkeypatch, use_graphs):
    """Decode steps of config D in bfloat16 with the even-shares decode kernel forced: three
    requests of unequal length, so that a block's range ends inside one request and begins in
    the next; against the plain implementation."""
    from paged_kv_serving_b200.engine.replay import ReplaySession
    from paged_kv_serving_b200.parts.attention import PagedAttention

    monkeypatch.setattr(PagedAttention, "FLAT_DECODE", "always")
    tensors = helpers.tensors_for("D", "bfloat16")
    model = helpers.build_model(helpers.TINY_D, tensors, "bfloat16")
    prompts = [helpers.random_tokens(helpers.TINY_D, n, seed=90 + n) for n in (330, 140, 70)]
    session = ReplaySession(model, max_tokens=1024, block_size=16)
    session.runner.use_graphs = use_graphs
    session.runner.storage.fill(float("nan"))
    for i, p in enumerate(prompts):
        session.step([{"id": f"s{i}", "tokens": p[:len(p) - 40], "want": []}])
    got = {i: [] for i in range(len(prompts))}
    for k in range(40, 0, -1):
        entries = [{"id": f"s{i}", "tokens": [p[len(p) - k]], "want": [0]} for i, p in enumerate(prompts)]
        logits = session.step(entries)
        for i in range(len(prompts)):
            got[i].append(logits[i])
    for i, p in enumerate(prompts):
        want = plain_model.forward(helpers.TINY_D, tensors, p)
        helpers.assert_close(np.stack(got[i]), want[len(p) - 40:], "bfloat16", f"even shares, request {i}")


def test_decode_steps_of_9_to_20_rows_on_the_streaming_tensor_core_kernel():
    """The tcgen05 weight-streaming product stands behind a switch (``ops.gemm.STREAM_ROWS``). With
    the switch on, decode steps of 9 to 20 rows of the head-64 model run their products, with the
    fused residual, norm and activation epilogues, on that kernel: the logits must be the plain
    implementation's as with the switch off."""
    from paged_kv_serving_b200 import ops
    from paged_kv_serving_b200.ops import gemm

    name, dtype = "D", "bfloat16"
    config = helpers.CONFIGS[name]
    before, original = gemm.STREAM_ROWS, ops.gemm_stream
    calls = []
    ops.gemm_stream = lambda *args, **options: calls.append(options.get("residual") is not None) or original(*args, **options)
    gemm.STREAM_ROWS = 32
    try:
        session, tensors = _session(name, dtype, 20 * 64)
        prompts = [helpers.random_tokens(config, 30 + i, seed=500 + i) for i in range(20)]
        wants = [_reference(name, tensors, p) for p in prompts]
        session.step([{"id": f"r{i}", "tokens": p[:20], "want": []} for i, p in enumerate(prompts)])
        for position in range(20, 30):
            live = range(20) if position < 25 else range(9)            # 20 rows, then 9
            got = session.step([{"id": f"r{i}", "tokens": [prompts[i][position]], "want": [0]} for i in live],
                               end=[f"r{i}" for i in range(9, 20)] if position == 24 else [])
            want = np.stack([wants[i][position] for i in live])
            helpers.assert_close(got, want, dtype, f"streaming kernel, {len(live)} rows at position {position}")
        session.runner.check_status()
    finally:
        gemm.STREAM_ROWS, ops.gemm_stream = before, original
    assert any(calls) and not all(calls), "plain and residual epilogues of the streaming kernel must have run"


def test_short_portions_take_the_library_product_and_the_activation_kernel(monkeypatch):
    """The routing as shipped: a portion of 150 tokens is far below the row count from which the
    fused gate/up kernel pays, so its gate/up product goes to the library and the activation
    kernel follows; the logits are the plain implementation's either way."""
    from paged_kv_serving_b200 import ops
    from paged_kv_serving_b200.ops import gemm

    name, dtype = "D", "bfloat16"
    config = helpers.CONFIGS[name]
    calls = {"fused": 0, "activation": 0}
    fused, activation = ops.gemm_tcgen05, ops.silu_mul

    def count_fused(*args, **options):
        calls["fused"] += 1 if (len(args) > 3 and args[3] == "silu_mul") or options.get("epilogue") == "silu_mul" else 0
        return fused(*args, **options)

    def count_activation(*args, **options):
        calls["activation"] += 1
        return activation(*args, **options)

    monkeypatch.setattr(ops, "gemm_tcgen05", count_fused)
    monkeypatch.setattr(ops, "silu_mul", count_activation)
    tokens = helpers.random_tokens(config, 150, seed=77)
    for threshold, expect_fused in ((1536, False), (gemm.TCGEN05_MIN_ROWS, True)):
        monkeypatch.setattr(gemm, "SILU_TCGEN05_MIN_ROWS", threshold)
        calls["fused"] = calls["activation"] = 0
        session, tensors = _session(name, dtype, 256)
        got = session.step([{"id": "a", "tokens": tokens, "want": list(range(150))}])
        helpers.assert_close(got, _reference(name, tensors, tokens), dtype, f"gate/up routing at threshold {threshold}")
        assert (calls["fused"] > 0) == expect_fused and (calls["activation"] > 0) != expect_fused, calls
        session.runner.check_status()
