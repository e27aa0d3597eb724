"""Logits at the layer sizes the benchmark runs, against the plain implementation (``-m gpu``).

Two layers at the full widths of three Llama-family shapes (hidden size, feed-forward size, head
counts, head size and vocabulary as the benchmark presets have them), with random weights, in
float32 and in bfloat16, through ``ReplaySession``: the step function, cache manager and kernels
that generation uses. These are the sizes at which the kernels take branches that tiny models
never reach: products whose tiles are cut into even ranges over all SMs, inner sizes of 14,336,
a vocabulary of 128,256 columns, head size 128, forty heads without grouping, and decode steps of
9 to 64 rows, which go to other kernels than steps of up to 8 rows.

Per shape and type, one model is built and replayed
  * whole: a prompt of 300 tokens in one step;
  * most of it in one step, the last 32 tokens one by one;
  * in portions of 2, 130, 16 and 2 tokens, and a prompt of 150 tokens in one step;
  * mixed: up to four live requests, portions of some beside decoded tokens of others, in a pool
    of 512 tokens that the requests need twice over, so pages are used again;
  * decode steps of 64, 16, 9, 8 and 1 rows.
The reference pins its numbers at the size it serves in the same manner
(tests/property/test_equivalence.py:33-141 of rouviere-german/paged-kv-serving).
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import helpers
import plain_model

pytestmark = pytest.mark.gpu

SHAPES = {
    "8b": {"architecture": "LlamaToyDecoder", "vocab_size": 128256, "d_model": 4096, "n_layers": 2, "n_heads": 32,
           "n_kv_heads": 8, "head_dim": 128, "d_ff": 14336, "max_seq_len": 512, "rope_theta": 500000.0,
           "norm_eps": 1e-5, "tie_embeddings": False},
    "13b": {"architecture": "LlamaToyDecoder", "vocab_size": 32000, "d_model": 5120, "n_layers": 2, "n_heads": 40,
            "n_kv_heads": 40, "head_dim": 128, "d_ff": 13824, "max_seq_len": 512, "rope_theta": 10000.0,
            "norm_eps": 1e-5, "tie_embeddings": False},
    "1b": {"architecture": "LlamaToyDecoder", "vocab_size": 128256, "d_model": 2048, "n_layers": 2, "n_heads": 32,
           "n_kv_heads": 8, "head_dim": 64, "d_ff": 8192, "max_seq_len": 512, "rope_theta": 500000.0,
           "norm_eps": 1e-5, "tie_embeddings": True},
}
LENGTHS = {"s0": 300, "s1": 150, "s2": 130, "s3": 70, "d0": 45, "d1": 45, "d2": 45, "d3": 45}

# Bounds. float32: the reference's own bound for paged against dense logits. bfloat16: the
# suite's bound (2.4 % of the largest logit of the compared rows plus a small floor).
F32_ATOL = 1e-4
bf16_atol = helpers.bf16_atol


def _weights(config: dict, dtype: str, seed: int):
    """Random tensors drawn on the GPU (matrices N(0, 0.02), norm weights near one), as float32
    NumPy arrays for the plain implementation; for bfloat16 the matrices are rounded first, so
    both sides hold the same values."""
    shapes = plain_model.tensor_shapes(config)
    generator = torch.Generator(device="cuda")
    generator.manual_seed(seed)
    out = {}
    for name in sorted(shapes):
        shape = shapes[name]
        if len(shape) == 1:
            values = 1.0 + 0.1 * torch.randn(shape, device="cuda", generator=generator)
        else:
            values = torch.randn(shape, device="cuda", generator=generator) * 0.02
            if dtype == "bfloat16":
                values = values.to(torch.bfloat16).float()
        out[name] = values.cpu().numpy()
    return out


class Trace:
    """Steps of one session and, for every wanted row, whose logits at which position it is."""

    def __init__(self) -> None:
        self.steps: list[tuple[list[dict], list[str], list[tuple[str, int]]]] = []

    def add(self, entries: list[tuple[str, str, int, int, list[int]]], end: tuple[str, ...] = ()) -> None:
        """``entries``: (request id, sequence, first position, token count, wanted places)."""
        records, checks = [], []
        for request, sequence, first, count, want in entries:
            records.append({"id": request, "seq": sequence, "first": first, "count": count, "want": list(want)})
            checks += [(sequence, first + place) for place in want]
        self.steps.append((records, list(end), checks))


def _single_request_trace() -> Trace:
    trace = Trace()
    trace.add([("whole", "s0", 0, 300, [0, 150, 299])], end=("whole",))
    trace.add([("tail", "s0", 0, 268, [267])])
    for position in range(268, 300):
        trace.add([("tail", "s0", position, 1, [0])], end=("tail",) if position == 299 else ())
    first = 0
    for count in (2, 130, 16, 2):
        trace.add([("cut", "s1", first, count, [count - 1])], end=("cut",) if first + count == 150 else ())
        first += count
    trace.add([("one-fifty", "s1", 0, 150, [0, 149])], end=("one-fifty",))
    return trace


def _mixed_trace() -> tuple[Trace, int]:
    """Up to four live requests in a pool of 512 tokens (each request's length rounded up to 64);
    returns the trace and the number of tokens all requests need together."""
    order = ["s1", "s3", "d0", "s2", "d1", "s3", "d2", "s1", "d3", "s2"]
    rng = np.random.default_rng(17)
    trace = Trace()
    waiting = list(enumerate(order))
    live: list[tuple[str, str]] = []
    progress: dict[str, int] = {}
    room = lambda: 512 - sum(-(-LENGTHS[seq] // 64) * 64 for _, seq in live)
    while waiting or live:
        while waiting and len(live) < 4 and -(-LENGTHS[waiting[0][1]] // 64) * 64 <= room():
            index, seq = waiting.pop(0)
            live.append((f"m{index}", seq))
            progress[f"m{index}"] = 0
        entries, finished = [], []
        for request, seq in live:
            remaining = LENGTHS[seq] - progress[request]
            count = 1 if remaining <= 6 else int(min(remaining - 6, rng.integers(2, 60)))
            entries.append((request, seq, progress[request], count, [count - 1]))
            progress[request] += count
            if progress[request] == LENGTHS[seq]:
                finished.append(request)
        trace.add(entries, end=tuple(finished))
        live = [(request, seq) for request, seq in live if request not in finished]
    return trace, sum(-(-LENGTHS[seq] // 64) * 64 for seq in order)


def _decode_rows_trace() -> Trace:
    """64 requests (16 copies of four sequences) filled 16 at a time, then decode steps of
    64, 16, 9, 8 and 1 rows."""
    trace = Trace()
    requests = [(f"r{i}", f"d{i % 4}") for i in range(64)]
    for first in range(0, 64, 16):
        trace.add([(request, seq, 0, 40, []) for request, seq in requests[first:first + 16]])
    position = 40
    for rows in (64, 16, 9, 8, 1):
        ended = tuple(request for request, _ in requests[rows:])
        requests = requests[:rows]
        if ended:
            trace.add([], end=ended)
        trace.add([(request, seq, position, 1, [0]) for request, seq in requests])
        position += 1
    trace.add([], end=tuple(request for request, _ in requests))
    return trace


def _replay(session, trace: Trace, tokens: dict, plain_rows: dict, dtype: str, what: str) -> float:
    worst = 0.0
    for number, (records, end, checks) in enumerate(trace.steps):
        entries = [{"id": r["id"], "tokens": tokens[r["seq"]][r["first"]:r["first"] + r["count"]], "want": r["want"]}
                   for r in records]
        got = session.step(entries, end=end)
        if not checks:
            assert got is None
            continue
        want = np.stack([plain_rows[check] for check in checks])
        atol = F32_ATOL if dtype == "float32" else bf16_atol(want)
        worst = max(worst, helpers.assert_close(got, want, dtype, f"{what}, step {number} {checks[:4]}", atol=atol) / atol)
        session.check_invariants()
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", ["1b", "8b", "13b"])
def test_logits_at_benchmark_layer_sizes(shape, dtype):
    from paged_kv_serving_b200.engine.replay import ReplaySession

    config = SHAPES[shape]
    tensors = _weights(config, dtype, seed=len(shape) + config["d_model"])
    rng = np.random.default_rng(3)
    tokens = {name: [int(t) for t in rng.integers(0, config["vocab_size"], size=n)] for name, n in LENGTHS.items()}
    single, (mixed, mixed_need), rows = _single_request_trace(), _mixed_trace(), _decode_rows_trace()
    assert mixed_need > 2 * 512 - 64, "the mixed requests must need the pool about twice over"
    assert max(len(records) for records, _, _ in mixed.steps) == 4, "four requests must be live together"

    # the plain logits at every place some trace asks for, one whole-sequence pass per sequence
    wanted: dict[str, set[int]] = {}
    for trace in (single, mixed, rows):
        for _, _, checks in trace.steps:
            for seq, position in checks:
                wanted.setdefault(seq, set()).add(position)
    plain_rows = {}
    for seq, positions in wanted.items():
        ordered = sorted(positions)
        logits = plain_model.forward(config, tensors, tokens[seq], rows=ordered)
        plain_rows.update({(seq, position): logits[i] for i, position in enumerate(ordered)})

    model = helpers.build_model(config, tensors, dtype)
    del tensors
    worst = {}
    session = ReplaySession(model, max_tokens=512, block_size=16)
    worst["single"] = _replay(session, single, tokens, plain_rows, dtype, f"{shape} {dtype} single requests")
    assert session.cache.num_free_blocks == session.num_blocks
    worst["mixed"] = _replay(session, mixed, tokens, plain_rows, dtype, f"{shape} {dtype} mixed requests")
    assert session.cache.num_free_blocks == session.num_blocks
    del session
    session = ReplaySession(model, max_tokens=64 * 64, block_size=16, max_live=64)
    worst["rows"] = _replay(session, rows, tokens, plain_rows, dtype, f"{shape} {dtype} decode rows")
    session.runner.check_status()
    print(f"\n[{shape} {dtype}] largest gap as a share of the bound: "
          + ", ".join(f"{k} {v:.3f}" for k, v in worst.items()))
