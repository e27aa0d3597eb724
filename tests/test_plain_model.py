"""The plain implementation against the reference's own code (golden files) and its own parts."""

import sys
from pathlib import Path

import numpy as np
import pytest

import plain_model

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import make_golden  # noqa: E402

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["mha_tied", "gqa_untied"])
def test_plain_forward_matches_reference_golden(name):
    config, tensors, tokens = make_golden.golden_inputs(name)
    want = np.load(GOLDEN / f"{name}.npy")
    got = plain_model.forward(config, tensors, tokens)
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= 1e-5


def test_plain_sampler_matches_reference_golden():
    """2,000 seeded cases whose token ids the reference's own ``sample_token`` produced
    (src/paged_kv_serving/engine/sampling.py:56-74): greedy, temperature, nucleus, ties."""
    want = np.load(GOLDEN / "sampling.npy")
    assert want.shape == (make_golden.SAMPLING_CASES,)
    sampled = 0
    for number in range(make_golden.SAMPLING_CASES):
        logits, temperature, top_p, generator = make_golden.sampling_case(number)
        if temperature < plain_model.GREEDY_TEMPERATURE:
            got = plain_model.greedy_token(logits)          # a greedy token draws no number
        else:
            got = plain_model.sample_token(logits, temperature, top_p, float(generator.random()))
            sampled += 1
        assert got == int(want[number]), f"case {number}"
    assert sampled > 1500


def test_forward_is_causal():
    config, tensors, tokens = make_golden.golden_inputs("gqa_untied")
    full = plain_model.forward(config, tensors, tokens)
    prefix = plain_model.forward(config, tensors, tokens[:9])
    assert np.abs(full[:9] - prefix).max() <= 1e-5


def test_rms_norm_unit_rms_and_eps():
    x = np.random.default_rng(0).standard_normal((5, 64)).astype(np.float32) * 7
    y = plain_model.rms_norm(x, np.ones(64, np.float32), 1e-6)
    assert np.allclose(np.sqrt((y * y).mean(-1)), 1.0, atol=1e-4)
    assert np.all(np.isfinite(plain_model.rms_norm(np.zeros((1, 8), np.float32), np.ones(8, np.float32), 1e-5)))


def test_silu_is_finite_at_extremes():
    x = np.array([-1e4, -60.0, 0.0, 60.0, 1e4], dtype=np.float32)
    y = plain_model.silu(x)
    assert np.all(np.isfinite(y)) and y[2] == 0.0 and y[-1] == pytest.approx(1e4)


def test_rope_keeps_norm_and_depends_on_distance_only():
    rng = np.random.default_rng(1)
    cos, sin = plain_model.rope_tables(64, 16, 10000.0)
    q = rng.standard_normal((1, 1, 16)).astype(np.float32)
    k = rng.standard_normal((1, 1, 16)).astype(np.float32)
    dots = []
    for offset in (0, 5, 20):
        qr = plain_model.apply_rope(q, np.array([7 + offset]), cos, sin)
        kr = plain_model.apply_rope(k, np.array([3 + offset]), cos, sin)
        assert np.linalg.norm(qr) == pytest.approx(np.linalg.norm(q), rel=1e-5)
        dots.append(float((qr * kr).sum()))
    assert dots[0] == pytest.approx(dots[1], abs=1e-4) and dots[0] == pytest.approx(dots[2], abs=1e-4)
    with pytest.raises(ValueError):
        plain_model.rope_tables(8, 7, 10000.0)


def test_grouped_attention_equals_expanded_multi_head():
    rng = np.random.default_rng(2)
    q = rng.standard_normal((9, 4, 8)).astype(np.float32)
    k = rng.standard_normal((9, 2, 8)).astype(np.float32)
    v = rng.standard_normal((9, 2, 8)).astype(np.float32)
    grouped = plain_model.causal_attention(q, k, v, 0.35)
    expanded = plain_model.causal_attention(q, np.repeat(k, 2, axis=1), np.repeat(v, 2, axis=1), 0.35)
    assert np.abs(grouped - expanded).max() <= 1e-6


def test_window_masks_old_keys():
    rng = np.random.default_rng(3)
    q = rng.standard_normal((12, 1, 4)).astype(np.float32)
    k = rng.standard_normal((12, 1, 4)).astype(np.float32)
    v = rng.standard_normal((12, 1, 4)).astype(np.float32)
    windowed = plain_model.causal_attention(q, k, v, 0.5, window=3)
    last = plain_model.causal_attention(q[9:], k[9:], v[9:], 0.5)
    assert np.abs(windowed[11] - last[2]).max() <= 1e-6


def test_sampling_plain():
    logits = np.array([0.1, 2.0, 2.0, -1.0], dtype=np.float32)
    assert plain_model.greedy_token(logits) == 1
    p = plain_model.top_p_filter(np.array([0.5, 0.3, 0.15, 0.05], np.float32), 0.7)
    assert np.count_nonzero(p) == 2 and p.sum() == pytest.approx(1.0)
    assert plain_model.sample_token(logits, 1e-6, 1.0, 0.99) == 1
    counts = np.zeros(4)
    rng = np.random.default_rng(0)
    for _ in range(400):
        counts[plain_model.sample_token(logits, 0.8, 1.0, float(rng.random()))] += 1
    assert counts[1] > counts[0] > counts[3]


def test_round_to_bfloat16_matches_torch():
    import torch

    x = np.random.default_rng(4).standard_normal(1000).astype(np.float32)
    want = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(plain_model.round_to_bfloat16(x), want)
