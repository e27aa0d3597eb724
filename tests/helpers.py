"""Shared pieces of the tests: the two tiny configurations, model builders, trace drivers."""

from __future__ import annotations

import numpy as np
import torch

import plain_model

# Two tiny configurations of the architecture that differ in every size and option
# (head counts and groups, sizes that are no power of two, layers, vocabulary, eps, rope base,
# tied or separate head). Page sizes differ too (see PAGE_SIZE).
TINY_A = {
    "architecture": "LlamaToyDecoder", "vocab_size": 256, "d_model": 64, "n_layers": 2, "n_heads": 4,
    "n_kv_heads": 2, "head_dim": 16, "d_ff": 172, "max_seq_len": 128, "rope_theta": 10000.0,
    "norm_eps": 1e-5, "tie_embeddings": False,
}
TINY_B = {
    "architecture": "LlamaToyDecoder", "vocab_size": 384, "d_model": 96, "n_layers": 3, "n_heads": 3,
    "n_kv_heads": 3, "head_dim": 32, "d_ff": 256, "max_seq_len": 256, "rope_theta": 500000.0,
    "norm_eps": 1e-6, "tie_embeddings": True,
}
# A third shape for longer sequences: head size 48 (a step of 16, no power of two), 6 query heads
# in 2 groups of 3, a vocabulary and widths that are no powers of two.
TINY_C = {
    "architecture": "LlamaToyDecoder", "vocab_size": 331, "d_model": 120, "n_layers": 2, "n_heads": 6,
    "n_kv_heads": 2, "head_dim": 48, "d_ff": 200, "max_seq_len": 1024, "rope_theta": 50000.0,
    "norm_eps": 3e-6, "tie_embeddings": True,
}
# A fourth shape at the sizes the Blackwell-specific kernels take (head size 64, pages of 16,
# widths that are multiples of 8): in bfloat16 its prompts run through the tcgen05 matrix product,
# the tcgen05 prefill attention and the TMA-fed decode attention.
TINY_D = {
    "architecture": "LlamaToyDecoder", "vocab_size": 512, "d_model": 256, "n_layers": 2, "n_heads": 8,
    "n_kv_heads": 2, "head_dim": 64, "d_ff": 392, "max_seq_len": 1024, "rope_theta": 500000.0,
    "norm_eps": 1e-5, "tie_embeddings": False,
}
PAGE_SIZE = {"A": 4, "B": 8, "C": 16, "D": 16}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
WEIGHT_SEED = {"A": 0, "B": 2, "C": 5, "D": 7}

# Tolerances. float32: the reference's own bound for paged against dense logits
# (tests/property/test_equivalence.py:33-34 of the reference). bfloat16: activations carry 8 bits
# of mantissa (relative 2^-8 per rounding); with a few roundings per layer the bound was first set
# to 3 % of the largest logit of the compared rows plus a small floor, before any GPU run. Every
# comparison of the suite (tiny models, two layers at the widths of 1-, 8- and 13-billion-parameter
# models, every way of cutting and batching) then stayed below 1.9 %, and the bound was tightened
# to 2.4 %: room for a quarter more than the worst case seen, none for a wrong key or page.
F32_ATOL = 1e-4


def bf16_atol(reference: np.ndarray) -> float:
    return 0.024 * float(np.abs(reference).max()) + 2e-3


def tensors_for(name: str, dtype: str, std: float | None = None, norm_jitter: float = 0.1) -> dict[str, np.ndarray]:
    """Random float32 tensors of a tiny configuration; for bfloat16 the matrices are rounded so
    that the plain implementation and the engine hold exactly the same values."""
    if std is None:
        std = 0.04 if name == "D" else 0.08     # wider layers: keep activations at the same scale
    tensors = plain_model.random_tensors(CONFIGS[name], WEIGHT_SEED[name], std=std, norm_jitter=norm_jitter)
    if dtype == "bfloat16":
        tensors = {k: (plain_model.round_to_bfloat16(v) if v.ndim == 2 else v) for k, v in tensors.items()}
    return tensors


def build_model(config: dict, tensors: dict[str, np.ndarray], dtype: str):
    from paged_kv_serving_b200.config import ModelConfig
    from paged_kv_serving_b200.models.decoder import DecoderModel

    torch_tensors = {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in tensors.items()}
    return DecoderModel.from_tensors(ModelConfig.from_dict(config), torch_tensors, dtype=dtype, device="cuda")


def random_tokens(config: dict, count: int, seed: int) -> list[int]:
    return [int(t) for t in np.random.default_rng(seed).integers(0, config["vocab_size"], size=count)]


#: The largest gap met so far as a share of its bound, per type (printed at the end of a run: it
#: shows how much room the bounds leave).
WORST_SHARE: dict[str, float] = {}


def assert_close(got: np.ndarray, want: np.ndarray, dtype: str, what: str, atol: float | None = None) -> float:
    """Raises when ``got`` misses ``want`` by more than the bound of ``dtype`` (or ``atol``);
    returns the largest gap."""
    if atol is None:
        atol = F32_ATOL if dtype == "float32" else bf16_atol(want)
    gap = np.abs(got.astype(np.float64) - want.astype(np.float64))
    worst = float(gap.max())
    WORST_SHARE[dtype] = max(WORST_SHARE.get(dtype, 0.0), worst / atol if atol > 0 else 0.0)
    if not worst <= atol:
        row, col = np.unravel_index(int(gap.argmax()), gap.shape)
        first_bad = int(np.argmax(gap.max(axis=-1) > atol))
        raise AssertionError(f"{what}: max |gap| {worst:.3e} > {atol:.3e} at row {row}, column {col}; "
                             f"first row beyond the bound: {first_bad}")
    return worst


def assert_greedy_tokens(config: dict, tensors: dict[str, np.ndarray], prompt, got, dtype: str, what: str) -> None:
    """Greedy tokens of the engine against the plain implementation. In float32 they are equal. In
    bfloat16 a token may differ from the plain choice only at a near tie: the plain logits are
    computed on the engine's own tokens (one whole-sequence pass), and at every place the logit of
    the engine's token must lie within the rounding bound of the plain maximum (twice the bound of
    one logit, since both may be off). A wrong cache or kernel moves logits by far more."""
    got = [int(t) for t in got]
    if dtype == "float32":
        want = plain_model.generate(config, tensors, prompt, len(got))
        assert got == want, f"{what}: float32 tokens {got} differ from the plain implementation's {want}"
        return
    rows = plain_model.forward(config, tensors, list(prompt) + got[:-1])[len(prompt) - 1:]
    for place, (token, row) in enumerate(zip(got, rows)):
        slack = 2 * bf16_atol(row)
        assert row[token] >= row.max() - slack, (
            f"{what}: token {place} is {token} (plain logit {row[token]:.4f}) but the plain maximum is "
            f"{row.max():.4f} at {int(row.argmax())}; allowed gap {slack:.4f}")
