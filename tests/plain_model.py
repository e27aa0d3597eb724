"""Plain, slow, cache-free implementation of the Llama-style toy decoder (NumPy, float32).

This file is the yardstick of the test-suite. It shares no code with the product package: it
reads a configuration as a plain ``dict`` (the keys of ``config.json``) and weights as a plain
``dict`` of NumPy arrays keyed by tensor name, runs whole sequences with dense attention and no
cache, and has one function per part. Every function cites the place in the reference project
(rouviere-german/paged-kv-serving, paths relative to its root) whose formula it restates.

Where the reference is multi-head and tied only, the two generalisations used here are the
grouped-query head mapping (query head ``h`` reads key/value head ``h // (n_heads // n_kv_heads)``)
and an optional separate ``lm_head`` matrix; both reduce to the reference when
``n_kv_heads == n_heads`` and ``tie_embeddings`` is true (checked against the reference's own
code once, see ``tests/golden``).
"""

from __future__ import annotations

import math

import numpy as np

F32 = np.float32


# --------------------------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------------------------


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """``x / sqrt(mean(x^2) + eps) * weight`` over the last axis, float32.

    Reference: src/paged_kv_serving/engine/model.py:43-46 (eps inside the root, divide first,
    then multiply by the weight; no bias, weight not offset by one).
    """
    x = x.astype(F32)
    mean_square = np.mean(x * x, axis=-1, keepdims=True, dtype=F32)
    root = np.sqrt(mean_square + F32(eps)).astype(F32)
    return ((x / root) * weight.astype(F32)).astype(F32)


def silu(x: np.ndarray) -> np.ndarray:
    """``x * sigmoid(x)`` with the argument of ``exp`` clipped to [-60, 60].

    Reference: src/paged_kv_serving/engine/model.py:49-51.
    """
    x = x.astype(F32)
    clipped = np.clip(x, F32(-60.0), F32(60.0))
    return (x * (F32(1.0) / (F32(1.0) + np.exp(-clipped)))).astype(F32)


def rope_tables(max_positions: int, head_dim: int, theta: float) -> tuple[np.ndarray, np.ndarray]:
    """Cosine and sine tables ``(max_positions, head_dim // 2)``; angles in float64, cast to f32.

    Reference: src/paged_kv_serving/engine/model.py:60-67
    (``inv_freq_j = theta ** -(2 j / head_dim)``, ``angle[p, j] = p * inv_freq_j``).
    """
    if head_dim % 2:
        raise ValueError("head_dim must be even")
    half = head_dim // 2
    inv_freq = 1.0 / (float(theta) ** (np.arange(half, dtype=np.float64) * 2.0 / head_dim))
    angles = np.arange(max_positions, dtype=np.float64)[:, None] * inv_freq[None, :]
    return np.cos(angles).astype(F32), np.sin(angles).astype(F32)


def apply_rope(x: np.ndarray, positions: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """Half-split rotation of ``x (tokens, heads, head_dim)`` by each token's absolute position.

    Reference: src/paged_kv_serving/engine/model.py:70-81
    (``out = concat(left*cos - right*sin, right*cos + left*sin)``; not interleaved).
    """
    half = x.shape[-1] // 2
    c = cos[positions][:, None, :]
    s = sin[positions][:, None, :]
    left = x[..., :half]
    right = x[..., half:]
    return np.concatenate([left * c - right * s, right * c + left * s], axis=-1).astype(F32)


def softmax_rows(scores: np.ndarray) -> np.ndarray:
    """Softmax over the last axis. Reference: src/paged_kv_serving/engine/model.py:54-57."""
    shifted = scores - np.max(scores, axis=-1, keepdims=True)
    e = np.exp(shifted)
    return (e / np.sum(e, axis=-1, keepdims=True)).astype(F32)


def causal_attention(
    q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window: int | None = None
) -> np.ndarray:
    """Dense causal attention. ``q (T, H, hd)``, ``k, v (T, KV, hd)``; returns ``(T, H, hd)``.

    Reference: src/paged_kv_serving/engine/model.py:206-221 (scores ``q k^T * scale``; a key at a
    later position than the query is masked with -inf; one softmax; ``P v``). The grouped-query
    mapping (``H // KV`` consecutive query heads share one key/value head) is this engine's
    generalisation. ``window`` (a test-only generalisation, ``None`` for the reference's
    behaviour) also masks keys more than ``window - 1`` positions behind the query.
    """
    tokens, n_heads, head_dim = q.shape
    n_kv = k.shape[1]
    group = n_heads // n_kv
    out = np.zeros((tokens, n_heads, head_dim), dtype=F32)
    key_pos = np.arange(tokens)[None, :]
    query_pos = np.arange(tokens)[:, None]
    masked = key_pos > query_pos
    if window is not None:
        masked = masked | (key_pos <= query_pos - window)
    for h in range(n_heads):
        g = h // group
        scores = (q[:, h, :] @ k[:, g, :].T) * F32(scale)
        scores = np.where(masked, F32(-np.inf), scores).astype(F32)
        out[:, h, :] = softmax_rows(scores) @ v[:, g, :]
    return out


def project_qkv(normed: np.ndarray, qkv_proj: np.ndarray, n_heads: int, n_kv: int, head_dim: int):
    """Fused projection ``normed @ qkv_proj`` split into q, k, v.

    Reference: src/paged_kv_serving/engine/model.py:249-253 (weights are ``(in, out)``, used as
    ``x @ W``; columns are Q then K then V, head-major inside each). With fewer key/value heads
    the K and V column blocks are narrower: ``[Q: H*hd | K: KV*hd | V: KV*hd]``.
    """
    fused = (normed @ qkv_proj.astype(F32)).astype(F32)
    tokens = normed.shape[0]
    q_cols = n_heads * head_dim
    kv_cols = n_kv * head_dim
    q = fused[:, :q_cols].reshape(tokens, n_heads, head_dim)
    k = fused[:, q_cols : q_cols + kv_cols].reshape(tokens, n_kv, head_dim)
    v = fused[:, q_cols + kv_cols :].reshape(tokens, n_kv, head_dim)
    return q, k, v


def swiglu(normed: np.ndarray, gate: np.ndarray, up: np.ndarray, down: np.ndarray) -> np.ndarray:
    """``(silu(x @ gate) * (x @ up)) @ down``, no biases.

    Reference: src/paged_kv_serving/engine/model.py:256-259.
    """
    g = (normed @ gate.astype(F32)).astype(F32)
    u = (normed @ up.astype(F32)).astype(F32)
    return ((silu(g) * u).astype(F32) @ down.astype(F32)).astype(F32)


def embed(token_embedding: np.ndarray, token_ids: np.ndarray) -> np.ndarray:
    """Row gather. Reference: src/paged_kv_serving/engine/model.py:266-267."""
    return token_embedding.astype(F32)[token_ids]


def lm_head(hidden: np.ndarray, final_norm: np.ndarray, eps: float, head_matrix: np.ndarray) -> np.ndarray:
    """Final norm, then ``normed @ head_matrix.T`` with ``head_matrix (vocab, d_model)``.

    Reference: src/paged_kv_serving/engine/model.py:261-264 (tied: the matrix is the token
    embedding). An untied ``lm_head`` tensor of the same shape replaces it when
    ``tie_embeddings`` is false.
    """
    return (rms_norm(hidden, final_norm, eps) @ head_matrix.astype(F32).T).astype(F32)


# --------------------------------------------------------------------------------------------
# whole model
# --------------------------------------------------------------------------------------------


def config_sizes(config: dict) -> dict:
    """Fill the derived defaults of a ``config.json`` dictionary."""
    n_heads = int(config["n_heads"])
    out = dict(config)
    out.setdefault("n_kv_heads", n_heads)
    out.setdefault("head_dim", int(config["d_model"]) // n_heads)
    out.setdefault("rope_theta", 10000.0)
    out.setdefault("norm_eps", 1e-5)
    out.setdefault("tie_embeddings", True)
    return out


def forward(config: dict, tensors: dict[str, np.ndarray], token_ids, rows=None) -> np.ndarray:
    """Logits ``(T, vocab)`` at every position of one whole sequence, recomputed from scratch
    (with ``rows``, a list of positions, only those rows of the logits: the whole sequence still
    runs through the layers, the head is applied where asked).

    Reference: src/paged_kv_serving/engine/model.py:269-288 (embed; per layer: pre-norm,
    fused QKV, RoPE on q and k, causal attention with scale ``1/sqrt(head_dim)``, output
    projection added to the stream, pre-norm SwiGLU added to the stream; final norm; head).
    """
    c = config_sizes(config)
    ids = np.asarray(token_ids, dtype=np.int64)
    if ids.ndim != 1 or ids.size == 0:
        raise ValueError("token_ids must be a non-empty 1-D sequence")
    if ids.size > c["max_seq_len"]:
        raise ValueError("sequence longer than max_seq_len")
    n_heads, n_kv, head_dim = int(c["n_heads"]), int(c["n_kv_heads"]), int(c["head_dim"])
    eps = float(c["norm_eps"])
    cos, sin = rope_tables(int(c["max_seq_len"]), head_dim, float(c["rope_theta"]))
    positions = np.arange(ids.size)
    scale = 1.0 / math.sqrt(head_dim)
    hidden = embed(tensors["token_embedding"], ids)
    for i in range(int(c["n_layers"])):
        p = f"layers.{i}."
        normed = rms_norm(hidden, tensors[p + "attn_norm"], eps)
        q, k, v = project_qkv(normed, tensors[p + "qkv_proj"], n_heads, n_kv, head_dim)
        q = apply_rope(q, positions, cos, sin)
        k = apply_rope(k, positions, cos, sin)
        attended = causal_attention(q, k, v, scale)
        hidden = (hidden + attended.reshape(ids.size, n_heads * head_dim) @ tensors[p + "out_proj"].astype(F32)).astype(F32)
        normed = rms_norm(hidden, tensors[p + "ffn_norm"], eps)
        hidden = (hidden + swiglu(normed, tensors[p + "gate_proj"], tensors[p + "up_proj"], tensors[p + "down_proj"])).astype(F32)
    head = tensors["token_embedding"] if c["tie_embeddings"] else tensors["lm_head"]
    if rows is not None:
        hidden = hidden[np.asarray(rows, dtype=np.int64)]
    return lm_head(hidden, tensors["final_norm"], eps, head)


# --------------------------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------------------------

GREEDY_TEMPERATURE = 1e-5  # reference: src/paged_kv_serving/engine/sequence.py:42


def greedy_token(logits: np.ndarray) -> int:
    """Highest logit, lowest id on ties. Reference: src/paged_kv_serving/engine/sampling.py:28-30."""
    return int(np.argmax(logits))


def top_p_filter(probabilities: np.ndarray, top_p: float) -> np.ndarray:
    """Keep the most probable tokens up to and including the one whose cumulative mass reaches
    ``top_p``; renormalise. Reference: src/paged_kv_serving/engine/sampling.py:33-53."""
    if top_p == 1.0:
        return probabilities
    order = np.argsort(-probabilities, kind="stable")
    ordered = probabilities[order]
    cumulative = np.cumsum(ordered, dtype=np.float64)
    keep = int(np.searchsorted(cumulative, top_p, side="left")) + 1
    filtered = np.zeros_like(probabilities)
    filtered[order[:keep]] = ordered[:keep]
    total = float(filtered.sum())
    return (filtered / total).astype(F32)


def sample_distribution(logits: np.ndarray, temperature: float, top_p: float) -> np.ndarray:
    """The float32 probabilities a non-greedy draw is taken from.

    Reference: src/paged_kv_serving/engine/sampling.py:65-69 (divide by the temperature in
    float32, subtract the maximum, exponentiate in float64, normalise, cast, nucleus filter).
    """
    scaled = (logits.astype(F32) / F32(temperature)).astype(F32)
    shifted = scaled - np.max(scaled)
    e = np.exp(shifted.astype(np.float64))
    return top_p_filter((e / e.sum()).astype(F32), top_p)


def sample_token(logits: np.ndarray, temperature: float, top_p: float, uniform: float) -> int:
    """Inverse-CDF draw with one uniform number.

    Reference: src/paged_kv_serving/engine/sampling.py:56-74 (float64 cumulative sum,
    ``draw = u * cum[-1]``, first index whose cumulative mass exceeds the draw).
    """
    if temperature < GREEDY_TEMPERATURE:
        return greedy_token(logits)
    p = sample_distribution(logits, temperature, top_p)
    cumulative = np.cumsum(p, dtype=np.float64)
    draw = float(uniform) * float(cumulative[-1])
    return int(np.searchsorted(cumulative, draw, side="right").clip(0, p.size - 1))


def sequence_generator(seed: int, sample_index: int) -> np.random.Generator:
    """Per-sample generator. Reference: src/paged_kv_serving/engine/sequence.py:165-170."""
    return np.random.default_rng(np.random.SeedSequence(entropy=seed, spawn_key=(sample_index,)))


def generate(config, tensors, prompt, max_new_tokens, temperature=0.0, top_p=1.0, seed=0, sample_index=0):
    """Token-by-token generation by full recomputation (no cache); returns the new tokens."""
    rng = sequence_generator(seed, sample_index)
    tokens = list(prompt)
    produced = []
    for _ in range(max_new_tokens):
        row = forward(config, tensors, tokens)[-1]
        if temperature < GREEDY_TEMPERATURE:
            token = greedy_token(row)
        else:
            token = sample_token(row, temperature, top_p, float(rng.random()))
        tokens.append(token)
        produced.append(token)
    return produced


# --------------------------------------------------------------------------------------------
# random weights for tests (independent of the product's generator)
# --------------------------------------------------------------------------------------------


def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    """Name -> shape of every tensor of a model folder.

    Reference: src/paged_kv_serving/engine/model.py:103-121 (names and ``(in, out)`` layouts),
    widened for grouped-query heads and the optional ``lm_head``.
    """
    c = config_sizes(config)
    d, ff, v = int(c["d_model"]), int(c["d_ff"]), int(c["vocab_size"])
    h, kv, hd = int(c["n_heads"]), int(c["n_kv_heads"]), int(c["head_dim"])
    shapes: dict[str, tuple[int, ...]] = {"token_embedding": (v, d), "final_norm": (d,)}
    if not c["tie_embeddings"]:
        shapes["lm_head"] = (v, d)
    for i in range(int(c["n_layers"])):
        p = f"layers.{i}."
        shapes[p + "attn_norm"] = (d,)
        shapes[p + "qkv_proj"] = (d, (h + 2 * kv) * hd)
        shapes[p + "out_proj"] = (h * hd, d)
        shapes[p + "ffn_norm"] = (d,)
        shapes[p + "gate_proj"] = (d, ff)
        shapes[p + "up_proj"] = (d, ff)
        shapes[p + "down_proj"] = (ff, d)
    return shapes


def random_tensors(config: dict, seed: int, std: float = 0.02, norm_jitter: float = 0.0) -> dict[str, np.ndarray]:
    """Seeded float32 tensors: matrices ``N(0, std)``, norm weights ``1 + norm_jitter * N(0, 1)``."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in sorted(tensor_shapes(config).items()):
        if len(shape) == 1:
            out[name] = (1.0 + norm_jitter * rng.standard_normal(shape)).astype(F32)
        else:
            out[name] = (rng.standard_normal(shape) * std).astype(F32)
    return out


def round_to_bfloat16(x: np.ndarray) -> np.ndarray:
    """Round float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    bits = np.ascontiguousarray(x, dtype=F32).view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(F32).reshape(x.shape)
