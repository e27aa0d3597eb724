"""One model whose layers differ in what their attention needs (``-m gpu``).

A toy architecture, registered from this file, alternates attention over every key with attention
over a window of keys, at the sizes the Blackwell kernels take (head size 64, pages of 16 keys).
Each kind of layer gets a page group of its own, and each must get a plan of its own for the
step's attention kernels: the windowed layers run over fewer 64-key tiles than the others. The
query and key columns of the projections are scaled up so that the softmax of most rows is
carried by a single key, often a far one: a layer that ran with the other layer's tile count
would lose or gain such a key and miss the plain result by far more than rounding.
"""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import helpers
import plain_model

pytestmark = pytest.mark.gpu

WINDOW = 80
MIXED = {"architecture": "ToyMixedWindowDecoder", "vocab_size": 211, "d_model": 256, "n_layers": 4, "n_heads": 8,
         "n_kv_heads": 2, "head_dim": 64, "d_ff": 384, "max_seq_len": 512, "rope_theta": 10000.0, "norm_eps": 1e-5,
         "tie_embeddings": True}


def _register():
    from paged_kv_serving_b200.config import registry
    from paged_kv_serving_b200.models.layout import LayerCall, ModelLayout, collect_param_specs
    from paged_kv_serving_b200.parts import PagedAttention, PreNormBlock, RMSNorm, RotaryEncoding, SwiGLU

    if "ToyMixedWindowDecoder" in registry.known_architectures():
        return

    @registry.register_architecture("ToyMixedWindowDecoder")
    class ToyMixedWindowDecoder:
        """Even layers attend to the last ``WINDOW`` positions, odd layers to every key (the windowed
        kind comes first, so a plan wrongly shared would be the one with fewer keys)."""

        @staticmethod
        def layout(config):
            blocks, names = [], {}
            for i in range(config.n_layers):
                mixer = PagedAttention(config.d_model, config.n_heads, config.n_kv_heads, config.head_dim,
                                       RotaryEncoding(config.head_dim, config.rope_theta, config.max_seq_len),
                                       window=None if i % 2 else WINDOW)
                block = PreNormBlock(RMSNorm(config.d_model, config.norm_eps), mixer,
                                     RMSNorm(config.d_model, config.norm_eps), SwiGLU(config.d_model, config.d_ff))
                blocks.append(block)
                collect_param_specs(f"blocks.{i}.", block, names)
            final = RMSNorm(config.d_model, config.norm_eps)
            names["final.weight"] = (final, "weight")
            return ModelLayout(width=config.d_model, vocab_size=config.vocab_size, max_positions=config.max_seq_len,
                               blocks=blocks, order=[LayerCall(i) for i in range(config.n_layers)], final_norm=final,
                               names=names, embedding_name="embed", head_name=None)


def _tensors(dtype: str) -> dict[str, np.ndarray]:
    from paged_kv_serving_b200.config import ModelConfig, registry

    specs = registry.architecture("ToyMixedWindowDecoder").layout(ModelConfig.from_dict(MIXED)).tensor_specs()
    rng = np.random.default_rng(77)
    tensors = {}
    for name, spec in specs.items():
        if spec.kind == "vector":
            tensors[name] = (1 + 0.1 * rng.standard_normal(spec.shape)).astype(np.float32)
            continue
        values = rng.standard_normal(spec.shape) * 0.05
        if name.endswith("qkv_proj"):
            values[:, :(MIXED["n_heads"] + MIXED["n_kv_heads"]) * MIXED["head_dim"]] *= 1.5   # peaked softmax rows
        if name == "embed":
            values *= 2.0
        values = values.astype(np.float32)
        tensors[name] = plain_model.round_to_bfloat16(values) if dtype == "bfloat16" else values
    return tensors


def _plain(tensors, tokens):
    """Whole-sequence forward of the toy architecture from the plain parts."""
    c = MIXED
    h, kv, hd, eps = c["n_heads"], c["n_kv_heads"], c["head_dim"], c["norm_eps"]
    cos, sin = plain_model.rope_tables(c["max_seq_len"], hd, c["rope_theta"])
    pos = np.arange(len(tokens))
    x = tensors["embed"][np.asarray(tokens)]
    for i in range(c["n_layers"]):
        p = f"blocks.{i}."
        normed = plain_model.rms_norm(x, tensors[p + "mixer_norm.weight"], eps)
        q, k, v = plain_model.project_qkv(normed, tensors[p + "mixer.qkv_proj"], h, kv, hd)
        q, k = plain_model.apply_rope(q, pos, cos, sin), plain_model.apply_rope(k, pos, cos, sin)
        attended = plain_model.causal_attention(q, k, v, 1 / math.sqrt(hd), window=None if i % 2 else WINDOW)
        x = (x + attended.reshape(len(tokens), h * hd) @ tensors[p + "mixer.out_proj"]).astype(np.float32)
        normed = plain_model.rms_norm(x, tensors[p + "ff_norm.weight"], eps)
        x = (x + plain_model.swiglu(normed, tensors[p + "feed_forward.gate_proj"], tensors[p + "feed_forward.up_proj"],
                                    tensors[p + "feed_forward.down_proj"])).astype(np.float32)
    return plain_model.rms_norm(x, tensors["final.weight"], eps) @ tensors["embed"].T


def _wrong_window_gap(tensors, tokens) -> float:
    """How far the logits move when every layer is given the other kind's window: the size of the
    fault this file looks for, to be compared with the tolerance."""
    c = MIXED
    h, kv, hd, eps = c["n_heads"], c["n_kv_heads"], c["head_dim"], c["norm_eps"]
    cos, sin = plain_model.rope_tables(c["max_seq_len"], hd, c["rope_theta"])
    pos = np.arange(len(tokens))
    x = tensors["embed"][np.asarray(tokens)]
    for i in range(c["n_layers"]):
        p = f"blocks.{i}."
        normed = plain_model.rms_norm(x, tensors[p + "mixer_norm.weight"], eps)
        q, k, v = plain_model.project_qkv(normed, tensors[p + "mixer.qkv_proj"], h, kv, hd)
        q, k = plain_model.apply_rope(q, pos, cos, sin), plain_model.apply_rope(k, pos, cos, sin)
        attended = plain_model.causal_attention(q, k, v, 1 / math.sqrt(hd), window=WINDOW)   # windowed everywhere
        x = (x + attended.reshape(len(tokens), h * hd) @ tensors[p + "mixer.out_proj"]).astype(np.float32)
        normed = plain_model.rms_norm(x, tensors[p + "ff_norm.weight"], eps)
        x = (x + plain_model.swiglu(normed, tensors[p + "feed_forward.gate_proj"], tensors[p + "feed_forward.up_proj"],
                                    tensors[p + "feed_forward.down_proj"])).astype(np.float32)
    wrong = plain_model.rms_norm(x, tensors["final.weight"], eps) @ tensors["embed"].T
    return float(np.abs(wrong - _plain(tensors, tokens))[WINDOW + 20:].max())


@pytest.mark.parametrize("flat", ["never", "always"])
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_global_and_windowed_layers_in_one_model(dtype, graphs, flat):
    from paged_kv_serving_b200.config import ModelConfig
    from paged_kv_serving_b200.engine.replay import ReplaySession
    from paged_kv_serving_b200.models.decoder import DecoderModel
    from paged_kv_serving_b200.parts import PagedAttention

    if dtype == "float32" and (flat == "always" or not graphs):
        pytest.skip("the float32 path has one attention kernel and no plan to share")
    _register()
    tensors = _tensors(dtype)
    rng = np.random.default_rng(5)
    a = [int(t) for t in rng.integers(0, MIXED["vocab_size"], size=330)]
    b = [int(t) for t in rng.integers(0, MIXED["vocab_size"], size=150)]
    want_a, want_b = _plain(tensors, a), _plain(tensors, b)
    if dtype == "bfloat16":
        assert _wrong_window_gap(tensors, a) > 4 * helpers.bf16_atol(want_a), \
            "the test's weights must make keys beyond the window matter"
    model = DecoderModel.from_tensors(ModelConfig.from_dict(MIXED), {k: torch.from_numpy(v) for k, v in tensors.items()},
                                      dtype, "cuda")
    before = PagedAttention.FLAT_DECODE
    PagedAttention.FLAT_DECODE = flat
    try:
        session = ReplaySession(model, max_tokens=640, block_size=16)
        session.runner.use_graphs = graphs
        assert sorted(g.window or 0 for g in session.runner.groups) == [0, WINDOW]
        # a long first portion, a short one that ends inside a page, then mixed steps and decoding
        got = session.step([{"id": "a", "tokens": a[:200], "want": [0, 100, 199]}])
        helpers.assert_close(got, want_a[[0, 100, 199]], dtype, "first portion")
        got = session.step([{"id": "a", "tokens": a[200:290], "want": [0, 89]}, {"id": "b", "tokens": b[:131], "want": [130]}])
        helpers.assert_close(got, np.stack([want_a[200], want_a[289], want_b[130]]), dtype, "portions of two requests")
        got = session.step([{"id": "a", "tokens": a[290:292], "want": [1]}, {"id": "b", "tokens": [b[131]], "want": [0]}])
        helpers.assert_close(got, np.stack([want_a[291], want_b[131]]), dtype, "two tokens beside a decoded one")
        for i in range(292, 330):
            entries = [{"id": "a", "tokens": [a[i]], "want": [0]}]
            j = 132 + i - 292
            if j < len(b):
                entries.append({"id": "b", "tokens": [b[j]], "want": [0]})
            got = session.step(entries)
            helpers.assert_close(got[:1], want_a[i:i + 1], dtype, f"decode a at {i}")
            if len(entries) == 2:
                helpers.assert_close(got[1:], want_b[j:j + 1], dtype, f"decode b at {j}")
        windowed = [g for g, spec in enumerate(session.runner.groups) if spec.window][0]
        held = [page for page in session.live["a"].block_tables[windowed] if page >= 0]
        assert len(held) <= WINDOW // 16 + 2, "pages behind the window are given back"
        session.step([], end=["a", "b"])
        session.check_invariants()
    finally:
        PagedAttention.FLAT_DECODE = before
