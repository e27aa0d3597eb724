"""Each part alone, and the framework's generality: a toy mixer with state of its own, a layer
order that names a layer twice and lets a layer read another layer's cache, a toy position
encoding; all registered from this file without touching the framework (``-m gpu``)."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import helpers
import plain_model

pytestmark = pytest.mark.gpu
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(array, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(array)).cuda()
    return t.to(dtype) if dtype is not None else t


def rounded(array, dtype):
    return torch.from_numpy(array).to(DTYPES[dtype]).float().numpy()


def test_rotary_tables_match_the_plain_ones():
    from paged_kv_serving_b200.parts import RotaryEncoding

    part = RotaryEncoding(48, 50000.0, 300)
    cos, sin = part.fused_tables(torch.device("cuda"))
    want_cos, want_sin = plain_model.rope_tables(300, 48, 50000.0)
    assert np.array_equal(cos.cpu().numpy(), want_cos) and np.array_equal(sin.cpu().numpy(), want_sin)
    with pytest.raises(ValueError):
        RotaryEncoding(7, 10000.0, 8)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part_and_swiglu_part(dtype):
    from paged_kv_serving_b200.parts import RMSNorm, StepContext, SwiGLU

    rng = np.random.default_rng(0)
    width, inner, tokens = 72, 150, 10
    norm = RMSNorm(width, 3e-6)
    weight = (1 + 0.3 * rng.standard_normal(width)).astype(np.float32)
    norm.load({"weight": dev(weight)})
    hidden = rng.standard_normal((tokens, width)).astype(np.float32)
    normed = norm.add_norm(dev(hidden), None, DTYPES[dtype])
    want = plain_model.rms_norm(hidden, weight, 3e-6)
    assert np.abs(normed.float().cpu().numpy() - want).max() <= (2e-5 if dtype == "float32" else 3e-2)

    ff = SwiGLU(width, inner, 60.0)
    gate, up, down = (rounded((rng.standard_normal(shape) * 0.2).astype(np.float32), dtype)
                      for shape in ((width, inner), (width, inner), (inner, width)))
    ff.load({"gate_proj": dev(gate, DTYPES[dtype]), "up_proj": dev(up, DTYPES[dtype]), "down_proj": dev(down, DTYPES[dtype])})
    x = rounded(rng.standard_normal((tokens, width)).astype(np.float32), dtype)
    got = ff.forward(dev(x, DTYPES[dtype]), None).float().cpu().numpy()
    want = plain_model.swiglu(x, gate, up, down)
    # bounds relative to the output's magnitude (sums of ~150 products): float32 rounding, or bfloat16's 2^-8
    scale = float(np.abs(want).max())
    assert np.abs(got - want).max() <= (2e-6 * scale + 1e-6 if dtype == "float32" else 3e-2 * scale + 1e-3)


# ---------------------------------------------------------------------------------------------
# toy parts and toy architectures, defined and registered here
# ---------------------------------------------------------------------------------------------


def _register_toys():
    from paged_kv_serving_b200.config import registry
    from paged_kv_serving_b200.models.layout import LayerCall, ModelLayout
    from paged_kv_serving_b200.ops import gemm
    from paged_kv_serving_b200.parts import (
        PagedAttention, ParamSpec, Part, PositionEncoding, PreNormBlock, RMSNorm, RotaryEncoding, StateRequest,
        StepContext, SwiGLU,
    )

    if "ToyStateDecoder" in registry.known_architectures():
        return

    @registry.register_part("mixer", "toy_running_mean")
    class RunningMean(Part):
        """out[t] = mean(x[0..t]) @ proj, resumable through a per-request state [width + 1]."""

        def __init__(self, width):
            self.width = width
            self.proj = None

        def param_specs(self):
            return {"proj": ParamSpec((self.width, self.width))}

        def cache_request(self):
            return StateRequest((self.width + 1,), "float32")

        def forward(self, x, ctx, binding):
            state = ctx.states[binding.state]
            slots = ctx.ints(ctx.STATE_SLOTS).tolist()
            out = torch.empty_like(x)
            start = 0
            for slot, count in zip(slots, ctx.seq_lens):
                rows = x[start:start + count].float()
                running = state[slot, :self.width] + torch.cumsum(rows, dim=0)
                counts = state[slot, self.width] + torch.arange(1, count + 1, device=x.device, dtype=torch.float32)
                out[start:start + count] = (running / counts[:, None]).to(x.dtype)
                state[slot, :self.width] = running[-1]
                state[slot, self.width] = counts[-1]
                start += count
            return gemm.matmul(out, self.proj)

    @registry.register_part("position", "toy_scale_by_position")
    class ScaleByPosition(PositionEncoding):
        """Not a rotation: multiplies queries and keys by 1 / (1 + position / 64)."""

        def apply_qk(self, qkv, positions, n_heads, n_kv, head_dim):
            factor = (1.0 / (1.0 + positions.float() / 64.0)).to(qkv.dtype)[:, None]
            qkv[:, :(n_heads + n_kv) * head_dim] *= factor

    @registry.register_architecture("ToyStateDecoder")
    class ToyStateDecoder:
        @staticmethod
        def layout(config):
            blocks, names = [], {}
            for i in range(config.n_layers):
                mixer = RunningMean(config.d_model) if i % 2 == 0 else PagedAttention(
                    config.d_model, config.n_heads, config.n_kv_heads, config.head_dim, ScaleByPosition(),
                    window=config.max_seq_len // 8)
                block = PreNormBlock(RMSNorm(config.d_model, config.norm_eps), mixer,
                                     RMSNorm(config.d_model, config.norm_eps), SwiGLU(config.d_model, config.d_ff))
                blocks.append(block)
                from paged_kv_serving_b200.models.layout import collect_param_specs

                collect_param_specs(f"blocks.{i}.", block, names)
            final = RMSNorm(config.d_model, config.norm_eps)
            names["final.weight"] = (final, "weight")
            return ModelLayout(width=config.d_model, vocab_size=config.vocab_size, max_positions=config.max_seq_len,
                               blocks=blocks, order=[LayerCall(i) for i in range(config.n_layers)], final_norm=final,
                               names=names, embedding_name="embed", head_name=None)

    @registry.register_part("feed_forward", "toy_routed")
    class RoutedFeedForward(Part):
        """Top-1 routing among a few small experts: router logits and their softmax in float32,
        out = p[e] * (relu(x @ w_in[e]) @ w_out[e]) for the expert e with the largest logit
        (lowest index on ties)."""

        def __init__(self, width, inner, experts):
            self.width, self.inner, self.experts = width, inner, experts
            self.router = self.w_in = self.w_out = None

        def param_specs(self):
            return {"router": ParamSpec((self.width, self.experts)),
                    "w_in": ParamSpec((self.experts * self.width, self.inner)),
                    "w_out": ParamSpec((self.experts * self.inner, self.width))}

        def forward(self, x, ctx):
            logits = gemm.matmul(x, self.router).float()
            probs = torch.softmax(logits, dim=-1)
            choice = torch.argmax(logits, dim=-1)
            out = torch.zeros_like(x)
            for e in range(self.experts):
                rows = torch.nonzero(choice == e).flatten()
                if rows.numel() == 0:
                    continue
                hidden = torch.relu(gemm.matmul(x[rows], self.w_in[e * self.width:(e + 1) * self.width]))
                expert_out = gemm.matmul(hidden, self.w_out[e * self.inner:(e + 1) * self.inner])
                out[rows] = (expert_out.float() * probs[rows, e:e + 1]).to(x.dtype)
            return out

    @registry.register_architecture("ToyRoutedDecoder")
    class ToyRoutedDecoder:
        """Llama-style attention in every layer; the feed-forward of odd layers is routed."""

        @staticmethod
        def layout(config):
            from paged_kv_serving_b200.models.layout import collect_param_specs

            blocks, names = [], {}
            for i in range(config.n_layers):
                mixer = PagedAttention(config.d_model, config.n_heads, config.n_kv_heads, config.head_dim,
                                       RotaryEncoding(config.head_dim, config.rope_theta, config.max_seq_len))
                ff = RoutedFeedForward(config.d_model, 40, 3) if i % 2 else SwiGLU(config.d_model, config.d_ff)
                block = PreNormBlock(RMSNorm(config.d_model, config.norm_eps), mixer,
                                     RMSNorm(config.d_model, config.norm_eps), ff)
                blocks.append(block)
                collect_param_specs(f"blocks.{i}.", block, names)
            final = RMSNorm(config.d_model, config.norm_eps)
            names["final.weight"] = (final, "weight")
            return ModelLayout(width=config.d_model, vocab_size=config.vocab_size, max_positions=config.max_seq_len,
                               blocks=blocks, order=[LayerCall(i) for i in range(config.n_layers)], final_norm=final,
                               names=names, embedding_name="embed", head_name=None)

    @registry.register_architecture("ToySharedCacheDecoder")
    class ToySharedCacheDecoder:
        """Two Llama-style layers; run order: layer 0, layer 1 reading layer 0's keys and values
        (writing none of its own), then layer 0 a second time with a cache of its own."""

        @staticmethod
        def layout(config):
            base = registry.architecture("LlamaToyDecoder").layout(config)
            base.order = [LayerCall(0, cache=0), LayerCall(1, cache=0, write=False), LayerCall(0, cache=1)]
            return base


TOY = {"architecture": "ToyStateDecoder", "vocab_size": 97, "d_model": 48, "n_layers": 3, "n_heads": 3, "n_kv_heads": 1,
       "head_dim": 16, "d_ff": 80, "max_seq_len": 128, "norm_eps": 1e-5}


def _toy_plain(tensors, tokens):
    """Plain whole-sequence forward of ToyStateDecoder (NumPy, no cache, no state)."""
    c = TOY
    x = tensors["embed"][np.asarray(tokens)]
    positions = np.arange(len(tokens))
    for i in range(c["n_layers"]):
        p = f"blocks.{i}."
        normed = plain_model.rms_norm(x, tensors[p + "mixer_norm.weight"], c["norm_eps"])
        if i % 2 == 0:
            mean = np.cumsum(normed, axis=0) / np.arange(1, len(tokens) + 1)[:, None]
            mixed = mean.astype(np.float32) @ tensors[p + "mixer.proj"]
        else:
            q, k, v = plain_model.project_qkv(normed, tensors[p + "mixer.qkv_proj"], 3, 1, 16)
            factor = (1.0 / (1.0 + positions / 64.0)).astype(np.float32)[:, None, None]
            attended = plain_model.causal_attention(q * factor, k * factor, v, 1 / math.sqrt(16), window=16)
            mixed = attended.reshape(len(tokens), 48) @ tensors[p + "mixer.out_proj"]
        x = (x + mixed).astype(np.float32)
        normed = plain_model.rms_norm(x, tensors[p + "ff_norm.weight"], c["norm_eps"])
        x = (x + plain_model.swiglu(normed, tensors[p + "feed_forward.gate_proj"], tensors[p + "feed_forward.up_proj"],
                                    tensors[p + "feed_forward.down_proj"])).astype(np.float32)
    return plain_model.rms_norm(x, tensors["final.weight"], c["norm_eps"]) @ tensors["embed"].T


def test_toy_mixer_with_state_and_toy_position_encoding_register_build_and_step():
    from paged_kv_serving_b200.config import ModelConfig, registry
    from paged_kv_serving_b200.engine.replay import ReplaySession
    from paged_kv_serving_b200.models.decoder import DecoderModel

    _register_toys()
    config = ModelConfig.from_dict(TOY)
    specs = registry.architecture("ToyStateDecoder").layout(config).tensor_specs()
    rng = np.random.default_rng(9)
    tensors = {name: ((1 + 0.1 * rng.standard_normal(spec.shape)) if spec.kind == "vector"
                      else rng.standard_normal(spec.shape) * 0.15).astype(np.float32) for name, spec in specs.items()}
    model = DecoderModel.from_tensors(config, {k: torch.from_numpy(v) for k, v in tensors.items()}, "float32", "cuda")
    session = ReplaySession(model, max_tokens=192, block_size=4)
    assert session.runner.num_state_slots > 0 and len(session.runner.groups) == 1
    assert session.runner.groups[0].window == 16 and not session.cache.prefix_cache.enabled
    a = [int(t) for t in rng.integers(0, 97, size=90)]
    b = [int(t) for t in rng.integers(0, 97, size=50)]
    want_a, want_b = _toy_plain(tensors, a), _toy_plain(tensors, b)
    got = session.step([{"id": "a", "tokens": a[:33], "want": [0, 32]}])
    helpers.assert_close(got, want_a[[0, 32]], "float32", "toy first portion")
    got = session.step([{"id": "a", "tokens": a[33:35], "want": [1]}, {"id": "b", "tokens": b[:20], "want": [19]}])
    helpers.assert_close(got, np.stack([want_a[34], want_b[19]]), "float32", "toy mixed")
    for i in range(35, 90):
        entries = [{"id": "a", "tokens": [a[i]], "want": [0]}]
        if 20 + (i - 35) < 50:
            entries.append({"id": "b", "tokens": [b[20 + i - 35]], "want": [0]})
        got = session.step(entries)
        helpers.assert_close(got[:1], want_a[i:i + 1], "float32", f"toy decode a {i}")
        if len(entries) == 2:
            helpers.assert_close(got[1:], want_b[20 + i - 35:21 + i - 35], "float32", f"toy decode b {i}")
    held = [page for page in session.live["a"].block_table if page >= 0]
    assert len(held) <= 16 // 4 + 2, "pages behind the window must have been given back"
    session.step([], end=["a", "b"])
    session.check_invariants()
    assert session.cache.num_free_blocks == session.num_blocks and session.cache.state_slots.num_free == 64
    # a slot that is taken again starts from a cleared state
    got = session.step([{"id": "c", "tokens": b[:20], "want": [19]}])
    helpers.assert_close(got, want_b[19:20], "float32", "toy reused slot")


def test_toy_routed_feed_forward_registers_builds_and_steps():
    """A feed-forward with routing, defined in this file, beside the dense one in other layers:
    whole prompt, portions and decoding agree with a plain forward. The router's weights are
    scaled so that the chosen expert is never a near tie that float32 rounding could flip."""
    from paged_kv_serving_b200.config import ModelConfig, registry
    from paged_kv_serving_b200.engine.replay import ReplaySession
    from paged_kv_serving_b200.models.decoder import DecoderModel

    _register_toys()
    c = dict(TOY, architecture="ToyRoutedDecoder", n_layers=4, n_kv_heads=3)
    config = ModelConfig.from_dict(c)
    specs = registry.architecture("ToyRoutedDecoder").layout(config).tensor_specs()
    rng = np.random.default_rng(21)
    tensors = {name: ((1 + 0.1 * rng.standard_normal(spec.shape)) if spec.kind == "vector"
                      else rng.standard_normal(spec.shape) * (2.0 if name.endswith("router") else 0.15)).astype(np.float32)
               for name, spec in specs.items()}

    def plain(tokens):
        cos, sin = plain_model.rope_tables(c["max_seq_len"], 16, 10000.0)
        pos = np.arange(len(tokens))
        x = tensors["embed"][np.asarray(tokens)]
        margins = []
        for i in range(c["n_layers"]):
            p = f"blocks.{i}."
            normed = plain_model.rms_norm(x, tensors[p + "mixer_norm.weight"], c["norm_eps"])
            q, k, v = plain_model.project_qkv(normed, tensors[p + "mixer.qkv_proj"], 3, 3, 16)
            q, k = plain_model.apply_rope(q, pos, cos, sin), plain_model.apply_rope(k, pos, cos, sin)
            attended = plain_model.causal_attention(q, k, v, 1 / math.sqrt(16))
            x = (x + attended.reshape(len(tokens), 48) @ tensors[p + "mixer.out_proj"]).astype(np.float32)
            normed = plain_model.rms_norm(x, tensors[p + "ff_norm.weight"], c["norm_eps"])
            if i % 2:
                logits = (normed @ tensors[p + "feed_forward.router"]).astype(np.float32)
                top = np.sort(logits, axis=-1)
                margins.append(top[:, -1] - top[:, -2])
                probs = np.exp(logits - logits.max(-1, keepdims=True))
                probs /= probs.sum(-1, keepdims=True)
                choice = logits.argmax(-1)
                out = np.zeros_like(normed)
                for t, e in enumerate(choice):
                    hidden = np.maximum(normed[t] @ tensors[p + "feed_forward.w_in"][e * 48:(e + 1) * 48], 0)
                    out[t] = probs[t, e] * (hidden @ tensors[p + "feed_forward.w_out"][e * 40:(e + 1) * 40])
                x = (x + out).astype(np.float32)
            else:
                x = (x + plain_model.swiglu(normed, tensors[p + "feed_forward.gate_proj"],
                                            tensors[p + "feed_forward.up_proj"],
                                            tensors[p + "feed_forward.down_proj"])).astype(np.float32)
        return plain_model.rms_norm(x, tensors["final.weight"], c["norm_eps"]) @ tensors["embed"].T, np.concatenate(margins)

    tokens = [int(t) for t in rng.integers(0, 97, size=60)]
    want, margins = plain(tokens)
    assert margins.min() > 1e-3, "the test's weights must not put a token on a routing tie"
    model = DecoderModel.from_tensors(config, {k: torch.from_numpy(v) for k, v in tensors.items()}, "float32", "cuda")
    session = ReplaySession(model, max_tokens=128, block_size=8)
    got = [session.step([{"id": "s", "tokens": tokens[:21], "want": list(range(21))}])]
    got.append(session.step([{"id": "s", "tokens": tokens[21:23], "want": [0, 1]}]))
    got.append(session.step([{"id": "s", "tokens": tokens[23:40], "want": list(range(17))}]))
    got += [session.step([{"id": "s", "tokens": [t], "want": [0]}]) for t in tokens[40:]]
    helpers.assert_close(np.concatenate(got), want, "float32", "routed feed-forward")


def test_parts_that_know_nothing_of_fused_norms_get_plain_tensors_in_bfloat16():
    """In bfloat16, the products of a decode step carry the residual add and leave the norm to the
    product that reads it. A mixer defined here, which knows nothing of that, must still receive
    an ordinary normalised tensor: the toy architecture at a width the fused kernels take, decoded
    token by token, against its plain forward on the bfloat16-rounded weights."""
    from paged_kv_serving_b200.config import ModelConfig, registry
    from paged_kv_serving_b200.engine.replay import ReplaySession
    from paged_kv_serving_b200.models.decoder import DecoderModel
    from paged_kv_serving_b200.ops import gemm

    _register_toys()
    c = dict(TOY, d_model=64, n_heads=4, n_kv_heads=2, d_ff=128, n_layers=4)
    config = ModelConfig.from_dict(c)
    specs = registry.architecture("ToyStateDecoder").layout(config).tensor_specs()
    rng = np.random.default_rng(33)
    tensors = {name: ((1 + 0.1 * rng.standard_normal(spec.shape)) if spec.kind == "vector"
                      else plain_model.round_to_bfloat16(rng.standard_normal(spec.shape) * 0.12)).astype(np.float32)
               for name, spec in specs.items()}

    def plain(tokens):
        x = tensors["embed"][np.asarray(tokens)]
        positions = np.arange(len(tokens))
        for i in range(c["n_layers"]):
            p = f"blocks.{i}."
            normed = plain_model.rms_norm(x, tensors[p + "mixer_norm.weight"], c["norm_eps"])
            if i % 2 == 0:
                mean = np.cumsum(normed, axis=0) / np.arange(1, len(tokens) + 1)[:, None]
                mixed = mean.astype(np.float32) @ tensors[p + "mixer.proj"]
            else:
                q, k, v = plain_model.project_qkv(normed, tensors[p + "mixer.qkv_proj"], 4, 2, 16)
                factor = (1.0 / (1.0 + positions / 64.0)).astype(np.float32)[:, None, None]
                attended = plain_model.causal_attention(q * factor, k * factor, v, 1 / math.sqrt(16), window=16)
                mixed = attended.reshape(len(tokens), 64) @ tensors[p + "mixer.out_proj"]
            x = (x + mixed).astype(np.float32)
            normed = plain_model.rms_norm(x, tensors[p + "ff_norm.weight"], c["norm_eps"])
            x = (x + plain_model.swiglu(normed, tensors[p + "feed_forward.gate_proj"], tensors[p + "feed_forward.up_proj"],
                                        tensors[p + "feed_forward.down_proj"])).astype(np.float32)
        return plain_model.rms_norm(x, tensors["final.weight"], c["norm_eps"]) @ tensors["embed"].T

    tokens = [int(t) for t in rng.integers(0, 97, size=40)]
    want = plain(tokens)
    model = DecoderModel.from_tensors(config, {k: torch.from_numpy(v) for k, v in tensors.items()}, "bfloat16", "cuda")
    handed_on = []
    original = gemm.PendingNorm.tensor
    gemm.PendingNorm.tensor = lambda self: handed_on.append(1) or original(self)
    try:
        session = ReplaySession(model, max_tokens=64, block_size=4)
        got = [session.step([{"id": "s", "tokens": tokens[:19], "want": [18]}])]
        got += [session.step([{"id": "s", "tokens": [t], "want": [0]}]) for t in tokens[19:]]
    finally:
        gemm.PendingNorm.tensor = original
    assert handed_on, "the decode steps of this model must have gone through the fused feed-forward"
    helpers.assert_close(np.concatenate(got), want[18:], "bfloat16", "toy mixer behind a fused feed-forward")


def test_layer_order_may_repeat_a_layer_and_read_another_layers_cache():
    from paged_kv_serving_b200.engine.replay import ReplaySession

    _register_toys()
    config = dict(helpers.TINY_A, architecture="ToySharedCacheDecoder")
    tensors = helpers.tensors_for("A", "float32")
    model = helpers.build_model(config, tensors, "float32")
    assert [(c.layer, c.cache, c.write) for c in model.layout.resolved_order()] == [(0, 0, True), (1, 0, False), (0, 1, True)]
    tokens = helpers.random_tokens(config, 40, seed=3)

    def plain(tokens):
        c = plain_model.config_sizes(helpers.TINY_A)
        h, kv, hd, eps = c["n_heads"], c["n_kv_heads"], c["head_dim"], c["norm_eps"]
        cos, sin = plain_model.rope_tables(c["max_seq_len"], hd, c["rope_theta"])
        pos = np.arange(len(tokens))
        x = plain_model.embed(tensors["token_embedding"], np.asarray(tokens))
        kept = None
        for layer, reads_kept in ((0, False), (1, True), (0, False)):
            p = f"layers.{layer}."
            normed = plain_model.rms_norm(x, tensors[p + "attn_norm"], eps)
            q, k, v = plain_model.project_qkv(normed, tensors[p + "qkv_proj"], h, kv, hd)
            q, k = plain_model.apply_rope(q, pos, cos, sin), plain_model.apply_rope(k, pos, cos, sin)
            if reads_kept:
                k, v = kept
            elif kept is None:
                kept = (k, v)
            att = plain_model.causal_attention(q, k, v, 1 / math.sqrt(hd))
            x = (x + att.reshape(len(tokens), h * hd) @ tensors[p + "out_proj"]).astype(np.float32)
            normed = plain_model.rms_norm(x, tensors[p + "ffn_norm"], eps)
            x = (x + plain_model.swiglu(normed, tensors[p + "gate_proj"], tensors[p + "up_proj"], tensors[p + "down_proj"])).astype(np.float32)
        return plain_model.lm_head(x, tensors["final_norm"], eps, tensors["lm_head"])

    want = plain(tokens)
    session = ReplaySession(model, max_tokens=64, block_size=4)
    got = [session.step([{"id": "s", "tokens": tokens[:23], "want": [22]}])]
    got += [session.step([{"id": "s", "tokens": [t], "want": [0]}]) for t in tokens[23:]]
    helpers.assert_close(np.concatenate(got), want[22:], "float32", "shared cache order")


def test_an_architecture_brings_its_own_embedding_and_head():
    """An embedding scaled by sqrt(width) and a head with a soft cap on its logits, both defined in
    this file, in an architecture registered from this file: the step function asks the layout for
    its two ends and knows nothing of what they do."""
    from paged_kv_serving_b200.config import ModelConfig, registry
    from paged_kv_serving_b200.engine.replay import ReplaySession
    from paged_kv_serving_b200.models.decoder import DecoderModel
    from paged_kv_serving_b200.parts import LinearHead, TokenEmbedding

    cap = 3.0

    class ScaledEmbedding(TokenEmbedding):
        def forward(self, ctx):
            return super().forward(ctx) * math.sqrt(self.width)

    class CappedHead(LinearHead):
        def forward(self, normed, ctx):
            return cap * torch.tanh(super().forward(normed, ctx) / cap)

    if "ToyCappedDecoder" not in registry.known_architectures():
        @registry.register_architecture("ToyCappedDecoder")
        class ToyCappedDecoder:
            @staticmethod
            def layout(config):
                base = registry.architecture("LlamaToyDecoder").layout(config)
                names = {name: target for name, target in base.names.items()
                         if target[0] is not base.embedding and target[0] is not base.head}
                embedding = ScaledEmbedding(config.vocab_size, config.d_model)
                head = CappedHead(config.vocab_size, config.d_model)           # a head of its own, not tied
                names["tokens.table"] = (embedding, "table")
                names["capped_head.weight"] = (head, "weight")
                from paged_kv_serving_b200.models.layout import ModelLayout

                return ModelLayout(width=base.width, vocab_size=base.vocab_size, max_positions=base.max_positions,
                                   blocks=base.blocks, order=base.order, final_norm=base.final_norm, names=names,
                                   embedding=embedding, head=head)

    config = dict(helpers.TINY_B, architecture="ToyCappedDecoder")
    tensors = helpers.tensors_for("B", "float32")
    rng = np.random.default_rng(4)
    head_weight = (rng.standard_normal(tensors["token_embedding"].shape) * 0.3).astype(np.float32)
    mine = {("tokens.table" if k == "token_embedding" else k): v for k, v in tensors.items()}
    mine["capped_head.weight"] = head_weight
    model = DecoderModel.from_tensors(ModelConfig.from_dict(config), {k: torch.from_numpy(v) for k, v in mine.items()},
                                      "float32", "cuda")
    tokens = helpers.random_tokens(config, 50, seed=9)

    # the plain forward with the scaled embedding and the capped, untied head
    plain_tensors = dict(tensors, token_embedding=tensors["token_embedding"] * np.float32(math.sqrt(config["d_model"])),
                         lm_head=head_weight)
    raw = plain_model.forward(dict(helpers.TINY_B, tie_embeddings=False), plain_tensors, tokens)
    want = cap * np.tanh(raw / cap)
    assert np.abs(raw).max() > cap, "the cap must bite for the test to mean anything"

    session = ReplaySession(model, max_tokens=64, block_size=8)
    got = [session.step([{"id": "s", "tokens": tokens[:31], "want": [0, 30]}])]
    got += [session.step([{"id": "s", "tokens": [t], "want": [0]}]) for t in tokens[31:]]
    helpers.assert_close(np.concatenate(got), want[[0] + list(range(30, 50))], "float32", "own embedding and head")
