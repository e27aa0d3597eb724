"""Writes the golden logits that anchor ``tests/plain_model.py`` to the reference's own code.

Run once, on the CPU, with the reference project's ``src`` directory given as the argument:

    python tests/golden/make_golden.py <path-to-reference>/src

It imports the reference's NumPy model (``paged_kv_serving.engine.model``), feeds it the
tensors that ``plain_model.random_tensors`` draws for two tiny configurations, and stores the
logits of the reference's cache-free forward pass next to this script:

* ``mha_tied.npy``: a configuration the reference expresses exactly (multi-head, tied head);
  the logits are ``LanguageModel.reference_forward``.
* ``gqa_untied.npy``: grouped-query heads and a separate ``lm_head``, which the reference does
  not have. The key/value column blocks are repeated ``H / KV`` times so that the reference's
  multi-head attention computes the same function, every layer runs through the reference's
  public parts (``embed``, ``project_qkv``, ``dense_causal_attention``, ``feed_forward``), and
  only the last matrix product uses the separate head.

* ``sampling.npy``: token ids that the reference's ``sample_token``
  (src/paged_kv_serving/engine/sampling.py:56-74) returns for 2,000 seeded cases (vocabularies of
  5 to 700, greedy and temperatures up to 2, nucleus masses of 0.05 to 1, ties in the logits),
  each with a generator seeded by the case's number, so that the draw can be repeated.

``tests/test_plain_model.py`` recomputes all three with the plain implementation and compares.
The files are small (tens of kilobytes) and are committed with this script.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import plain_model  # noqa: E402

MHA_TIED = {
    "vocab_size": 384, "d_model": 96, "n_layers": 3, "n_heads": 3, "n_kv_heads": 3, "head_dim": 32,
    "d_ff": 256, "max_seq_len": 256, "rope_theta": 500000.0, "norm_eps": 1e-6, "tie_embeddings": True,
}
GQA_UNTIED = {
    "vocab_size": 256, "d_model": 64, "n_layers": 2, "n_heads": 4, "n_kv_heads": 2, "head_dim": 16,
    "d_ff": 172, "max_seq_len": 128, "rope_theta": 10000.0, "norm_eps": 1e-5, "tie_embeddings": False,
}
SEEDS = {"mha_tied": (2, 3, 24), "gqa_untied": (0, 1, 17)}  # weights seed, token seed, tokens
STD = 0.08  # wide enough that attention and the gate are far from their linear regime
NORM_JITTER = 0.1


def golden_inputs(name: str):
    config = MHA_TIED if name == "mha_tied" else GQA_UNTIED
    weight_seed, token_seed, count = SEEDS[name]
    tensors = plain_model.random_tensors(config, weight_seed, std=STD, norm_jitter=NORM_JITTER)
    tokens = np.random.default_rng(token_seed).integers(0, config["vocab_size"], size=count)
    return config, tensors, tokens


SAMPLING_CASES = 2000


def sampling_case(number: int):
    """Logits, temperature, nucleus mass and the generator of one sampling case."""
    rng = np.random.default_rng(10_000 + number)
    vocab = int(rng.integers(5, 701))
    logits = (rng.standard_normal(vocab) * rng.uniform(0.5, 4.0)).astype(np.float32)
    if number % 5 == 0:                      # ties, also among the most probable tokens
        logits = np.round(logits)
    temperature = 0.0 if number % 7 == 0 else float(rng.uniform(0.05, 2.0))
    top_p = 1.0 if number % 3 == 0 else float(rng.uniform(0.05, 1.0))
    return logits, temperature, top_p, np.random.default_rng(number)


def main(reference_src: str) -> None:
    sys.path.insert(0, reference_src)
    from paged_kv_serving.engine.sampling import sample_token as reference_sample_token
    from paged_kv_serving.engine.sequence import SamplingParams

    ids = np.zeros(SAMPLING_CASES, dtype=np.int32)
    for number in range(SAMPLING_CASES):
        logits, temperature, top_p, generator = sampling_case(number)
        ids[number] = reference_sample_token(logits, SamplingParams(temperature=temperature, top_p=top_p), generator)
    np.save(HERE / "sampling.npy", ids)
    from paged_kv_serving.engine.config import ModelConfig
    from paged_kv_serving.engine.model import (
        LanguageModel, LayerWeights, TransformerWeights, dense_causal_attention, rms_norm,
    )

    def reference_model(config, tensors, qkv_of):
        ref_config = ModelConfig(
            vocab_size=config["vocab_size"], d_model=config["d_model"], n_layers=config["n_layers"],
            n_heads=config["n_heads"], d_ff=config["d_ff"], max_seq_len=config["max_seq_len"],
            rope_theta=config["rope_theta"], norm_eps=config["norm_eps"],
        )
        layers = tuple(
            LayerWeights(
                attn_norm=tensors[f"layers.{i}.attn_norm"], qkv_proj=qkv_of(i),
                out_proj=tensors[f"layers.{i}.out_proj"], ffn_norm=tensors[f"layers.{i}.ffn_norm"],
                gate_proj=tensors[f"layers.{i}.gate_proj"], up_proj=tensors[f"layers.{i}.up_proj"],
                down_proj=tensors[f"layers.{i}.down_proj"],
            )
            for i in range(config["n_layers"])
        )
        weights = TransformerWeights(tensors["token_embedding"], layers, tensors["final_norm"])
        return LanguageModel(ref_config, weights)

    # multi-head, tied: the reference's own forward pass
    config, tensors, tokens = golden_inputs("mha_tied")
    model = reference_model(config, tensors, lambda i: tensors[f"layers.{i}.qkv_proj"])
    np.save(HERE / "mha_tied.npy", model.reference_forward(tokens))

    # grouped-query, untied: expanded key/value columns through the reference's parts
    config, tensors, tokens = golden_inputs("gqa_untied")
    h, kv, hd, d = config["n_heads"], config["n_kv_heads"], config["head_dim"], config["d_model"]

    def expanded(i):
        w = tensors[f"layers.{i}.qkv_proj"]
        q = w[:, : h * hd]
        k = w[:, h * hd : (h + kv) * hd].reshape(d, kv, hd)
        v = w[:, (h + kv) * hd :].reshape(d, kv, hd)
        k = np.repeat(k, h // kv, axis=1).reshape(d, h * hd)
        v = np.repeat(v, h // kv, axis=1).reshape(d, h * hd)
        return np.ascontiguousarray(np.concatenate([q, k, v], axis=1))

    model = reference_model(config, tensors, expanded)
    positions = np.arange(tokens.size, dtype=np.int64)
    hidden = model.embed(tokens.astype(np.int64))
    for layer in model.weights.layers:
        q, k, v = model.project_qkv(hidden, layer, positions)
        attended = dense_causal_attention(q, k, v, model.attention_scale)
        hidden = hidden + attended.reshape(tokens.size, d) @ layer.out_proj
        hidden = (hidden + model.feed_forward(hidden, layer)).astype(np.float32)
    logits = rms_norm(hidden, tensors["final_norm"], config["norm_eps"]) @ tensors["lm_head"].T
    np.save(HERE / "gqa_untied.npy", logits.astype(np.float32))
    print("wrote", HERE / "mha_tied.npy", HERE / "gqa_untied.npy")


if __name__ == "__main__":
    main(sys.argv[1])
