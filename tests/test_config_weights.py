"""Configuration, registry, model folders and their errors (no GPU)."""

import json

import numpy as np
import pytest
import torch

import helpers
from paged_kv_serving_b200.config import EngineConfig, ModelConfig, architecture, known_architectures
from paged_kv_serving_b200.weights import (
    ModelIntegrityError, WeightsError, check_tensors, manifest_digest, read_model_folder,
)
from paged_kv_serving_b200.weights.random_init import random_tensors, write_model_folder, write_random_model_folder


def _config(name="A"):
    return ModelConfig.from_dict(helpers.CONFIGS[name])


def test_config_defaults_and_derived_sizes():
    c = ModelConfig(vocab_size=64, d_model=32, n_layers=2, n_heads=2, d_ff=64, max_seq_len=192)
    assert (c.n_kv_heads, c.head_dim, c.tie_embeddings, c.rope_theta, c.norm_eps) == (2, 16, True, 10000.0, 1e-5)
    # the reference's parameter count for a tied multi-head model (engine/config.py:68-75)
    assert c.parameter_count == 64 * 32 + 2 * (32 * 96 + 32 * 32 + 3 * 32 * 64 + 64) + 32
    assert _config("A").parameter_count == 123_712


@pytest.mark.parametrize("change, message", [
    ({"n_layers": 0}, "n_layers"), ({"d_model": 30, "head_dim": None, "n_heads": 4}, "divisible"),
    ({"rope_theta": 1.0}, "rope_theta"), ({"norm_eps": 0.0}, "norm_eps"), ({"n_kv_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"), ({"vocab_size": 2.5}, "vocab_size"),
])
def test_config_validation(change, message):
    data = dict(helpers.TINY_A)
    data.update(change)
    data = {k: v for k, v in data.items() if v is not None}
    with pytest.raises(ValueError, match=message):
        ModelConfig.from_dict(data)


def test_config_rejects_unknown_and_missing_fields():
    with pytest.raises(ValueError, match="unknown model config fields: flash"):
        ModelConfig.from_dict({**helpers.TINY_A, "flash": 1})
    data = dict(helpers.TINY_A)
    del data["d_ff"]
    with pytest.raises(ValueError, match="missing model config fields: d_ff"):
        ModelConfig.from_dict(data)


def test_config_round_trips_through_json(tmp_path):
    c = _config("B")
    c.write_json(tmp_path)
    assert ModelConfig.from_json_file(tmp_path) == c
    assert json.loads((tmp_path / "config.json").read_text())["architecture"] == "LlamaToyDecoder"


def test_registry_names_the_architecture_and_lists_known_ones():
    assert "LlamaToyDecoder" in known_architectures()
    layout = architecture("LlamaToyDecoder").layout(_config("A"))
    assert len(layout.blocks) == 2 and layout.head_name == "lm_head"
    with pytest.raises(ValueError, match="unknown architecture 'Nope'.*LlamaToyDecoder"):
        architecture("Nope")


def test_engine_config_validation():
    EngineConfig()
    with pytest.raises(ValueError, match="cannot hold"):
        EngineConfig(num_blocks=4, block_size=16)
    with pytest.raises(ValueError, match="max_context_tokens"):
        EngineConfig(max_context_tokens=100)
    with pytest.raises(ValueError, match="watermark"):
        EngineConfig(watermark=1.0)
    with pytest.raises(ValueError, match="dtype"):
        EngineConfig(dtype="float16")


def test_layout_tensor_names_match_the_plain_implementation():
    import plain_model

    for name in ("A", "B", "C"):
        layout = architecture("LlamaToyDecoder").layout(_config(name))
        specs = {k: tuple(v.shape) for k, v in layout.tensor_specs().items()}
        assert specs == plain_model.tensor_shapes(helpers.CONFIGS[name])


def test_random_folder_is_deterministic_and_loads(tmp_path):
    c = _config("A")
    first = write_random_model_folder(tmp_path / "a", c, seed=3, dtype="bfloat16")
    second = write_random_model_folder(tmp_path / "b", c, seed=3, dtype="bfloat16")
    assert first["artifacts"] == second["artifacts"]
    other = write_random_model_folder(tmp_path / "c", c, seed=4, dtype="bfloat16")
    assert other["artifacts"][1]["sha256"] != first["artifacts"][1]["sha256"]
    config, tensors = read_model_folder(tmp_path / "a")
    assert config == c
    assert tensors["layers.0.qkv_proj"].dtype == torch.bfloat16 and tensors["final_norm"].dtype == torch.float32
    assert sum(t.numel() for t in tensors.values()) == c.parameter_count
    assert float(tensors["layers.1.down_proj"].float().std()) == pytest.approx(0.02, rel=0.1)


def test_weight_errors_are_reported_together():
    layout = architecture("LlamaToyDecoder").layout(_config("A"))
    specs = layout.tensor_specs()
    tensors = random_tensors(specs, 0)
    del tensors["layers.1.up_proj"]
    del tensors["lm_head"]
    tensors["layers.0.rotary_inv_freq"] = torch.zeros(8)
    tensors["layers.0.qkv_proj"] = torch.zeros(64, 192)
    tensors["final_norm"] = torch.zeros(64, dtype=torch.int64)
    with pytest.raises(WeightsError) as error:
        check_tensors(specs, tensors)
    text = str(error.value)
    assert "missing tensors (2): layers.1.up_proj, lm_head" in text
    assert "unexpected tensors (1): layers.0.rotary_inv_freq" in text
    assert "layers.0.qkv_proj: expected shape (64, 128), found (64, 192)" in text
    assert "final_norm: expected a floating-point tensor" in text
    assert error.value.missing == ["layers.1.up_proj", "lm_head"]


def test_manifest_catches_tampering(tmp_path):
    c = _config("B")
    manifest = write_random_model_folder(tmp_path, c, seed=1, dtype="float32")
    read_model_folder(tmp_path, expect_manifest_sha256=manifest_digest(manifest))
    with pytest.raises(ModelIntegrityError, match="pinned"):
        read_model_folder(tmp_path, expect_manifest_sha256="0" * 64)
    weights = tmp_path / "model.safetensors"
    data = bytearray(weights.read_bytes())
    data[-1] ^= 0xFF
    weights.write_bytes(bytes(data))
    with pytest.raises(ModelIntegrityError, match="does not match its manifest digest"):
        read_model_folder(tmp_path)
    weights.write_bytes(bytes(data) + b"x")
    with pytest.raises(ModelIntegrityError, match="unexpected size"):
        read_model_folder(tmp_path)
    weights.unlink()
    with pytest.raises(ModelIntegrityError, match="missing model file"):
        read_model_folder(tmp_path)


def test_manifest_rules(tmp_path):
    c = _config("A")
    write_random_model_folder(tmp_path, c, seed=1, dtype="float32")
    path = tmp_path / "manifest.json"
    good = json.loads(path.read_text())
    for edit, message in [
        (lambda m: m["artifacts"].pop(), "does not cover"),
        (lambda m: m["artifacts"].append(dict(m["artifacts"][0])), "more than once"),
        (lambda m: m["artifacts"][0].update(name="../config.json"), "plain file name"),
        (lambda m: m.update(extra=1), "exactly the keys"),
    ]:
        bad = json.loads(json.dumps(good))
        edit(bad)
        path.write_text(json.dumps(bad))
        with pytest.raises(ModelIntegrityError, match=message):
            read_model_folder(tmp_path)
    path.unlink()
    read_model_folder(tmp_path)          # a folder without a manifest loads unchecked
    with pytest.raises(ModelIntegrityError, match="no manifest.json"):
        read_model_folder(tmp_path, expect_manifest_sha256="0" * 64)


def test_folder_written_from_given_tensors_round_trips(tmp_path):
    c = _config("B")
    tensors = {k: torch.from_numpy(v) for k, v in helpers.tensors_for("B", "float32").items()}
    write_model_folder(tmp_path, c, tensors)
    _, back = read_model_folder(tmp_path)
    assert set(back) == set(tensors)
    assert all(torch.equal(back[k], tensors[k]) for k in tensors)
    assert np.isfinite(back["token_embedding"].numpy()).all()
