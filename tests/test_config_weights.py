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


def test_weights_with_nan_or_infinite_values_are_refused():
    """Reference: src/paged_kv_serving/engine/model.py:103-128 refuses non-finite tensors."""
    from paged_kv_serving_b200.models.decoder import DecoderModel
    from paged_kv_serving_b200.weights import non_finite_tensors

    c = _config("A")
    specs = architecture("LlamaToyDecoder").layout(c).tensor_specs()
    tensors = random_tensors(specs, 3)
    assert non_finite_tensors(tensors) == []
    DecoderModel.from_tensors(c, tensors, "float32", "cpu")           # finite weights load
    tensors["layers.1.down_proj"][5, 7] = float("nan")
    tensors["final_norm"][0] = float("inf")
    assert non_finite_tensors(tensors) == ["final_norm", "layers.1.down_proj"]
    with pytest.raises(WeightsError) as error:
        DecoderModel.from_tensors(c, tensors, "float32", "cpu")
    assert "final_norm: holds NaN or infinite values" in str(error.value)
    assert "layers.1.down_proj: holds NaN or infinite values" in str(error.value)
    # a value that is finite in float32 and overflows the compute type is caught after the cast
    tensors = random_tensors(specs, 3)
    tensors["layers.0.up_proj"][0, 0] = 3.4e38
    DecoderModel.from_tensors(c, tensors, "float32", "cpu")
    with pytest.raises(WeightsError, match="layers.0.up_proj"):
        DecoderModel.from_tensors(c, tensors, "bfloat16", "cpu")


def test_manifest_must_agree_with_the_configuration_and_the_tensors(tmp_path):
    """Reference: src/paged_kv_serving/engine/weights.py:191-200 (parameter count and architecture
    of the manifest against the model that was read)."""
    from safetensors.torch import save_file

    from paged_kv_serving_b200.weights.manifest import sha256_file

    c = _config("B")
    write_random_model_folder(tmp_path, c, seed=1, dtype="float32")
    path = tmp_path / "manifest.json"
    good = json.loads(path.read_text())
    assert good["parameter_count"] == c.parameter_count and good["architecture"] == c.to_dict()
    read_model_folder(tmp_path)
    lying = json.loads(json.dumps(good))
    lying["parameter_count"] += 1
    path.write_text(json.dumps(lying))
    with pytest.raises(ModelIntegrityError, match="parameter count mismatch"):
        read_model_folder(tmp_path)
    lying = json.loads(json.dumps(good))
    lying["architecture"]["n_layers"] = 4
    path.write_text(json.dumps(lying))
    with pytest.raises(ModelIntegrityError, match="not the configuration"):
        read_model_folder(tmp_path)
    # defaults written out or left out describe the same configuration
    same = json.loads(json.dumps(good))
    del same["architecture"]["rope_theta"]
    same["architecture"]["rope_theta"] = c.rope_theta
    path.write_text(json.dumps(same))
    read_model_folder(tmp_path)
    # tensors that hold another number of parameters than the manifest records (digests in order)
    _, tensors = read_model_folder(tmp_path)
    tensors["stowaway"] = torch.zeros(3)
    save_file(tensors, str(tmp_path / "model.safetensors"))
    forged = json.loads(json.dumps(good))
    for artifact in forged["artifacts"]:
        artifact["sha256"] = sha256_file(tmp_path / artifact["name"])
        artifact["size_bytes"] = (tmp_path / artifact["name"]).stat().st_size
    path.write_text(json.dumps(forged))
    with pytest.raises(ModelIntegrityError, match="parameter count mismatch"):
        read_model_folder(tmp_path)


def test_build_checkpoint_takes_an_architecture_with_a_configuration_class_of_its_own(tmp_path):
    """The command line and the random-weights mode go through the architecture's own typed
    configuration: a toy architecture registered here, whose config.json has a key the shared
    class does not know, builds a model folder and reads back."""
    from dataclasses import dataclass, fields

    from paged_kv_serving_b200 import cli
    from paged_kv_serving_b200.config import load_config, registry

    if "ToyOwnConfigDecoder" not in known_architectures():
        @dataclass(frozen=True)
        class ToyConfig:
            vocab_size: int
            d_model: int
            n_layers: int
            n_heads: int
            d_ff: int
            max_seq_len: int
            ff_widening: int = 1          # a key of this architecture alone
            architecture: str = "ToyOwnConfigDecoder"

            def to_dict(self):
                return {f.name: getattr(self, f.name) for f in fields(self)}

            @classmethod
            def from_dict(cls, data):
                return cls(**data)

        @registry.register_architecture("ToyOwnConfigDecoder")
        class ToyOwnConfigDecoder:
            config_class = ToyConfig

            @staticmethod
            def layout(config):
                shared = ModelConfig(vocab_size=config.vocab_size, d_model=config.d_model, n_layers=config.n_layers,
                                     n_heads=config.n_heads, d_ff=config.d_ff * config.ff_widening,
                                     max_seq_len=config.max_seq_len)
                return architecture("LlamaToyDecoder").layout(shared)

    source = tmp_path / "toy.json"
    source.write_text(json.dumps({"architecture": "ToyOwnConfigDecoder", "vocab_size": 50, "d_model": 32, "n_layers": 1,
                                  "n_heads": 2, "d_ff": 24, "max_seq_len": 64, "ff_widening": 2}))
    out = tmp_path / "folder"
    assert cli.main(["build-checkpoint", "--out", str(out), "--config", str(source), "--seed", "3", "--dtype", "float32"]) == 0
    config, tensors = read_model_folder(out)
    assert type(config).__name__ == "ToyConfig" and config.ff_widening == 2 and load_config(out) == config
    assert tensors["layers.0.gate_proj"].shape == (32, 48)
    assert json.loads((out / "manifest.json").read_text())["parameter_count"] == sum(t.numel() for t in tensors.values())
