"""Reading a model folder: ``config.json`` + ``model.safetensors`` (+ ``manifest.json``).

Tensors are found by name (the reference's names, src/paged_kv_serving/engine/model.py:130-170,
plus ``lm_head`` for an untied head). All problems of a folder are reported in one error that
lists missing tensors, unexpected tensors and wrong shapes together. Placement on the device
follows each tensor's kind: operands of matrix products go to the engine's compute type
(bfloat16 stays bfloat16; nothing is widened to float32 in a bfloat16 engine), element-wise
vectors are held in float32 (a tensor stored in 32-bit stays so), integer tables in int32.
"""

from __future__ import annotations

from pathlib import Path

import torch

from paged_kv_serving_b200.config.model_config import CONFIG_FILE, ModelConfig
from paged_kv_serving_b200.parts.base import ParamSpec
from paged_kv_serving_b200.weights import manifest as manifest_module

__all__ = ["WEIGHTS_FILE", "WeightsError", "check_finite", "check_tensors", "cross_check_manifest", "non_finite_tensors",
           "place", "read_model_folder", "read_safetensors"]

WEIGHTS_FILE = "model.safetensors"
_FLOAT_TYPES = (torch.float32, torch.bfloat16, torch.float16, torch.float64)


class WeightsError(ValueError):
    """The tensors of a model folder do not match what the model expects."""

    def __init__(self, missing: list[str], unexpected: list[str], wrong: list[str]) -> None:
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = ["the model's tensors do not match its configuration:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or type ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


def check_tensors(expected: dict[str, ParamSpec], found: dict[str, torch.Tensor]) -> None:
    """Raise one ``WeightsError`` naming every missing, unexpected and ill-shaped tensor."""
    missing = sorted(set(expected) - set(found))
    unexpected = sorted(set(found) - set(expected))
    wrong = []
    for name in sorted(set(expected) & set(found)):
        spec, tensor = expected[name], found[name]
        if tuple(tensor.shape) != tuple(spec.shape):
            wrong.append(f"{name}: expected shape {tuple(spec.shape)}, found {tuple(tensor.shape)}")
        elif spec.kind == "int_table" and tensor.dtype.is_floating_point:
            wrong.append(f"{name}: expected an integer table, found {tensor.dtype}")
        elif spec.kind != "int_table" and tensor.dtype not in _FLOAT_TYPES:
            wrong.append(f"{name}: expected a floating-point tensor, found {tensor.dtype}")
    if missing or unexpected or wrong:
        raise WeightsError(missing, unexpected, wrong)


def place(tensor: torch.Tensor, spec: ParamSpec, compute_dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    """Move one tensor to the device in the type its kind asks for."""
    if spec.kind == "int_table":
        target = torch.int32
    elif spec.kind == "vector":
        target = torch.float32
    else:
        target = compute_dtype
    return tensor.to(device=device, dtype=target).contiguous()


def read_safetensors(path: Path) -> dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    return load_file(str(path), device="cpu")


def read_model_folder(folder: str | Path, expect_manifest_sha256: str | None = None):
    """``(ModelConfig, name -> tensor)`` of a folder. When the folder has a manifest (or a pinned
    digest is given) every listed file is verified before anything is parsed."""
    folder = Path(folder)
    if not folder.is_dir():
        raise FileNotFoundError(f"model folder {folder} does not exist")
    manifest = None
    if (folder / manifest_module.MANIFEST_FILE).is_file() or expect_manifest_sha256 is not None:
        manifest = manifest_module.verify_manifest(folder, (CONFIG_FILE, WEIGHTS_FILE), expect_manifest_sha256)
    for name in (CONFIG_FILE, WEIGHTS_FILE):
        if not (folder / name).is_file():
            raise FileNotFoundError(f"model folder {folder} has no {name}")
    from paged_kv_serving_b200.config import load_config

    config = load_config(folder / CONFIG_FILE)
    tensors = read_safetensors(folder / WEIGHTS_FILE)
    if manifest is not None:
        cross_check_manifest(manifest, config, tensors)
    return config, tensors


def cross_check_manifest(manifest: dict, config, tensors: dict[str, torch.Tensor]) -> None:
    """What the manifest says about the model against what the folder holds: its
    ``architecture`` must be the configuration that ``config.json`` gives (read through the same
    typed class, so defaults compare equal), and its ``parameter_count`` must be both the number
    of elements in the tensors found and the number the architecture's layout declares
    (reference: src/paged_kv_serving/engine/weights.py:191-200)."""
    from paged_kv_serving_b200.config import registry

    recorded = manifest.get("architecture")
    try:
        same = isinstance(recorded, dict) and type(config).from_dict(recorded).to_dict() == config.to_dict()
    except (TypeError, ValueError):
        same = False
    if not same:
        raise manifest_module.ModelIntegrityError("the manifest's architecture is not the configuration in config.json")
    found = sum(int(t.numel()) for t in tensors.values())
    declared = registry.architecture(config.architecture).layout(config).parameter_count()
    count = manifest.get("parameter_count")
    if count != found or count != declared:
        raise manifest_module.ModelIntegrityError(
            f"parameter count mismatch: the manifest records {count}, the tensors hold {found}, "
            f"the configuration declares {declared}")


def non_finite_tensors(tensors: dict[str, torch.Tensor]) -> list[str]:
    """Names of the floating-point tensors that hold a NaN or an infinite value. The flags are
    gathered where the tensors live and read in one transfer."""
    names = [name for name, t in tensors.items() if t.is_floating_point()]
    if not names:
        return []
    flags = torch.stack([torch.isfinite(tensors[name]).all() for name in names])
    return sorted(name for name, ok in zip(names, flags.cpu().tolist()) if not ok)


def check_finite(tensors: dict[str, torch.Tensor]) -> None:
    """Refuse weights with NaN or infinite values (reference: src/paged_kv_serving/engine/model.py:
    103-128 validates every tensor as finite), in the same error form as the other tensor faults."""
    bad = non_finite_tensors(tensors)
    if bad:
        raise WeightsError([], [], [f"{name}: holds NaN or infinite values" for name in bad])
