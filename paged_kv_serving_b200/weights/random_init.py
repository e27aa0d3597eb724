"""The random-weights mode: tensors from a configuration and a seed, and model folders of them.

Matrices are drawn from ``N(0, std)`` and norm weights are ones (plus an optional jitter, for
tests that must notice a wrong norm weight). Two generators exist and are documented apart:
``random_tensors`` draws on the host with NumPy's PCG64 in sorted tensor-name order and is what
model folders are written from, so that any other program can draw the same arrays;
``random_tensors_on_device`` draws with torch's device generator for shapes too large to pass
through the host (benchmarks). A bfloat16 tensor is the round-to-nearest of the float32 draw.
The reference's own scheme (src/paged_kv_serving/engine/model.py:173-203) uses other scales
(``d^-0.5``, ``ff^-0.5``, 0.05); ``std`` may be a callable of the tensor name to imitate it.
"""

from __future__ import annotations

from collections.abc import Callable
from pathlib import Path

import numpy as np
import torch

from paged_kv_serving_b200.config import registry
from paged_kv_serving_b200.config.model_config import CONFIG_FILE
from paged_kv_serving_b200.parts.base import ParamSpec
from paged_kv_serving_b200.weights import manifest as manifest_module
from paged_kv_serving_b200.weights.loader import WEIGHTS_FILE

__all__ = ["random_tensors", "random_tensors_on_device", "write_model_folder", "write_random_model_folder"]


def random_tensors(specs: dict[str, ParamSpec], seed: int, std: float | Callable[[str], float] = 0.02,
                   norm_jitter: float = 0.0, dtype: torch.dtype = torch.float32) -> dict[str, torch.Tensor]:
    """Host tensors for every name in ``specs``; matrices in ``dtype``, vectors in float32."""
    rng = np.random.default_rng(seed)
    out: dict[str, torch.Tensor] = {}
    for name in sorted(specs):
        spec = specs[name]
        if spec.kind == "int_table":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32)
        elif spec.kind == "vector":
            values = (1.0 + norm_jitter * rng.standard_normal(spec.shape)).astype(np.float32)
            out[name] = torch.from_numpy(values)
        else:
            scale = std(name) if callable(std) else std
            values = (rng.standard_normal(spec.shape) * scale).astype(np.float32)
            out[name] = torch.from_numpy(values).to(dtype)
    return out


def random_tensors_on_device(specs: dict[str, ParamSpec], seed: int, std: float, dtype: torch.dtype,
                             device: torch.device) -> dict[str, torch.Tensor]:
    generator = torch.Generator(device=device)
    generator.manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for name in sorted(specs):
        spec = specs[name]
        if spec.kind == "int_table":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
        elif spec.kind == "vector":
            out[name] = torch.ones(spec.shape, dtype=torch.float32, device=device)
        else:
            rows = spec.shape[0]
            tensor = torch.empty(spec.shape, dtype=dtype, device=device)
            step = max(1, (64 << 20) // max(1, int(np.prod(spec.shape[1:]))))   # draw in float32 slabs
            for start in range(0, rows, step):
                stop = min(rows, start + step)
                slab = torch.randn((stop - start, *spec.shape[1:]), dtype=torch.float32, device=device,
                                   generator=generator)
                tensor[start:stop] = (slab * std).to(dtype)
            out[name] = tensor
    return out


def write_model_folder(folder: str | Path, config, tensors: dict[str, torch.Tensor]) -> dict:
    """Write ``config.json``, ``model.safetensors`` and ``manifest.json``; returns the manifest.
    ``config`` is the typed configuration of any registered architecture (it names its
    architecture and offers ``to_dict``); the parameter count comes from the architecture's
    layout, not from a formula of one model."""
    from safetensors.torch import save_file

    from paged_kv_serving_b200.config import write_config

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    write_config(config, folder / CONFIG_FILE)
    save_file({name: tensor.detach().cpu().contiguous() for name, tensor in tensors.items()},
              str(folder / WEIGHTS_FILE))
    layout = registry.architecture(config.architecture).layout(config)
    return manifest_module.write_manifest(folder, config.to_dict(), layout.parameter_count(),
                                          (CONFIG_FILE, WEIGHTS_FILE))


def write_random_model_folder(folder: str | Path, config, seed: int = 0, dtype: str = "bfloat16",
                              std: float = 0.02, norm_jitter: float = 0.0) -> dict:
    """The random-weights mode: a model folder from a configuration and a seed."""
    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    layout = registry.architecture(config.architecture).layout(config)
    tensors = random_tensors(layout.tensor_specs(), seed, std, norm_jitter, torch_dtype)
    return write_model_folder(folder, config, tensors)
