"""A model instance: a layout whose parts hold their tensors on the device."""

from __future__ import annotations

from pathlib import Path

import torch

from paged_kv_serving_b200.config import registry
from paged_kv_serving_b200.config.model_config import ModelConfig
from paged_kv_serving_b200.models.layout import ModelLayout
from paged_kv_serving_b200.weights import loader, random_init

__all__ = ["DecoderModel", "TORCH_DTYPES"]

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class DecoderModel:
    """Configuration, layout and loaded tensors of one model, in one compute type.

    ``dtype`` is ``"bfloat16"`` (matrices and activations in bfloat16, residual stream, norms,
    softmax and rotation in float32) or ``"float32"`` (everything in true float32).
    """

    def __init__(self, config: ModelConfig, layout: ModelLayout, dtype: str, device: torch.device) -> None:
        if dtype not in TORCH_DTYPES:
            raise ValueError(f"dtype must be one of {', '.join(TORCH_DTYPES)}")
        self.config = config
        self.layout = layout
        self.dtype_name = dtype
        self.dtype = TORCH_DTYPES[dtype]
        self.device = torch.device(device)

    # --- construction --------------------------------------------------------------------

    @classmethod
    def from_tensors(cls, config: ModelConfig, tensors: dict[str, torch.Tensor], dtype: str = "bfloat16",
                     device: str | torch.device = "cuda") -> "DecoderModel":
        """Build from a name -> tensor mapping (as read from safetensors, or drawn at random)."""
        layout = registry.architecture(config.architecture).layout(config)
        model = cls(config, layout, dtype, torch.device(device))
        specs = layout.tensor_specs()
        loader.check_tensors(specs, tensors)
        placed = {name: loader.place(tensors[name], spec, model.dtype, model.device) for name, spec in specs.items()}
        loader.check_finite(placed)      # one pass on the device, after the cast to the compute type
        per_part: dict[int, tuple[object, dict[str, torch.Tensor]]] = {}
        for name, (part, local) in layout.names.items():
            per_part.setdefault(id(part), (part, {}))[1][local] = placed[name]
        for part, params in per_part.values():
            part.load(params)
        return model

    @classmethod
    def from_folder(cls, folder: str | Path, dtype: str = "bfloat16", device: str | torch.device = "cuda",
                    expect_manifest_sha256: str | None = None) -> "DecoderModel":
        """Load ``config.json`` and ``model.safetensors`` (checked against ``manifest.json`` when
        the folder has one) and build the model the configuration names."""
        config, tensors = loader.read_model_folder(folder, expect_manifest_sha256=expect_manifest_sha256)
        return cls.from_tensors(config, tensors, dtype, device)

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int = 0, dtype: str = "bfloat16",
                    device: str | torch.device = "cuda", std: float = 0.02) -> "DecoderModel":
        """Random weights drawn directly on the device (for sizes that are never written out)."""
        layout = registry.architecture(config.architecture).layout(config)
        tensors = random_init.random_tensors_on_device(layout.tensor_specs(), seed, std, TORCH_DTYPES[dtype],
                                                       torch.device(device))
        return cls.from_tensors(config, tensors, dtype, device)

    # --- sizes used by the measurement ----------------------------------------------------

    def weight_bytes_read_per_step(self) -> int:
        """Bytes of weights one decode step has to read: every matrix once (the embedding table
        only by row, so it counts only as the head when tied or not at all when untied)."""
        element = torch.empty((), dtype=self.dtype).element_size()
        head = getattr(self.layout.head, "weight", None)
        total = head.numel() * head.element_size() if head is not None else 0
        seen = set()
        for name, (part, local) in self.layout.names.items():
            if part is self.layout.embedding or part is self.layout.head:
                continue                    # the table is read by row; the head is counted above
            spec = part.param_specs()[local]
            count = 1
            for s in spec.shape:
                count *= s
            key = (id(part), local)
            if key in seen:
                continue
            seen.add(key)
            total += count * (element if spec.kind == "matrix" else 4)
        return total
