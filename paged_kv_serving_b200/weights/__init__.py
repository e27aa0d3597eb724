"""Weights: safetensors by tensor name, the manifest check, the random-weights mode."""

from paged_kv_serving_b200.weights.loader import (
    WEIGHTS_FILE, WeightsError, check_finite, check_tensors, cross_check_manifest, non_finite_tensors, place,
    read_model_folder, read_safetensors,
)
from paged_kv_serving_b200.weights.manifest import (
    MANIFEST_FILE, ModelIntegrityError, manifest_digest, sha256_file, verify_manifest, write_manifest,
)

__all__ = [
    "MANIFEST_FILE", "WEIGHTS_FILE", "ModelIntegrityError", "WeightsError", "check_finite", "check_tensors",
    "cross_check_manifest", "manifest_digest", "non_finite_tensors",
    "place", "read_model_folder", "read_safetensors", "sha256_file", "verify_manifest", "write_manifest",
]
