"""The hash manifest of a model folder.

A model folder may carry ``manifest.json`` with the SHA-256 and size of its other files; when
it does, every digest is checked before a single tensor is parsed, and a caller can pin the
manifest's own digest. Behaviour follows the reference's checkpoint check
(src/paged_kv_serving/engine/weights.py:61-121, 168-200; canonical JSON digest:
src/paged_kv_serving/core/canonical.py:47-58): plain file names only, no duplicates, required
files must be covered, size before hash.
"""

from __future__ import annotations

import hashlib
import json
import os
import re
import tempfile
from pathlib import Path
from typing import Any

__all__ = ["MANIFEST_FILE", "ModelIntegrityError", "manifest_digest", "sha256_file", "verify_manifest", "write_manifest"]

MANIFEST_FILE = "manifest.json"
_PLAIN_NAME = re.compile(r"^[A-Za-z0-9][A-Za-z0-9._-]{0,127}$")
_HEX64 = re.compile(r"^[0-9a-f]{64}$")
_KEYS = {"schema_version", "architecture", "parameter_count", "artifacts"}


class ModelIntegrityError(ValueError):
    """A file of a model folder does not match what its manifest records."""


def sha256_file(path: Path, chunk: int = 1 << 20) -> str:
    digest = hashlib.sha256()
    with open(path, "rb") as handle:
        while True:
            block = handle.read(chunk)
            if not block:
                break
            digest.update(block)
    return digest.hexdigest()


def canonical_json(value: Any) -> bytes:
    return json.dumps(value, sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode("utf-8")


def manifest_digest(manifest: dict[str, Any]) -> str:
    """SHA-256 of the manifest's canonical JSON: the value to pin out of band."""
    return hashlib.sha256(canonical_json(manifest)).hexdigest()


def _atomic_write(path: Path, text: str) -> None:
    handle, temp = tempfile.mkstemp(dir=str(path.parent), prefix=path.name + ".")
    try:
        with os.fdopen(handle, "w", encoding="utf-8") as out:
            out.write(text)
        os.replace(temp, path)
    except BaseException:
        Path(temp).unlink(missing_ok=True)
        raise


def write_manifest(folder: Path, architecture: dict[str, Any], parameter_count: int, files: tuple[str, ...]) -> dict:
    manifest = {
        "schema_version": 1,
        "architecture": architecture,
        "parameter_count": int(parameter_count),
        "artifacts": [
            {"name": name, "sha256": sha256_file(folder / name), "size_bytes": (folder / name).stat().st_size}
            for name in files
        ],
    }
    _atomic_write(folder / MANIFEST_FILE, json.dumps(manifest, indent=2, sort_keys=True) + "\n")
    return manifest


def verify_manifest(folder: Path, required: tuple[str, ...], expect_sha256: str | None = None) -> dict[str, Any]:
    """Check every digest the manifest lists; raise ``ModelIntegrityError`` on any mismatch."""
    path = folder / MANIFEST_FILE
    if not path.is_file():
        raise ModelIntegrityError(f"no {MANIFEST_FILE} in {folder}")
    try:
        manifest = json.loads(path.read_text(encoding="utf-8"))
    except json.JSONDecodeError as error:
        raise ModelIntegrityError(f"{MANIFEST_FILE} is not valid JSON: {error}") from None
    if not isinstance(manifest, dict) or set(manifest) != _KEYS:
        raise ModelIntegrityError(f"{MANIFEST_FILE} must have exactly the keys {sorted(_KEYS)}")
    if manifest["schema_version"] != 1:
        raise ModelIntegrityError("unknown manifest schema_version")
    if expect_sha256 is not None and manifest_digest(manifest) != expect_sha256:
        raise ModelIntegrityError("manifest digest does not match the pinned value")
    artifacts = manifest["artifacts"]
    if not isinstance(artifacts, list):
        raise ModelIntegrityError("manifest artifacts must be a list")
    names = []
    for artifact in artifacts:
        if not isinstance(artifact, dict) or set(artifact) != {"name", "sha256", "size_bytes"}:
            raise ModelIntegrityError("a manifest artifact must have exactly name, sha256 and size_bytes")
        name = artifact["name"]
        if not isinstance(name, str) or not _PLAIN_NAME.fullmatch(name) or ".." in name:
            raise ModelIntegrityError("an artifact name must be a plain file name inside the model folder")
        if not isinstance(artifact["sha256"], str) or not _HEX64.fullmatch(artifact["sha256"]):
            raise ModelIntegrityError(f"{name}: malformed sha256")
        if not isinstance(artifact["size_bytes"], int) or artifact["size_bytes"] < 0:
            raise ModelIntegrityError(f"{name}: malformed size_bytes")
        names.append(name)
    if len(names) != len(set(names)):
        raise ModelIntegrityError("an artifact is listed more than once")
    for name in required:
        if name not in names:
            raise ModelIntegrityError(f"manifest does not cover {name}")
    for artifact in artifacts:
        file_path = folder / artifact["name"]
        if not file_path.is_file():
            raise ModelIntegrityError(f"missing model file {artifact['name']}")
        if file_path.stat().st_size != artifact["size_bytes"]:
            raise ModelIntegrityError(f"{artifact['name']} has an unexpected size")
        if sha256_file(file_path) != artifact["sha256"]:
            raise ModelIntegrityError(f"{artifact['name']} does not match its manifest digest")
    return manifest
