"""Builds and loads the CUDA libraries of ``csrc`` on demand.

Each ``.cu`` file becomes one shared library, compiled for sm_100a with ``nvcc`` the first
time a function of it is needed and cached under a name that carries a hash of its sources and
flags. The cache lives in ``_build`` inside the package when that is writable, else in a
per-user folder under the system's temporary directory, so a fresh checkout owned by another
user, or a user without a home directory, still works. While ``nvcc`` runs, a line is printed
every few seconds. There is no fallback: a missing compiler or a failed build raises.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

__all__ = ["CSRC", "NVCC_FLAGS", "build_all", "library", "library_names"]

CSRC = Path(__file__).resolve().parent.parent / "csrc"
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
)
_LOADED: dict[str, ctypes.CDLL] = {}
_LOCK = threading.Lock()


def library_names() -> tuple[str, ...]:
    return tuple(sorted(path.stem for path in CSRC.glob("*.cu")))


def _nvcc() -> str:
    for candidate in (os.environ.get("PKV_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    raise RuntimeError(
        "the CUDA kernels of paged_kv_serving_b200 are not built and nvcc was not found "
        "(looked at $PKV_NVCC, PATH and /usr/local/cuda/bin/nvcc); there is no fallback path"
    )


def _source_hash(name: str) -> str:
    digest = hashlib.sha256()
    digest.update(" ".join(NVCC_FLAGS).encode())
    for path in [CSRC / f"{name}.cu", *sorted(CSRC.glob("*.cuh")), *sorted(CSRC.glob("*.h"))]:
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()[:16]


def _build_dirs() -> list[Path]:
    dirs = []
    if os.environ.get("PKV_BUILD_DIR"):
        dirs.append(Path(os.environ["PKV_BUILD_DIR"]))
    dirs.append(CSRC.parent / "_build")
    dirs.append(Path(tempfile.gettempdir()) / f"paged_kv_serving_b200-build-{os.getuid()}")
    return dirs


def _writable(directory: Path) -> bool:
    try:
        directory.mkdir(parents=True, exist_ok=True)
        probe = directory / f".probe-{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return True
    except OSError:
        return False


def _compile(name: str, target: Path) -> None:
    nvcc = _nvcc()
    source = CSRC / f"{name}.cu"
    partial = target.with_name(f"{target.name}.{os.getpid()}.tmp")
    command = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), str(source), "-o", str(partial)]
    started = time.monotonic()
    print(f"[paged_kv_serving_b200] compiling {source.name} for sm_100a ...", file=sys.stderr, flush=True)
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    output: list[str] = []
    reader = threading.Thread(target=lambda: output.append(process.stdout.read()), daemon=True)
    reader.start()
    while True:
        try:
            process.wait(timeout=5.0)
            break
        except subprocess.TimeoutExpired:
            print(f"[paged_kv_serving_b200] still compiling {source.name} "
                  f"({time.monotonic() - started:.0f} s)", file=sys.stderr, flush=True)
    reader.join()
    if process.returncode != 0:
        partial.unlink(missing_ok=True)
        raise RuntimeError(f"nvcc failed for {source}:\n{''.join(output)}")
    os.replace(partial, target)
    print(f"[paged_kv_serving_b200] built {target.name} in {time.monotonic() - started:.1f} s",
          file=sys.stderr, flush=True)


def _locate_or_build(name: str) -> Path:
    if not (CSRC / f"{name}.cu").is_file():
        raise RuntimeError(f"no CUDA source {name}.cu in {CSRC}")
    file_name = f"{name}-{_source_hash(name)}.so"
    for directory in _build_dirs():
        if (directory / file_name).is_file():
            return directory / file_name
    for directory in _build_dirs():
        if _writable(directory):
            _compile(name, directory / file_name)
            return directory / file_name
    raise RuntimeError("no writable folder for the compiled CUDA kernels (set PKV_BUILD_DIR)")


def library(name: str) -> ctypes.CDLL:
    """The loaded shared library of ``csrc/<name>.cu``, building it first if needed."""
    with _LOCK:
        lib = _LOADED.get(name)
        if lib is None:
            lib = ctypes.CDLL(str(_locate_or_build(name)))
            _LOADED[name] = lib
        return lib


def build_all(prune: bool = True) -> list[Path]:
    """Compile every library (used by the build check); returns their paths. ``prune`` removes
    libraries of earlier source versions from the folders the new ones went to."""
    built = [_locate_or_build(name) for name in library_names()]
    if prune:
        current = {path.name for path in built}
        for directory in {path.parent for path in built}:
            for stale in directory.glob("*-????????????????.so"):
                if stale.name not in current:
                    stale.unlink(missing_ok=True)
    return built
