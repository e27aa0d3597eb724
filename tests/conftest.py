"""Test configuration: the ``gpu`` marker and import paths."""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for path in (str(ROOT), str(ROOT / "tests")):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA GPU in this environment")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    try:
        import helpers
    except Exception:  # pragma: no cover
        return
    if helpers.WORST_SHARE:
        shares = ", ".join(f"{dtype} {share:.2f}" for dtype, share in sorted(helpers.WORST_SHARE.items()))
        terminalreporter.write_line(f"largest logit gap as a share of its bound: {shares}")
