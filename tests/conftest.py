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


@pytest.fixture(autouse=True)
def fused_gate_up_at_test_sizes(request):
    """The engine sends the gate/up product of a portion to the fused tcgen05 kernel only from
    ``ops.gemm.SILU_TCGEN05_MIN_ROWS`` rows on (about 1,500: below that the library is faster at
    the sizes of real models). The prompts of these tests are far shorter, so the GPU tests lower
    the switch to the kernel's own minimum and keep running it inside whole models; one test of
    tests/test_gpu_replay.py runs the routing as shipped."""
    if "gpu" not in request.keywords:
        yield
        return
    from paged_kv_serving_b200.ops import gemm

    before = gemm.SILU_TCGEN05_MIN_ROWS
    gemm.SILU_TCGEN05_MIN_ROWS = gemm.TCGEN05_MIN_ROWS
    try:
        yield
    finally:
        gemm.SILU_TCGEN05_MIN_ROWS = before


def pytest_terminal_summary(terminalreporter):
    try:
        import helpers
    except Exception:  # pragma: no cover
        return
    if helpers.WORST_SHARE:
        shares = ", ".join(f"{dtype} {share:.2f}" for dtype, share in sorted(helpers.WORST_SHARE.items()))
        terminalreporter.write_line(f"largest logit gap as a share of its bound: {shares}")
