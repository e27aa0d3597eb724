"""What ``bench.py`` promises without a GPU: the reference arm's line and the refusal of more than one GPU."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_reference_arm_prints_one_unavailable_line_and_exits_zero():
    done = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert done.returncode == 0
    lines = [line for line in done.stdout.splitlines() if line.strip()]
    assert len(lines) == 1
    record = json.loads(lines[0])
    assert record["impl"] == "reference" and isinstance(record["unavailable"], str) and "\n" not in record["unavailable"]


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_two():
    done = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert done.returncode == 2
    lines = [line for line in (done.stdout + done.stderr).splitlines() if line.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]
