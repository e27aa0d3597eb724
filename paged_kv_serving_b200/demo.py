"""The offline demo: a tiny random model, generated tokens, and the logit gap between ways of
cutting the same work (whole prompt, token by token, uneven portions). The reference's demo
does the same on its NumPy engine (src/paged_kv_serving/engine/demo.py:97-152)."""

from __future__ import annotations

from pathlib import Path

import numpy as np

__all__ = ["run_demo"]


def run_demo(workdir: str | Path) -> dict:
    from paged_kv_serving_b200.api import generate
    from paged_kv_serving_b200.config.presets import preset
    from paged_kv_serving_b200.engine.replay import ReplaySession
    from paged_kv_serving_b200.models.decoder import DecoderModel
    from paged_kv_serving_b200.weights.random_init import write_random_model_folder

    workdir = Path(workdir)
    folder = workdir / "checkpoint"
    config = preset("reference-default")
    write_random_model_folder(folder, config, seed=0, dtype="float32", std=0.05)
    summary: dict = {"parameters": config.parameter_count}
    rng = np.random.default_rng(1)
    prompts = [[int(t) for t in rng.integers(0, config.vocab_size, size=n)] for n in (5, 9, 17)]
    for dtype in ("float32", "bfloat16"):
        model = DecoderModel.from_folder(folder, dtype=dtype)
        summary[f"tokens_{dtype}"] = generate(model, prompts, max_new_tokens=8)
        tokens = [int(t) for t in rng.integers(0, config.vocab_size, size=90)]
        rows = {}
        for name, sizes in (("whole", [90]), ("token_by_token", [1] * 90), ("uneven", [7, 3, 11, 5, 2, 2, 13, 47])):
            session = ReplaySession(model, max_tokens=128, block_size=16)
            start = 0
            for size in sizes:
                out = session.step([{"id": "d", "tokens": tokens[start:start + size], "want": [size - 1]}])
                start += size
            rows[name] = out[0]
        summary[f"gap_{dtype}"] = {name: float(np.abs(rows[name] - rows["whole"]).max()) for name in rows}
    return summary
