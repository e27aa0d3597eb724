"""The Python entry point: host token ids in, host token ids out.

``generate`` is the call a user makes; it wraps what the reference reaches through
``Engine.generate`` (src/paged_kv_serving/engine/engine.py:601-605): requests are submitted to
a continuous-batching engine and drained.
"""

from __future__ import annotations

from collections.abc import Sequence as SequenceOf
from pathlib import Path

from paged_kv_serving_b200.config.engine_config import EngineConfig
from paged_kv_serving_b200.engine.engine import Engine
from paged_kv_serving_b200.engine.sequence import Request, SamplingParams

__all__ = ["engine_for", "generate"]


def engine_for(model, prompts: SequenceOf[SequenceOf[int]], *, max_new_tokens: int, n: int = 1,
               dtype: str = "bfloat16", eos_token_id: int | None = None, block_size: int = 16,
               num_blocks: int | None = None, max_batched_tokens: int = 256, max_running_seqs: int = 32,
               enable_prefix_cache: bool = True, expect_manifest_sha256: str | None = None) -> Engine:
    """An engine whose limits fit the given prompts (``model``: a loaded model or a folder)."""
    from paged_kv_serving_b200.models.decoder import DecoderModel

    if isinstance(model, (str, Path)):
        model = DecoderModel.from_folder(model, dtype=dtype, expect_manifest_sha256=expect_manifest_sha256)
    longest = max(len(p) for p in prompts)
    context = min(model.layout.max_positions, longest + max_new_tokens)
    if num_blocks is None:
        per_sequence = -(-context // block_size) + 1
        num_blocks = max(per_sequence, per_sequence * min(max_running_seqs, len(prompts) * n))
    num_blocks = max(num_blocks, -(-context // block_size))
    config = EngineConfig(
        block_size=block_size, num_blocks=num_blocks, max_batched_tokens=max_batched_tokens,
        max_running_seqs=max(max_running_seqs, n), max_prompt_tokens=longest, max_new_tokens=max_new_tokens,
        max_context_tokens=longest + max_new_tokens, enable_prefix_cache=enable_prefix_cache,
        dtype=model.dtype_name)
    return Engine(model, config, eos_token_id=eos_token_id)


def generate(model, prompts: SequenceOf[SequenceOf[int]], *, max_new_tokens: int = 32, temperature: float = 0.0,
             top_p: float = 1.0, seed: int = 0, n: int = 1, **engine_options) -> list[list[list[int]]]:
    """Generated token ids for every prompt: ``result[prompt][sample]`` is a list of ids.

    ``seed`` is the first request's seed; request ``i`` uses ``seed + i`` so that equal prompts
    do not repeat each other's draws.
    """
    engine = engine_for(model, prompts, max_new_tokens=max_new_tokens, n=n, **engine_options)
    requests = [
        Request(request_id=f"request-{i}", prompt_token_ids=tuple(int(t) for t in prompt),
                sampling=SamplingParams(max_new_tokens=max_new_tokens, temperature=temperature, top_p=top_p,
                                        seed=seed + i), n=n)
        for i, prompt in enumerate(prompts)
    ]
    refused = [r.request_id for r in requests if not engine.submit(r).admitted]
    if refused:
        raise ValueError(f"requests refused by the engine's limits: {', '.join(refused)}")
    outputs = {o.request_id: o for o in engine.run_until_idle()}
    return [[list(s.token_ids) for s in outputs[r.request_id].samples] for r in requests]
