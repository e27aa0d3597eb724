"""Command line: ``python -m paged_kv_serving_b200 <command>``.

Sub-commands follow the reference's command line where it has them
(src/paged_kv_serving/cli.py:124-179: ``build-checkpoint --out --seed``, ``demo --workdir``);
``generate`` and ``replay`` are this engine's (the reference reaches generation through Python
and HTTP only), with option names taken from the reference's ``SamplingParams`` and
``EngineConfig`` fields.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

__all__ = ["main"]


def _model_config(args):
    """The typed configuration of whatever architecture the file names (its own config class
    where it has one), or a preset."""
    from paged_kv_serving_b200.config import load_config
    from paged_kv_serving_b200.config.presets import preset

    if args.config is not None:
        return load_config(args.config)
    return preset(args.preset)


def _build_checkpoint(args) -> int:
    from paged_kv_serving_b200.weights.manifest import manifest_digest
    from paged_kv_serving_b200.weights.random_init import write_random_model_folder

    config = _model_config(args)
    manifest = write_random_model_folder(args.out, config, seed=args.seed, dtype=args.dtype, std=args.std)
    print(json.dumps({"directory": str(args.out), "parameters": manifest["parameter_count"],
                      "vocab_size": config.vocab_size, "manifest_sha256": manifest_digest(manifest)}, indent=2))
    return 0


def _engine_config(args, model_config):
    from paged_kv_serving_b200.config.engine_config import EngineConfig

    return EngineConfig(
        block_size=args.block_size, num_blocks=args.num_blocks, max_batched_tokens=args.max_batched_tokens,
        max_running_seqs=args.max_running_seqs, max_prompt_tokens=args.max_prompt_tokens,
        max_new_tokens=max(args.max_new_tokens, 1),
        max_context_tokens=min(model_config.max_seq_len, args.max_prompt_tokens + max(args.max_new_tokens, 1)),
        enable_prefix_cache=not args.no_prefix_cache, dtype=args.dtype)


def _parse_prompts(args) -> list[list[int]]:
    prompts: list[list[int]] = []
    for text in args.prompt_ids or []:
        prompts.append([int(t) for t in text.replace(",", " ").split()])
    if args.prompt_file is not None:
        for line in Path(args.prompt_file).read_text(encoding="utf-8").splitlines():
            line = line.strip()
            if line:
                prompts.append([int(t) for t in (json.loads(line) if line.startswith("[") else line.replace(",", " ").split())])
    if not prompts:
        raise SystemExit("give at least one prompt with --prompt-ids or --prompt-file")
    return prompts


def _generate(args) -> int:
    from paged_kv_serving_b200.api import generate

    prompts = _parse_prompts(args)
    outputs = generate(
        args.model, prompts, max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_p=args.top_p,
        seed=args.seed, n=args.n, dtype=args.dtype, eos_token_id=args.eos_token_id, block_size=args.block_size,
        num_blocks=args.num_blocks, max_batched_tokens=args.max_batched_tokens,
        max_running_seqs=args.max_running_seqs, enable_prefix_cache=not args.no_prefix_cache,
        expect_manifest_sha256=args.expect_manifest_sha256)
    for prompt, samples in zip(prompts, outputs):
        print(json.dumps({"prompt_token_ids": prompt, "samples": samples}))
    return 0


def _replay(args) -> int:
    from paged_kv_serving_b200.engine.replay import main as replay_main

    forwarded = ["--model", str(args.model), "--dtype", args.dtype, "--out", str(args.out),
                 "--max-tokens", str(args.max_tokens), "--block-size", str(args.block_size)]
    if args.trace is not None:
        sys.stdin = open(args.trace, encoding="utf-8")
    return replay_main(forwarded)


def _demo(args) -> int:
    from paged_kv_serving_b200.demo import run_demo

    summary = run_demo(args.workdir)
    print(json.dumps(summary, indent=2, sort_keys=True))
    return 0


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="paged_kv_serving_b200")
    sub = parser.add_subparsers(dest="command", required=True)

    build = sub.add_parser("build-checkpoint", help="write a deterministic random-weights model folder")
    build.add_argument("--out", type=Path, default=Path("var/checkpoint"))
    build.add_argument("--seed", type=int, default=0)
    build.add_argument("--preset", default="reference-default")
    build.add_argument("--config", type=Path, default=None, help="a config.json to use instead of a preset")
    build.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    build.add_argument("--std", type=float, default=0.02)

    gen = sub.add_parser("generate", help="generate tokens for prompts given as token ids")
    gen.add_argument("--model", type=Path, required=True, help="folder with config.json and model.safetensors")
    gen.add_argument("--prompt-ids", action="append", help="token ids, comma or space separated (repeatable)")
    gen.add_argument("--prompt-file", type=Path, default=None, help="one prompt per line")
    gen.add_argument("--max-new-tokens", type=int, default=32)
    gen.add_argument("--temperature", type=float, default=0.0)
    gen.add_argument("--top-p", type=float, default=1.0)
    gen.add_argument("--seed", type=int, default=0)
    gen.add_argument("--n", type=int, default=1)
    gen.add_argument("--eos-token-id", type=int, default=None)
    gen.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    gen.add_argument("--block-size", type=int, default=16)
    gen.add_argument("--num-blocks", type=int, default=512)
    gen.add_argument("--max-batched-tokens", type=int, default=256)
    gen.add_argument("--max-running-seqs", type=int, default=32)
    gen.add_argument("--no-prefix-cache", action="store_true")
    gen.add_argument("--expect-manifest-sha256", default=None)

    replay = sub.add_parser("replay", help="feed a trace of token ids step by step and write logits")
    replay.add_argument("trace", nargs="?", type=Path, default=None, help="trace file (default: standard input)")
    replay.add_argument("--model", type=Path, required=True)
    replay.add_argument("--dtype", choices=("bfloat16", "float32"), required=True)
    replay.add_argument("--out", type=Path, required=True)
    replay.add_argument("--max-tokens", type=int, required=True)
    replay.add_argument("--block-size", type=int, default=16)

    demo = sub.add_parser("demo", help="run the offline end-to-end demo on the GPU")
    demo.add_argument("--workdir", type=Path, default=Path("var/demo"))

    args = parser.parse_args(argv)
    if args.command == "build-checkpoint":
        return _build_checkpoint(args)
    if args.command == "generate":
        return _generate(args)
    if args.command == "replay":
        return _replay(args)
    return _demo(args)


if __name__ == "__main__":
    raise SystemExit(main())
