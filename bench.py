"""Measurement of the engine on one B200: decode and prefill throughput against the roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of the Llama-3-8B shape (the third configuration of the
baseline list) with random bfloat16 weights: 8 sequences, each with a 1,024-token random prompt
in the cache, decode one token per step. A "step" is one decode step of the whole batch. One JSON
line is printed with

* ``value``      decoded tokens a second, timed on the device with CUDA events over K steps;
                 each step runs the model and samples, the sampled ids enter the next step on the
                 device, and the host prepares step k + 1 while the GPU runs step k (synchronised
                 before and after the K steps)
* ``e2e``        the same through the Python entry point (``Engine.step``): host token ids in,
                 sampled ids read back every step, with the host-to-device and device-to-host
                 bytes of a step and the roofline fraction that its time amounts to
* ``prefill``    one 2,048-token prompt in one step: tokens a second, milliseconds and the
                 fraction of the bfloat16 matrix peak its flops reach
* ``roofline``   the bytes a decode step must read (every weight once, the cache of the live
                 requests) over its time, against the measured copy bandwidth
* ``points``     decode tokens a second at batch 1 and 64
* ``mixed``      Llama-2-13B layer sizes: one step of 32 decoding sequences at 2,048 tokens of
                 context beside a 512-token portion of a prompt, with its bytes against the bandwidth
* ``serve``      Llama-3.2-1B layer sizes: 256 requests with prompts of 128 to 4,096 tokens sharing a
                 512-token prefix, 128 tokens each at temperature 0.7, through ``Engine`` with the
                 prefix cache: output tokens a second, prefix hit ratio, preemptions
* ``reference_workload``  this engine on the reference's own published workload (a tiny float32
                 model); ``--impl reference`` times the reference itself on it, as context

Peaks come from ``MEASURED_PEAKS.json`` beside this file when it exists, else from fallback
figures (6.65 TB/s, 1.59 PFLOP/s). Weights of a step (16 GB) are far larger than L2, so nothing is flushed
between steps. With ``--gpus`` above 1 the program says that it measures one GPU only and exits 2.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "decode tok/s at batch {batch}, {model} shape, {prompt}-token prompts"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            peaks = {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in data:
                peaks["bf16_tflops_sustained"] = float(data["bf16_tflops_sustained"])
            return peaks
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self) -> None:
        self.process = None
        self.samples: list[str] = []

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None

    def stop(self) -> None:
        if self.process is None:
            return
        self.process.terminate()
        try:
            out, _ = self.process.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
            out, _ = self.process.communicate()
        self.samples += [line for line in out.splitlines() if line.strip()]
        self.process = None

    def summary(self) -> dict:
        clocks, maxima, reasons = [], [], set()
        for line in self.samples:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                maxima.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(self.NAMES, parts[2:6]):
                if value.lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": sorted(reasons), "samples": len(clocks)}


def scattered_tables(num_seqs: int, pages_per_seq: int) -> list[tuple[int, ...]]:
    """Page tables that interleave the sequences' pages, so that no sequence is contiguous."""
    return [tuple(j * num_seqs + i for j in range(pages_per_seq)) for i in range(num_seqs)]


def run(args) -> dict:
    import numpy as np
    import torch

    from paged_kv_serving_b200 import ops
    from paged_kv_serving_b200.config import EngineConfig
    from paged_kv_serving_b200.config.presets import PRESETS, preset
    from paged_kv_serving_b200.engine.batch import BatchEntry, ExecutionBatch
    from paged_kv_serving_b200.engine.engine import Engine
    from paged_kv_serving_b200.engine.runner import ModelRunner
    from paged_kv_serving_b200.engine.sequence import Request, SamplingParams
    from paged_kv_serving_b200.models.decoder import DecoderModel
    from paged_kv_serving_b200.sampling.sampler import Sampler

    peaks = load_peaks()
    full_layers = PRESETS[args.model]["n_layers"]
    layers = args.layers or full_layers
    config = preset(args.model, n_layers=layers)
    torch.cuda.set_device(0)
    model = DecoderModel.from_random(config, seed=0, dtype="bfloat16", device="cuda:0")
    rng = np.random.default_rng(1)
    prompt_len, block, batch = args.prompt_len, 16, args.batch
    max_batch = max(batch, 64 if not args.skip_points else batch)
    decode_room = args.warmup + args.steps + 8
    pages_per_seq = -(-(prompt_len + 3 * decode_room) // block)
    prefill_pages = -(-args.prefill_tokens // block)
    runner = ModelRunner(model, num_blocks=max_batch * pages_per_seq + prefill_pages, block_size=block,
                         max_running_seqs=max_batch)
    sampler = Sampler(model.device)
    tables = scattered_tables(max_batch, pages_per_seq)
    prompts = rng.integers(0, config.vocab_size, size=(max_batch, prompt_len + 4 * decode_room))
    greedy = SamplingParams(max_new_tokens=1)
    clocks = ClockSampler()

    def timed(fn, repeat: int) -> float:
        """Milliseconds for ``repeat`` calls of fn(i), on the device."""
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for i in range(repeat):
            fn(i)
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop)

    # ---- prefill: one 2,048-token prompt in one step, time to its last logits -----------------
    prefill_table = tuple(range(max_batch * pages_per_seq, max_batch * pages_per_seq + prefill_pages))
    prefill_ids = tuple(int(t) for t in rng.integers(0, config.vocab_size, size=args.prefill_tokens))
    prefill_batch = ExecutionBatch((BatchEntry("prefill", prefill_ids, 0, (prefill_table,), (args.prefill_tokens - 1,)),))
    for _ in range(3):
        runner.step(prefill_batch)
    clocks.start()
    prefill_ms = timed(lambda i: runner.step(prefill_batch), 3) / 3
    t = args.prefill_tokens
    gemm_flops = 2.0 * t * layers * (config.d_model * (config.q_width + 2 * config.kv_width)
                                     + config.q_width * config.d_model + 3 * config.d_model * config.d_ff)
    gemm_flops += 2.0 * config.d_model * config.vocab_size
    attention_flops = 4.0 * layers * config.n_heads * config.head_dim * (t * (t + 1) / 2)
    prefill_flops = gemm_flops + attention_flops
    prefill = {"value": t / (prefill_ms / 1e3), "tokens": t, "ms": prefill_ms,
               "frac": prefill_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)}
    if "bf16_tflops_sustained" in peaks:
        # beside the burst rate: the library's rate in a seconds-long loop under the power cap
        prefill["frac_of_sustained"] = prefill_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12)

    # ---- fill the cache of every sequence (not timed) ------------------------------------------
    per_step = max(1, 4096 // prompt_len)
    for first in range(0, max_batch, per_step):
        entries = tuple(BatchEntry(f"s{i}", tuple(int(x) for x in prompts[i, :prompt_len]), 0, (tables[i],), ())
                        for i in range(first, min(max_batch, first + per_step)))
        runner.step(ExecutionBatch(entries))
    torch.cuda.synchronize()

    # ---- decode, timed on the device ------------------------------------------------------------
    weight_bytes = model.weight_bytes_read_per_step()
    kv_bytes_per_token = sum(2 * len(g.entries) * g.n_kv_heads * g.head_dim * 2 for g in runner.groups)

    def decode(num_seqs: int, warmup: int, steps: int, offset: int):
        """``steps`` decode steps of the first ``num_seqs`` sequences; returns (ms, launches)."""
        feedback = {f"s{i}": i for i in range(num_seqs)}
        fed = [None]        # the first step of a run takes its tokens from the host, the others feed back

        def one(k):
            position = prompt_len + offset + k
            entries = tuple(BatchEntry(f"s{i}", (int(prompts[i, position]),), position, (tables[i],), (0,))
                            for i in range(num_seqs))
            result = runner.step(ExecutionBatch(entries), feedback=fed[0])
            # sampled on the device into the buffer that the next step's embedding lookup reads:
            # every step runs the tokens the step before it sampled, and between the
            # synchronisations around the timed steps the host prepares step k + 1 while the GPU
            # runs step k (the end-to-end number below also reads every step's tokens back)
            sampler.sample_on_device(result.logits, [greedy] * num_seqs, [None] * num_seqs, out=runner.sampled_ids)
            runner.prepare_next()
            fed[0] = feedback
        for k in range(warmup):
            one(k)
        before = ops.launch_count()
        ms = timed(lambda k: one(warmup + k), steps)
        return ms, ops.launch_count() - before

    points = {}
    offset = 0
    if not args.skip_points:
        for name, size in (("decode_b1", 1), ("decode_b64", 64)):
            ms, _ = decode(size, 3, min(args.steps, 32), offset)
            offset += 3 + min(args.steps, 32)
            points[name] = size * min(args.steps, 32) / (ms / 1e3)
    decode_ms, launches = decode(batch, args.warmup, args.steps, offset)
    offset += args.warmup + args.steps
    ms_per_step = decode_ms / args.steps
    value = batch * args.steps / (decode_ms / 1e3)
    mean_context = prompt_len + offset - args.steps / 2
    step_bytes = weight_bytes + batch * mean_context * kv_bytes_per_token
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "of": peaks["source"]}
    del runner
    torch.cuda.empty_cache()

    # ---- end to end through the Python entry point ----------------------------------------------
    # sequences whose prompt is finished early decode while the others are still being prefilled
    prefill_steps = -(-batch * prompt_len // 4096) + batch
    new_tokens = args.warmup + args.steps + 4 + prefill_steps
    engine = Engine(model, EngineConfig(
        block_size=block, num_blocks=batch * (-(-(prompt_len + new_tokens) // block) + 1), max_batched_tokens=4096,
        max_running_seqs=batch, max_prompt_tokens=prompt_len, max_new_tokens=new_tokens,
        max_context_tokens=prompt_len + new_tokens, enable_prefix_cache=False, dtype="bfloat16", watermark=0.0))
    for i in range(batch):
        engine.submit(Request(f"e{i}", tuple(int(x) for x in prompts[i, :prompt_len]),
                              SamplingParams(max_new_tokens=new_tokens, ignore_eos=True)))
    while any(not s.is_decoding for s in engine.live_sequences()):
        engine.step()
    for _ in range(args.warmup):
        engine.step()
    torch.cuda.synchronize()
    h2d = d2h = 0
    started = time.perf_counter()
    produced = 0
    for _ in range(args.steps):
        out = engine.step()
        produced += len(out.tokens)
        h2d += engine.h2d_bytes_last_step
        d2h += engine.d2h_bytes_last_step
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - started
    clocks.stop()
    e2e_ms = 1e3 * elapsed / args.steps
    e2e = {"value": produced / elapsed, "unit": "tok/s", "h2d_bytes_per_step": h2d // args.steps,
           "d2h_bytes_per_step": d2h // args.steps, "ms_per_step": e2e_ms,
           "roofline_frac": step_bytes / (e2e_ms / 1e3) / 1e9 / peaks["hbm_gbs"]}

    return {
        "metric": METRIC.format(batch=batch, model=args.model, prompt=prompt_len), "value": value, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, random N(0, 0.02) weights", "impl": "ours",
        "config": {
            "model": f"{args.model}-shape", "n_layers": layers, "n_layers_full": full_layers, "d_model": config.d_model,
            "n_heads": config.n_heads, "n_kv_heads": config.n_kv_heads, "head_dim": config.head_dim,
            "d_ff": config.d_ff, "vocab_size": config.vocab_size, "global_batch": batch, "seq_len": prompt_len,
            "kv_block_size": block, "prefill_tokens": args.prefill_tokens, "parallelism": "single-gpu",
            "l2": "weights read each step (GBs) exceed L2; no flush", "peaks": peaks["source"],
            "value_timing": "K steps back to back, sampled ids fed to the next step on the device; e2e also reads them back",
        },
        "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline, "points": points,
        "clocks": clocks.summary(),
    }


def run_mixed(args, peaks) -> dict:
    """The fourth configuration of the baseline list as it is worded: Llama-2-13B layer sizes
    (40 heads without grouping), one step of 32 decoding sequences at 2,048 tokens of context
    beside one 512-token portion of a prompt (a step of 544 tokens), sampled on the device."""
    import numpy as np
    import torch

    from paged_kv_serving_b200.config.presets import PRESETS, preset
    from paged_kv_serving_b200.engine.batch import BatchEntry, ExecutionBatch
    from paged_kv_serving_b200.engine.runner import ModelRunner
    from paged_kv_serving_b200.engine.sequence import SamplingParams
    from paged_kv_serving_b200.models.decoder import DecoderModel
    from paged_kv_serving_b200.sampling.sampler import Sampler

    full_layers = PRESETS["llama-2-13b"]["n_layers"]
    layers = args.workload_layers or full_layers
    config = preset("llama-2-13b", n_layers=layers)
    model = DecoderModel.from_random(config, seed=0, dtype="bfloat16", device="cuda:0")
    rng = np.random.default_rng(2)
    seqs, context, portion, block, steps, warmup = 32, 2048, 512, 16, 12, 3
    pages = -(-(context + steps + warmup + 8) // block)
    runner = ModelRunner(model, num_blocks=(seqs + 1) * pages, block_size=block, max_running_seqs=64)
    sampler = Sampler(model.device)
    tables = [tuple(range(i * pages, (i + 1) * pages)) for i in range(seqs + 1)]
    tokens = rng.integers(0, config.vocab_size, size=(seqs + 1, context + steps + warmup + 8))
    for first in range(0, seqs, 2):           # fill the cache of the decoding sequences, 4,096 tokens a step
        runner.step(ExecutionBatch(tuple(
            BatchEntry(f"d{i}", tuple(int(t) for t in tokens[i, :context]), 0, (tables[i],), ()) for i in (first, first + 1))))
    runner.step(ExecutionBatch((BatchEntry("p", tuple(int(t) for t in tokens[seqs, :portion]), 0, (tables[seqs],), ()),)))
    chunk = tuple(int(t) for t in tokens[seqs, portion:2 * portion])
    greedy = SamplingParams(max_new_tokens=1)

    def one(k):
        entries = [BatchEntry(f"d{i}", (int(tokens[i, context + k]),), context + k, (tables[i],), (0,)) for i in range(seqs)]
        entries.append(BatchEntry("p", chunk, portion, (tables[seqs],), ()))     # the prompt's second 512 tokens
        result = runner.step(ExecutionBatch(tuple(entries)))
        sampler.sample_on_device(result.logits, [greedy] * seqs, [None] * seqs)

    for k in range(warmup):
        one(k)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for k in range(steps):
        one(warmup + k)
    stop.record()
    torch.cuda.synchronize()
    runner.check_status()
    ms = start.elapsed_time(stop) / steps
    kv_per_token = sum(2 * len(g.entries) * g.n_kv_heads * g.head_dim * 2 for g in runner.groups)
    cache_tokens = seqs * (context + warmup + steps / 2) + 2 * portion
    step_bytes = model.weight_bytes_read_per_step() + cache_tokens * kv_per_token
    step_tokens = seqs + portion
    flops = 2.0 * step_tokens * layers * (config.d_model * (config.q_width + 2 * config.kv_width)
                                          + config.q_width * config.d_model + 3 * config.d_model * config.d_ff)
    flops += 2.0 * seqs * config.d_model * config.vocab_size
    flops += 4.0 * layers * config.n_heads * config.head_dim * (seqs * context + portion * 1.5 * portion)
    out = {"model": "llama-2-13b-shape", "n_layers": layers, "n_layers_full": full_layers, "decode_seqs": seqs,
           "context": context, "prefill_portion": portion, "ms_per_step": ms, "tokens_per_s": step_tokens / (ms / 1e3),
           "decode_tokens_per_s": seqs / (ms / 1e3), "bound": "hbm (weights once + keys and values of the live requests)",
           "gbytes_per_step": step_bytes / 1e9, "hbm_frac": step_bytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"],
           "flops_frac": flops / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12)}
    del runner, model
    torch.cuda.empty_cache()
    return out


def run_serve(args) -> dict:
    """The fifth configuration of the baseline list as it is worded: Llama-3.2-1B layer sizes,
    256 requests with prompts of 128 to 4,096 tokens that share a 512-token prefix, 128 tokens
    each at temperature 0.7, through ``Engine`` with its scheduler and prefix cache."""
    import numpy as np
    import torch

    from paged_kv_serving_b200.config import EngineConfig
    from paged_kv_serving_b200.config.presets import PRESETS, preset
    from paged_kv_serving_b200.engine.engine import Engine
    from paged_kv_serving_b200.engine.sequence import Request, SamplingParams
    from paged_kv_serving_b200.models.decoder import DecoderModel

    full_layers = PRESETS["llama-3.2-1b"]["n_layers"]
    layers = args.workload_layers or full_layers
    config = preset("llama-3.2-1b", n_layers=layers)
    model = DecoderModel.from_random(config, seed=0, dtype="bfloat16", device="cuda:0")
    rng = np.random.default_rng(3)
    count, shared_len, new_tokens, block = args.serve_requests, 512, 128, 16
    shared = [int(t) for t in rng.integers(0, config.vocab_size, size=shared_len)]
    lengths = [int(n) for n in rng.integers(128, 4097, size=count)]
    prompts = [shared[:min(n, shared_len)] + [int(t) for t in rng.integers(0, config.vocab_size, size=max(0, n - shared_len))]
               for n in lengths]
    per_sequence = -(-(4096 + new_tokens) // block) + 1
    engine = Engine(model, EngineConfig(
        block_size=block, num_blocks=count * per_sequence, max_batched_tokens=8192, max_running_seqs=count,
        max_prompt_tokens=4096, max_new_tokens=new_tokens, max_context_tokens=4096 + new_tokens,
        enable_prefix_cache=True, dtype="bfloat16"))
    # warm-up outside the timed run, as a server has behind it when requests arrive: a full portion of
    # prompts and decode steps of every row-count bucket, so that the library's kernels for these shapes
    # are loaded; the graphs of the block-table widths to come are still captured inside the run
    warm = [Request(f"warm{i}", tuple(int(t) for t in rng.integers(0, config.vocab_size, size=1365)),
                    SamplingParams(max_new_tokens=3, temperature=0.7)) for i in range(12)]
    engine.generate(warm)
    for size in (24, 48, 100, count):         # decode steps of the 32-, 64-, 128- and 256-row buckets
        engine.generate([Request(f"warm{size}-{i}", tuple(int(t) for t in rng.integers(0, config.vocab_size, size=24)),
                                 SamplingParams(max_new_tokens=3, temperature=0.7)) for i in range(min(size, count))])
    engine.flush_prefix_cache()
    torch.cuda.synchronize()
    started = time.perf_counter()
    requests = [Request(f"u{i}", tuple(p), SamplingParams(max_new_tokens=new_tokens, temperature=0.7, seed=i, ignore_eos=True),
                        arrival_time=started) for i, p in enumerate(prompts)]
    outputs = engine.generate(requests)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - started
    produced = sum(o.output_tokens for o in outputs)
    stats = engine.scheduler.stats
    out = {"model": "llama-3.2-1b-shape", "n_layers": layers, "n_layers_full": full_layers, "requests": len(outputs),
           "prompt_tokens": sum(lengths), "output_tokens": produced, "seconds": elapsed,
           "output_tokens_per_s": produced / elapsed, "total_tokens_per_s": (produced + sum(lengths)) / elapsed,
           "prefix_hit_ratio": engine.prefix_cache.stats.hit_ratio,
           "cached_prompt_tokens": sum(o.cached_prompt_tokens for o in outputs),
           "preemptions": stats.preemptions, "steps": stats.iterations,
           "mean_ttft_s": sum(o.ttft for o in outputs) / max(1, len(outputs))}
    del engine, model
    torch.cuda.empty_cache()
    return out


REFERENCE_SRC = ROOT / "baseline" / "_ref"
REFERENCE_OBSTACLE = ("the reference is a NumPy engine for the CPU whose ModelConfig has neither grouped-query heads nor "
                      "an untied head, so the benchmark's 8B configuration cannot be expressed on its stock path")


def reference_workload_requests():
    """The reference's own published engine workload (bench/bench_baseline.py:189-214 of
    rouviere-german/paged-kv-serving): 24 requests of 48 random tokens, 12 new tokens each, on its
    default random model (4 layers, width 128, 4 heads, feed-forward 320, vocabulary 512)."""
    import numpy as np

    rng = np.random.default_rng(4)
    return [([int(v) for v in rng.integers(1, 256, 48)], 12, index) for index in range(24)]


def reference_context() -> dict | None:
    """Times the unmodified reference (copied to ``baseline/_ref``) through its own public API
    (``Engine.generate``) on its published workload. Context only: another model and another
    machine part (the host's CPU) than the headline, so no ratio is formed from it."""
    if not (REFERENCE_SRC / "paged_kv_serving").is_dir():
        return None
    sys.path.insert(0, str(REFERENCE_SRC))
    try:
        from paged_kv_serving.engine.config import EngineConfig, ModelConfig
        from paged_kv_serving.engine.engine import Engine
        from paged_kv_serving.engine.model import LanguageModel, random_weights
        from paged_kv_serving.engine.sequence import Request, SamplingParams
    except Exception as error:                                  # the copy does not import here
        return {"error": f"{type(error).__name__}: {error}"}
    config = ModelConfig(vocab_size=512, d_model=128, n_layers=4, n_heads=4, d_ff=320, max_seq_len=1024)
    model = LanguageModel(config, random_weights(config, 0))
    limits = EngineConfig(block_size=16, num_blocks=192, max_batched_tokens=128, max_running_seqs=12,
                          max_prompt_tokens=192, max_new_tokens=24, max_context_tokens=256)
    best = None
    for _ in range(3):
        requests = [Request(request_id=f"bench-{i}", prompt_token_ids=tuple(p), sampling=SamplingParams(max_new_tokens=n, seed=i))
                    for p, n, i in reference_workload_requests()]
        engine = Engine(model, limits)
        started = time.perf_counter()
        outputs = engine.generate(requests)
        elapsed = time.perf_counter() - started
        tokens = sum(o.output_tokens for o in outputs)
        best = elapsed if best is None else min(best, elapsed)
    return {"workload": "24 requests x 48 prompt tokens x 12 new tokens, 820k-parameter model, float32, CPU (NumPy)",
            "output_tokens": tokens, "seconds": best, "output_tokens_per_s": tokens / best}


def run_reference_workload() -> dict:
    """This engine on the reference's published workload (same model sizes, same requests, same
    limits), on the GPU in float32 through ``Engine.generate``: the number that stands beside
    ``reference_context`` of the reference arm."""
    import torch

    from paged_kv_serving_b200.config import EngineConfig
    from paged_kv_serving_b200.config.presets import preset
    from paged_kv_serving_b200.engine.engine import Engine
    from paged_kv_serving_b200.engine.sequence import Request, SamplingParams
    from paged_kv_serving_b200.models.decoder import DecoderModel

    model = DecoderModel.from_random(preset("reference-default"), seed=0, dtype="float32", device="cuda:0", std=0.08)
    limits = EngineConfig(block_size=16, num_blocks=192, max_batched_tokens=128, max_running_seqs=12,
                          max_prompt_tokens=192, max_new_tokens=24, max_context_tokens=256, dtype="float32")
    best = None
    for _ in range(3):
        requests = [Request(f"bench-{i}", tuple(p), SamplingParams(max_new_tokens=n, seed=i)) for p, n, i in reference_workload_requests()]
        engine = Engine(model, limits)
        torch.cuda.synchronize()
        started = time.perf_counter()
        outputs = engine.generate(requests)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - started
        tokens = sum(o.output_tokens for o in outputs)
        best = elapsed if best is None else min(best, elapsed)
    return {"workload": "24 requests x 48 prompt tokens x 12 new tokens, 820k-parameter model, float32, one B200",
            "output_tokens": tokens, "seconds": best, "output_tokens_per_s": tokens / best}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--model", default="llama-3-8b")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the preset (0: all)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--prompt-len", type=int, default=1024)
    parser.add_argument("--prefill-tokens", type=int, default=2048)
    parser.add_argument("--skip-points", action="store_true", help="leave out the batch-1 and batch-64 points")
    parser.add_argument("--skip-workloads", action="store_true",
                        help="leave out the mixed step (13B sizes), the 256-request run (1B sizes) and the reference's workload")
    parser.add_argument("--workloads", default="all", help="which of mixed,serve,reference to run beside the headline")
    parser.add_argument("--only-workloads", action="store_true", help="leave out the headline run (for profiling a workload)")
    parser.add_argument("--workload-layers", type=int, default=0, help="fewer layers for those workloads (0: all)")
    parser.add_argument("--serve-requests", type=int, default=256)
    args = parser.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_OBSTACLE, "context": reference_context()}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this engine is single-GPU by design, --gpus {args.gpus} is not run")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    wanted = set() if args.skip_workloads else {w for w in args.workloads.split(",") if w}
    if "all" in wanted:
        wanted = {"mixed", "serve", "reference"}
    line = run(args) if not args.only_workloads else {"impl": "ours", "n_gpus": 1}
    if "mixed" in wanted:
        line["mixed"] = run_mixed(args, load_peaks())
    if "serve" in wanted:
        line["serve"] = run_serve(args)
    if "reference" in wanted:
        line["reference_workload"] = run_reference_workload()
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
