"""Timing of single kernels at Llama-family layer sizes: ``python kernel_bench.py``.

Each case captures a few dozen launches in a CUDA graph (so that no host launch cost is timed),
rotates over 32 layers' worth of buffers (so that weights, keys and values come from DRAM as in
a real step) and reports microseconds per launch with the achieved bandwidth or arithmetic rate.
The sizes come from a preset of ``config/presets.py``; nothing here is used by the engine.

    python kernel_bench.py [gemm] [decode-gemm] [prefill-attention] [decode-attention] [elementwise]
"""

from __future__ import annotations

import argparse
import math
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.config.presets import preset

LAYERS = 32


def timed(fn, launches: int = 32, replays: int = 4) -> float:
    """Microseconds per call of ``fn(i)``, measured on graph replays."""
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(launches):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(replays):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / (replays * launches) * 1000.0


def bench_gemm(config, rows: int) -> None:
    status = ops.status_word("cuda")
    d, ff = config.d_model, config.d_ff
    qkv = (config.n_heads + 2 * config.n_kv_heads) * config.head_dim
    cases = [("qkv", qkv, d, "bf16"), ("output", d, config.n_heads * config.head_dim, "bf16"),
             ("gate/up + SiLU", 2 * (-(-ff // 128) * 128), d, "silu_mul"), ("down", d, ff, "bf16")]
    for name, n, k, epilogue in cases:
        a = torch.randn(rows, k, device="cuda").to(torch.bfloat16)
        w = [torch.randn(n, k, device="cuda").to(torch.bfloat16) for _ in range(3)]
        ours = timed(lambda i: ops.gemm_tcgen05(a, w[i % 3], status, epilogue, n_out=ff), launches=8)
        single = timed(lambda i: ops.gemm_tcgen05(a, w[i % 3], status, epilogue, n_out=ff, pairs=False), launches=8)
        lib = timed(lambda i: torch.mm(a, w[i % 3].t()), launches=8)
        flops = 2.0 * rows * n * k
        print(f"gemm {name:15s} [{rows} x {k}] x [{n} x {k}]^T: tcgen05 pairs {ours:7.1f} us {flops / ours / 1e6:6.0f} TFLOP/s"
              f" | single {single:7.1f} us {flops / single / 1e6:6.0f} TFLOP/s"
              f" | cuBLAS (no epilogue) {lib:7.1f} us {flops / lib / 1e6:6.0f} TFLOP/s")
    assert int(status.item()) == 0


def bench_decode_gemm(config) -> None:
    """The four products of a layer at decode sizes, launched back to back as in a step, against cuBLAS."""
    d, ff = config.d_model, config.d_ff
    qkv = (config.n_heads + 2 * config.n_kv_heads) * config.head_dim
    ff_rows = 2 * (-(-ff // 128) * 128)
    copies = 3
    weights = [[torch.randn(n, k, device="cuda").to(torch.bfloat16) for _ in range(copies)]
               for n, k in ((qkv, d), (d, config.n_heads * config.head_dim), (ff_rows, d), (d, ff))]
    layer_bytes = 2.0 * sum(w[0].numel() for w in weights)
    for rows in (1, 8, 16, 32):
        x_d = torch.randn(rows, d, device="cuda").to(torch.bfloat16)
        x_ff = torch.randn(rows, ff, device="cuda").to(torch.bfloat16)

        def ours(i, chained=True):
            ops.gemm_small_m(x_d, weights[0][i % copies], chained=chained)
            ops.gemm_small_m(x_d, weights[1][i % copies], chained=chained)
            if rows <= 32:
                ops.gemm_small_m(x_d, weights[2][i % copies], "silu_mul", n_out=ff, chained=chained)
            else:
                ops.silu_mul(torch.mm(x_d, weights[2][i % copies].t()), 60.0, ff=ff, interleave=128)
            ops.gemm_small_m(x_ff, weights[3][i % copies], chained=chained)

        def lib(i):
            torch.mm(x_d, weights[0][i % copies].t())
            torch.mm(x_d, weights[1][i % copies].t())
            ops.silu_mul(torch.mm(x_d, weights[2][i % copies].t()), 60.0, ff=ff, interleave=128)
            torch.mm(x_ff, weights[3][i % copies].t())

        t_chain = timed(ours, launches=12)
        t_plain = timed(lambda i: ours(i, False), launches=12)
        t_lib = timed(lib, launches=12)
        print(f"decode products of one layer, {rows:2d} rows ({layer_bytes / 1e6:.0f} MB of weights): "
              f"streaming kernel {t_chain:6.1f} us {layer_bytes / t_chain / 1e6:5.2f} TB/s"
              f" | not chained {t_plain:6.1f} us | cuBLAS + activation kernel {t_lib:6.1f} us {layer_bytes / t_lib / 1e6:5.2f} TB/s")


def _cache(config, batch: int, context: int, page: int):
    kv, hd = config.n_kv_heads, config.head_dim
    pages_per = -(-context // page)
    pages = batch * pages_per
    # as many layers' pools as fit in 16 GiB each for keys and values (at least two, so that a
    # replay does not find its keys in L2): callers rotate over k.shape[0]
    layers = int(max(2, min(LAYERS, (16 << 30) // max(1, pages * kv * page * hd * 2))))
    k = torch.randn((layers, pages, kv, page, hd), device="cuda", dtype=torch.bfloat16)
    v = torch.randn((layers, pages, kv, page, hd), device="cuda", dtype=torch.bfloat16)
    table = torch.tensor([[j * batch + i for j in range(pages_per)] for i in range(batch)], dtype=torch.int32, device="cuda")
    return k, v, table


def bench_prefill_attention(config, page: int) -> None:
    h, kv, hd = config.n_heads, config.n_kv_heads, config.head_dim
    status = ops.status_word("cuda")
    for batch, context, queries in ((1, 2048, 2048), (4, 1024, 1024), (1, 8192, 8192), (2, 4096, 512)):
        k, v, table = _cache(config, batch, context, page)
        tokens = batch * queries
        qkv = torch.randn((tokens, (h + 2 * kv) * hd), device="cuda", dtype=torch.bfloat16)
        out = torch.empty((tokens, h * hd), device="cuda", dtype=torch.bfloat16)
        starts = torch.arange(0, tokens + 1, queries, dtype=torch.int32, device="cuda")
        first = torch.full((batch,), context - queries, dtype=torch.int32, device="cuda")
        flops = 4.0 * batch * h * hd * (queries * (queries + 1) / 2 + queries * (context - queries))
        for name, rows in (("tcgen05", ops.attention_tcgen05_rows()), ("mma.sync", ops.attention_bf16_rows()[0])):
            blocks = -(-queries // rows)
            seq = torch.tensor([s for q in reversed(range(blocks)) for s in range(batch)], dtype=torch.int32, device="cuda")
            q0 = torch.tensor([q * rows for q in reversed(range(blocks)) for s in range(batch)], dtype=torch.int32, device="cuda")
            if name == "tcgen05":
                if not ops.attention_tcgen05_supports(hd, page, qkv.shape[1]):
                    continue
                fn = lambda i: ops.attention_prefill_tcgen05(qkv, out, k[i % k.shape[0]], v[i % k.shape[0]], table, starts, first,
                                                             seq, q0, h, kv, hd, page, 0, 1 / math.sqrt(hd), status)
            else:
                fn = lambda i: ops.attention_prefill_bf16(qkv, out, k[i % k.shape[0]], v[i % k.shape[0]], table, starts, first,
                                                          seq, q0, h, kv, hd, page, 0, 1 / math.sqrt(hd))
            us = timed(fn, launches=8)
            print(f"prefill attention {name:8s} {batch} x {queries} queries over {context} keys: {us:8.1f} us "
                  f"{flops / us / 1e6:6.0f} TFLOP/s")
    assert int(status.item()) == 0


def bench_decode_attention(config, page: int) -> None:
    h, kv, hd = config.n_heads, config.n_kv_heads, config.head_dim
    status = ops.status_word("cuda")
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for batch, context in ((1, 1024), (8, 1024), (64, 1024), (8, 4096), (64, 4096)):
        k, v, table = _cache(config, batch, context, page)
        qkv = torch.randn((batch, (h + 2 * kv) * hd), device="cuda", dtype=torch.bfloat16)
        out = torch.empty((batch, h * hd), device="cuda", dtype=torch.bfloat16)
        starts = torch.arange(0, batch + 1, dtype=torch.int32, device="cuda")
        first = torch.full((batch,), context - 1, dtype=torch.int32, device="cuda")
        work = torch.arange(batch, dtype=torch.int32, device="cuda")
        nbytes = 2.0 * batch * context * kv * hd * 2
        if ops.attention_decode_tma_supports(hd, page, qkv.shape[1]):
            resident = min(2, ops.attention_decode_tma_blocks_per_sm(hd, False)) * sms
            splits = max(1, min(8, -(-context // 64), resident // (batch * kv)))
            pushed = ops.attention_decode_tma_pushed_splits(hd, h // kv)
            if splits > 4 and 4 <= pushed < splits:
                splits = pushed
            us = timed(lambda i: ops.attention_decode_tma(qkv, out, k[i % k.shape[0]], v[i % k.shape[0]], table, starts, first, work,
                                                          1, h, kv, hd, page, 0, 1 / math.sqrt(hd), splits, status, False))
            print(f"decode attention TMA      batch {batch:3d} context {context}: {splits} splits {us:7.1f} us {nbytes / us / 1e6:5.2f} TB/s")
        if ops.attention_decode_flat_supports(hd, page, qkv.shape[1]):
            tiles = -(-context // 64)
            units = torch.arange(0, batch + 1, dtype=torch.int32, device="cuda") * tiles
            blocks = min(min(2, ops.attention_decode_flat_blocks_per_sm(hd)) * sms, batch * kv * tiles)
            us = timed(lambda i: ops.attention_decode_flat(qkv, out, k[i % k.shape[0]], v[i % k.shape[0]], table, starts, first, work,
                                                           units, 1, h, kv, hd, page, 0, 1 / math.sqrt(hd), blocks, status))
            print(f"decode attention even shares batch {batch:3d} context {context}: {blocks} blocks {us:7.1f} us {nbytes / us / 1e6:5.2f} TB/s")
        resident = ops.attention_decode_blocks_per_sm(hd) * sms
        splits = max(1, min(8, -(-context // 64), resident // (batch * kv)))
        us = timed(lambda i: ops.attention_decode_bf16(qkv, out, k[i % k.shape[0]], v[i % k.shape[0]], table, starts, first, work,
                                                       1, h, kv, hd, page, 0, 1 / math.sqrt(hd), splits, None))
        print(f"decode attention cp.async batch {batch:3d} context {context}: {splits} splits {us:7.1f} us {nbytes / us / 1e6:5.2f} TB/s")
    assert int(status.item()) == 0


def bench_elementwise(config, page: int) -> None:
    d, ff = config.d_model, config.d_ff
    h, kv, hd = config.n_heads, config.n_kv_heads, config.head_dim
    for tokens in (8, 64, 2048):
        hidden = torch.randn((LAYERS, tokens, d), device="cuda")
        delta = torch.randn((LAYERS, tokens, d), device="cuda", dtype=torch.bfloat16)
        weight = torch.ones(d, device="cuda")
        us = timed(lambda i: ops.add_rmsnorm(hidden[i % LAYERS], delta[i % LAYERS], weight, 1e-5, torch.bfloat16))
        print(f"add_rmsnorm   {tokens:5d} tokens: {us:6.1f} us {tokens * d * 12 / us / 1e6:5.2f} TB/s")
        gate_up = torch.randn((4, tokens, 2 * ff), device="cuda", dtype=torch.bfloat16)
        us = timed(lambda i: ops.silu_mul(gate_up[i % 4], 60.0))
        print(f"silu_mul      {tokens:5d} tokens: {us:6.1f} us {tokens * ff * 6 / us / 1e6:5.2f} TB/s")
        qkv = torch.randn((4, tokens, (h + 2 * kv) * hd), device="cuda", dtype=torch.bfloat16)
        positions = torch.arange(tokens, dtype=torch.int32, device="cuda")
        cos = torch.randn((config.max_seq_len, hd // 2), device="cuda")
        sin = torch.randn((config.max_seq_len, hd // 2), device="cuda")
        pages = max(64, tokens // page + 1)
        k_pool = torch.zeros((pages, kv, page, hd), device="cuda", dtype=torch.bfloat16)
        v_pool = torch.zeros_like(k_pool)
        us = timed(lambda i: ops.rope_kv_store(qkv[i % 4], positions, cos, sin, k_pool, v_pool, positions, h, kv, hd, page))
        print(f"rope_kv_store {tokens:5d} tokens: {us:6.1f} us {tokens * (h + 2 * kv) * hd * 4 / us / 1e6:5.2f} TB/s")


def main() -> int:
    cases = {"gemm": None, "decode-gemm": None, "prefill-attention": bench_prefill_attention, "decode-attention": bench_decode_attention,
             "elementwise": bench_elementwise}
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("cases", nargs="*", choices=[*cases, []], help="which kernels to time (default: all)")
    parser.add_argument("--preset", default="llama-3-8b")
    parser.add_argument("--rows", type=int, default=2048, help="activation rows of the matrix products")
    parser.add_argument("--page-size", type=int, default=16)
    args = parser.parse_args()
    config = preset(args.preset)
    for name in args.cases or list(cases):
        if name == "gemm":
            bench_gemm(config, args.rows)
        elif name == "decode-gemm":
            bench_decode_gemm(config)
        else:
            cases[name](config, args.page_size)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
