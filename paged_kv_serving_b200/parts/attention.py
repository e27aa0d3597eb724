"""The attention mixer: fused QKV projection, position encoding, paged cache, output projection."""

from __future__ import annotations

import contextlib
import math

import numpy as np
import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import arena, gemm
from paged_kv_serving_b200.parts.base import CacheBinding, PagedKVRequest, ParamSpec, Part, StepContext
from paged_kv_serving_b200.parts.position import PositionEncoding

__all__ = ["PagedAttention"]

_SM_COUNT: dict[str, int] = {}


def _sm_count(device: torch.device) -> int:
    key = str(device)
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT[key]


_SIDE_STREAM: dict[str, "torch.cuda.Stream"] = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    """A second stream of the device, of the highest priority: its few blocks find places first."""
    key = str(device)
    if key not in _SIDE_STREAM:
        _SIDE_STREAM[key] = torch.cuda.Stream(device=device, priority=-1)
    return _SIDE_STREAM[key]


@contextlib.contextmanager
def _second_stream(device: torch.device):
    """What is launched inside runs on the device's second stream, after everything the current
    stream holds so far; the caller lets the current stream wait for it when it needs the result."""
    main = torch.cuda.current_stream(device)
    side = _side_stream(device)
    side.wait_stream(main)
    torch.cuda.set_stream(side)
    try:
        yield side
    finally:
        torch.cuda.set_stream(main)


@register_part("mixer", "attention")
class PagedAttention(Part):
    """Causal grouped-query attention over the paged cache.

    ``qkv_proj`` is ``(width, (H + 2*KV) * hd)`` with columns ``[Q | K | V]``, head-major inside
    each, used as ``x @ W`` (reference: src/paged_kv_serving/engine/model.py:249-253, widened for
    fewer key/value heads); query head ``h`` reads key/value head ``h // (H // KV)``. Scores are
    ``q.k * scale`` with ``scale = 1/sqrt(hd)`` unless given
    (src/paged_kv_serving/engine/model.py:239-241), masked by absolute position
    (src/paged_kv_serving/engine/attention.py:102-104), optionally within a window of positions.
    Keys are cached after position encoding (src/paged_kv_serving/engine/runner.py:194-196).
    ``out_proj`` is ``(H * hd, width)``.
    """

    @property
    def graph_safe(self) -> bool:
        return self.position.graph_safe


    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: PositionEncoding, scale: float | None = None, window: int | None = None) -> None:
        if n_heads % n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if head_dim % 2 or head_dim > 256:
            raise ValueError(f"attention kernels take an even head_dim up to 256, not {head_dim}")
        if window is not None and window < 1:
            raise ValueError("window must be >= 1 or None")
        self.width = int(width)
        self.n_heads = int(n_heads)
        self.n_kv_heads = int(n_kv_heads)
        self.head_dim = int(head_dim)
        self.position = position
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.window = window
        self.qkv_proj: torch.Tensor | None = None
        self.out_proj: torch.Tensor | None = None
        self._fast_ok: bool | None = None
        self._tcgen05_ok: dict = {}

    @property
    def group_size(self) -> int:
        return self.n_heads // self.n_kv_heads

    def param_specs(self) -> dict[str, ParamSpec]:
        qkv_width = (self.n_heads + 2 * self.n_kv_heads) * self.head_dim
        return {
            "qkv_proj": ParamSpec((self.width, qkv_width)),
            "out_proj": ParamSpec((self.n_heads * self.head_dim, self.width)),
        }

    def load(self, params: dict[str, torch.Tensor]) -> None:
        # held as [out, in]: the inner size contiguous, as the matrix-product kernels read it
        self.qkv_proj = params["qkv_proj"].t().contiguous()
        self.out_proj = params["out_proj"].t().contiguous()

    def cache_request(self) -> PagedKVRequest:
        return PagedKVRequest(self.n_kv_heads, self.head_dim, self.window)

    # --- per step ------------------------------------------------------------------------

    def _work_names(self) -> tuple[str, str]:
        return (f"attention/work_seq/g{self.group_size}", f"attention/work_row0/g{self.group_size}")

    def _fast(self, ctx: StepContext) -> bool:
        """Whether the tensor-core bfloat16 kernels serve this mixer in this step."""
        if ctx.dtype != torch.bfloat16:
            return False
        if self._fast_ok is None:
            qkv_width = (self.n_heads + 2 * self.n_kv_heads) * self.head_dim
            self._fast_ok = ops.attention_bf16_supports(self.head_dim, qkv_width)
        return self._fast_ok

    #: Set to False to keep runs of queries on the mma.sync kernel (tests compare the two).
    USE_TCGEN05 = True
    #: When decode entries go to the kernel that cuts the step's keys into even shares
    #: (``ops.attention_decode_flat``) rather than to one block per (entry, head, split):
    #: "auto" where measurement says so, "always" (where it takes the sizes) or "never".
    #: The even shares cost about 4 us more per launch (parts meet in global memory, all blocks
    #: start and end together), so they pay only when the other kernel's last round of blocks
    #: would be nearly empty: 320 (entry, head) pairs on 296 places, 34 against 37 us at 1,100
    #: keys and 83 against 112 us at 4,096; not at 512 pairs on 296 places (59 against 52 us).
    FLAT_DECODE = "auto"
    FLAT_DECODE_IDLE_SHARE = 0.4
    #: The attention kernels need nearly all of an SM's memory as shared memory; the decode
    #: products stream their weights through L1. An SM changes the division only when it is idle:
    #: blocks of a product that arrive while attention blocks are still resident keep the small
    #: L1, run at half speed, and hand the division on to the products chained after them (the
    #: gate/up product then took 92 us instead of 46, at random). So the output projection starts
    #: only after the attention kernel has left the SMs.
    chains_last_linear = False
    #: Whether, in a step that holds portions of prompts beside decode entries, the two attention
    #: kernels run side by side on two streams (measured on the mixed step of a 13-billion-parameter
    #: shape: 33 us a layer of portion attention disappear behind 209 us of decode attention).
    OVERLAP_MIXED = True

    def _tcgen05(self, page_size: int) -> bool:
        """Whether runs of queries go to the tcgen05 kernel (head 64 or 128, pages of 8k keys)."""
        if not self.USE_TCGEN05:
            return False
        key = page_size
        if key not in self._tcgen05_ok:
            qkv_width = (self.n_heads + 2 * self.n_kv_heads) * self.head_dim
            self._tcgen05_ok[key] = ops.attention_tcgen05_supports(self.head_dim, page_size, qkv_width)
        return self._tcgen05_ok[key]

    def _decode_tma(self, page_size: int) -> bool:
        """Whether short entries go to the TMA-fed decode kernel."""
        key = ("decode", page_size)
        if key not in self._tcgen05_ok:
            qkv_width = (self.n_heads + 2 * self.n_kv_heads) * self.head_dim
            self._tcgen05_ok[key] = self.USE_TCGEN05 and ops.attention_decode_tma_supports(self.head_dim, page_size, qkv_width)
        return self._tcgen05_ok[key]

    def _flat_pays(self, entries: int, device: torch.device) -> bool:
        if self.FLAT_DECODE != "auto":
            return self.FLAT_DECODE == "always"
        places = 2 * _sm_count(device)
        pairs = entries * self.n_kv_heads
        rounds = pairs / places
        return pairs > places and 1.0 - rounds / math.ceil(rounds) > self.FLAT_DECODE_IDLE_SHARE

    def _fast_key(self, page_size: int) -> str:
        """Name of this mixer's plan among a step's plans. Everything the plan depends on is part
        of it (head counts and size decide splits and grids, the window the tiles of an entry,
        the page size which kernels serve), so that layers share a plan only when it is the same."""
        return (f"attention/fast/h{self.n_heads}k{self.n_kv_heads}d{self.head_dim}w{self.window or 0}p{page_size}/"
                f"{'t' if self._tcgen05(page_size) else 'm'}")

    def _plan_fast(self, ctx: StepContext, page_size: int) -> None:
        """Work lists of the bfloat16 kernels: entries of at most 16 rows per key/value head go
        to the split-KV decode kernel, longer ones are cut into blocks of queries (128 for the
        tcgen05 kernel, 64 for the mma.sync one) for the prefill kernel, heaviest blocks first."""
        key = self._fast_key(page_size)
        if key in ctx.scratch:
            return
        block_rows, decode_rows = ops.attention_bf16_rows()
        if self._tcgen05(page_size):
            block_rows = ops.attention_tcgen05_rows()
        lens = np.asarray(ctx.seq_lens, dtype=np.int64)
        first = np.asarray(ctx.first_positions, dtype=np.int64)
        small = lens * self.group_size <= decode_rows
        decode_entries = np.nonzero(small)[0]
        large = np.nonzero(~small)[0]
        blocks = (lens[large] + block_rows - 1) // block_rows
        work_seq = np.repeat(large, blocks)
        starts = np.cumsum(blocks) - blocks
        work_q0 = (np.arange(int(blocks.sum()), dtype=np.int64) - np.repeat(starts, blocks)) * block_rows
        cost = first[work_seq] + work_q0
        order = np.argsort(-cost, kind="stable")
        num_splits, deep_ring = 1, True
        if len(decode_entries):
            longest = int((first[decode_entries] + lens[decode_entries]).max())
            if ctx.planning_context_len is not None:
                longest = ctx.planning_context_len
            # as many splits of the key range as still run in one wave of blocks, at most 8 (the
            # splits of an entry form one thread-block cluster) and at most one per 64-key tile
            tiles = max(1, -(-longest // 64))
            blocks_per_split = len(decode_entries) * self.n_kv_heads
            deep_ring = True
            if self._decode_tma(page_size):
                # the three-stage ring (two blocks per SM) measured at least as fast as the six-stage
                # one (one block per SM) at every batch size and context length tried
                deep_ring = False
                # (more than two blocks of a cluster per SM measured slower than fewer splits)
                per_sm = min(2, ops.attention_decode_tma_blocks_per_sm(self.head_dim, deep_ring))
            else:
                per_sm = ops.attention_decode_blocks_per_sm(self.head_dim)
            resident = per_sm * _sm_count(ctx.device)
            num_splits = int(max(1, min(tiles, 8, resident // blocks_per_split)))
            if self._decode_tma(page_size) and num_splits > 4:
                # up to a number of splits the kernel merges them the fast way; a few splits less
                # cost less than the slow merge
                rows = int(lens[decode_entries].max()) * self.group_size
                pushed = ops.attention_decode_tma_pushed_splits(self.head_dim, rows)
                if 4 <= pushed < num_splits:
                    num_splits = pushed
        names = {k: f"{key}/{k}" for k in ("prefill_seq", "prefill_q0", "decode_seq", "decode_units")}
        ctx.arena.add(names["prefill_seq"], work_seq[order] if len(order) else [0])
        ctx.arena.add(names["prefill_q0"], work_q0[order] if len(order) else [0])
        ctx.arena.add(names["decode_seq"], decode_entries if len(decode_entries) else [0])
        flat_blocks = 0
        if len(decode_entries) and self._decode_tma(page_size) and self._flat_pays(len(decode_entries), ctx.device):
            # the even-shares kernel: 64-key tiles of every entry, as many blocks as the GPU holds
            # at once (a captured graph keeps its grid: sized for the planning length)
            key_hi = first[decode_entries] + lens[decode_entries]
            key_lo = np.maximum(0, first[decode_entries] - self.window + 1) if self.window else np.zeros_like(key_hi)
            tiles = (key_hi - 1) // 64 - key_lo // 64 + 1
            ctx.arena.add(names["decode_units"], np.concatenate([[0], np.cumsum(tiles)]))
            planned = int(tiles.sum())
            if ctx.planning_context_len is not None:
                planned = len(decode_entries) * -(-ctx.planning_context_len // 64)
            per_sm = min(2, ops.attention_decode_flat_blocks_per_sm(self.head_dim))
            flat_blocks = int(max(1, min(per_sm * _sm_count(ctx.device), planned * self.n_kv_heads)))
        else:
            ctx.arena.add(names["decode_units"], [0])
        ctx.scratch[key] = {
            "names": names, "n_prefill": int(len(order)), "n_decode": int(len(decode_entries)),
            "max_small_tokens": int(lens[decode_entries].max()) if len(decode_entries) else 0,
            "num_splits": num_splits, "deep_ring": deep_ring, "flat_blocks": flat_blocks,
        }

    def plan_step(self, ctx: StepContext, binding: CacheBinding | None) -> None:
        if self._fast(ctx):
            self._plan_fast(ctx, ctx.groups[binding.group].page_size)
            return
        seq_name, row_name = self._work_names()
        if seq_name in ctx.arena:
            return
        rows_per_block = ops.attention_rows_per_block()
        rows = np.asarray(ctx.seq_lens, dtype=np.int64) * self.group_size
        blocks = (rows + rows_per_block - 1) // rows_per_block
        work_seq = np.repeat(np.arange(len(rows), dtype=np.int64), blocks)
        starts = np.cumsum(blocks) - blocks
        work_row0 = (np.arange(int(blocks.sum()), dtype=np.int64) - np.repeat(starts, blocks)) * rows_per_block
        ctx.arena.add(seq_name, work_seq)
        ctx.arena.add(row_name, work_row0)

    fuses_last_linear = True
    accepts_pending_norm = True

    def forward(self, x: torch.Tensor, ctx: StepContext, binding: CacheBinding, finish=None) -> torch.Tensor:
        project_out = finish if finish is not None else (lambda a, w: gemm.linear(a, w, chain=self.chains_last_linear))
        group = ctx.groups[binding.group]
        k_pool = group.k_pool[binding.index]
        v_pool = group.v_pool[binding.index]
        positions = ctx.ints(ctx.POSITIONS)
        slots = ctx.ints(group.slots_name) if binding.write else None
        tables = self.position.fused_tables(ctx.device)
        if tables is None:
            qkv = gemm.linear(x, self.qkv_proj, chain=True)
            self.position.apply_qk(qkv, positions, self.n_heads, self.n_kv_heads, self.head_dim)
            ops.rope_kv_store(qkv, positions, None, None, k_pool, v_pool, slots,
                              self.n_heads, self.n_kv_heads, self.head_dim, group.page_size)
        else:
            # projection, rotation and cache write: one kernel for the few rows of a decode step
            qkv = gemm.linear_rope_kv_store(x, self.qkv_proj, positions, tables[0], tables[1], k_pool, v_pool, slots,
                                            self.n_heads, self.n_kv_heads, self.head_dim, group.page_size,
                                            chain=True)
        if self._fast(ctx):
            attended = self._attend_fast(qkv, ctx, group, k_pool, v_pool)
            return project_out(attended, self.out_proj)
        seq_name, row_name = self._work_names()
        attended = ops.paged_attention_generic(
            qkv, k_pool, v_pool, ctx.ints(group.table_name), ctx.ints(ctx.SEQ_STARTS), ctx.ints(ctx.FIRST_POS),
            ctx.ints(seq_name), ctx.ints(row_name), self.n_heads, self.n_kv_heads, self.head_dim,
            group.page_size, self.window or 0, self.scale)
        return project_out(attended, self.out_proj)

    def _attend_fast(self, qkv, ctx: StepContext, group, k_pool, v_pool) -> torch.Tensor:
        plan = ctx.scratch[self._fast_key(group.page_size)]
        names = plan["names"]
        out = arena.empty((qkv.shape[0], self.n_heads * self.head_dim), qkv.dtype, qkv.device)
        joined = False
        table, starts, first = ctx.ints(group.table_name), ctx.ints(ctx.SEQ_STARTS), ctx.ints(ctx.FIRST_POS)
        if plan["n_prefill"] and self._tcgen05(group.page_size):
            # In a mixed step the portions' kernel (few blocks, bound by its own latencies) and the
            # decode kernel (bound by memory) work on different entries and write different rows:
            # the first runs on a second stream of higher priority beside the other
            joined = bool(self.OVERLAP_MIXED and plan["n_decode"] and self._decode_tma(group.page_size)
                          and not torch.cuda.is_current_stream_capturing())
            with _second_stream(qkv.device) if joined else contextlib.nullcontext():
                ops.attention_prefill_tcgen05(qkv, out, k_pool, v_pool, table, starts, first,
                                              ctx.ints(names["prefill_seq"]), ctx.ints(names["prefill_q0"]), self.n_heads,
                                              self.n_kv_heads, self.head_dim, group.page_size, self.window or 0,
                                              self.scale, ops.status_word(qkv.device))
        elif plan["n_prefill"]:
            ops.attention_prefill_bf16(qkv, out, k_pool, v_pool, table, starts, first, ctx.ints(names["prefill_seq"]),
                                       ctx.ints(names["prefill_q0"]), self.n_heads, self.n_kv_heads, self.head_dim,
                                       group.page_size, self.window or 0, self.scale)
        if plan["n_decode"] and plan["flat_blocks"]:
            ops.attention_decode_flat(qkv, out, k_pool, v_pool, table, starts, first, ctx.ints(names["decode_seq"]),
                                      ctx.ints(names["decode_units"]), plan["max_small_tokens"], self.n_heads,
                                      self.n_kv_heads, self.head_dim, group.page_size, self.window or 0, self.scale,
                                      plan["flat_blocks"], ops.status_word(qkv.device))
        elif plan["n_decode"] and self._decode_tma(group.page_size):
            ops.attention_decode_tma(qkv, out, k_pool, v_pool, table, starts, first, ctx.ints(names["decode_seq"]),
                                     plan["max_small_tokens"], self.n_heads, self.n_kv_heads, self.head_dim,
                                     group.page_size, self.window or 0, self.scale, plan["num_splits"],
                                     ops.status_word(qkv.device), plan["deep_ring"])
        elif plan["n_decode"]:
            splits = plan["num_splits"]
            scratch = None
            if splits > 8:
                size = qkv.shape[0] * self.n_heads * splits * (self.head_dim + 2)
                scratch = ctx.scratch.get("attention/split_scratch")
                if scratch is None or scratch.numel() < size:
                    scratch = torch.empty((size,), dtype=torch.float32, device=qkv.device)
                    ctx.scratch["attention/split_scratch"] = scratch
            ops.attention_decode_bf16(qkv, out, k_pool, v_pool, table, starts, first, ctx.ints(names["decode_seq"]),
                                      plan["max_small_tokens"], self.n_heads, self.n_kv_heads, self.head_dim,
                                      group.page_size, self.window or 0, self.scale, splits, scratch)
        if joined:
            torch.cuda.current_stream(qkv.device).wait_stream(_side_stream(qkv.device))
        return out
