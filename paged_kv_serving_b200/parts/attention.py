"""The attention mixer: fused QKV projection, position encoding, paged cache, output projection."""

from __future__ import annotations

import math

import numpy as np
import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.config.registry import register_part
from paged_kv_serving_b200.ops import gemm
from paged_kv_serving_b200.parts.base import CacheBinding, PagedKVRequest, ParamSpec, Part, StepContext
from paged_kv_serving_b200.parts.position import PositionEncoding

__all__ = ["PagedAttention"]


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

    @property
    def group_size(self) -> int:
        return self.n_heads // self.n_kv_heads

    def param_specs(self) -> dict[str, ParamSpec]:
        qkv_width = (self.n_heads + 2 * self.n_kv_heads) * self.head_dim
        return {
            "qkv_proj": ParamSpec((self.width, qkv_width)),
            "out_proj": ParamSpec((self.n_heads * self.head_dim, self.width)),
        }

    def cache_request(self) -> PagedKVRequest:
        return PagedKVRequest(self.n_kv_heads, self.head_dim, self.window)

    # --- per step ------------------------------------------------------------------------

    def _work_names(self) -> tuple[str, str]:
        return (f"attention/work_seq/g{self.group_size}", f"attention/work_row0/g{self.group_size}")

    def plan_step(self, ctx: StepContext, binding: CacheBinding | None) -> None:
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

    def forward(self, x: torch.Tensor, ctx: StepContext, binding: CacheBinding) -> torch.Tensor:
        group = ctx.groups[binding.group]
        k_pool = group.k_pool[binding.index]
        v_pool = group.v_pool[binding.index]
        qkv = gemm.matmul(x, self.qkv_proj)
        positions = ctx.ints(ctx.POSITIONS)
        tables = self.position.fused_tables(ctx.device)
        if tables is None:
            self.position.apply_qk(qkv, positions, self.n_heads, self.n_kv_heads, self.head_dim)
            cos = sin = None
        else:
            cos, sin = tables
        slots = ctx.ints(group.slots_name) if binding.write else None
        ops.rope_kv_store(qkv, positions, cos, sin, k_pool, v_pool, slots,
                          self.n_heads, self.n_kv_heads, self.head_dim, group.page_size)
        seq_name, row_name = self._work_names()
        attended = ops.paged_attention_generic(
            qkv, k_pool, v_pool, ctx.ints(group.table_name), ctx.ints(ctx.SEQ_STARTS), ctx.ints(ctx.FIRST_POS),
            ctx.ints(seq_name), ctx.ints(row_name), self.n_heads, self.n_kv_heads, self.head_dim,
            group.page_size, self.window or 0, self.scale)
        return gemm.matmul(attended, self.out_proj)
