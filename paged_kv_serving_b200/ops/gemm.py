"""Matrix products of the product path.

Weights are held as ``[out, in]`` with the inner size contiguous. In bfloat16, products with at
least ``TCGEN05_MIN_ROWS`` rows of activations (prompt portions) can run on the hand-written
tcgen05/TMA kernels of ``csrc/gemm_tcgen05.cu``: the gate/up product of the feed-forward always
does, with its SiLU-times-up step fused into the epilogue, the plain products when
``PLAIN_PRODUCT_KERNEL`` says so. The up to ``SMALL_M_ROWS`` rows of a decode step go to the
weight-streaming kernel of ``csrc/gemm_small_m.cu``; a tcgen05 twin of it for up to 128 rows
(``csrc/gemm_stream.cu``) stands behind the switch ``STREAM_ROWS``. Everything else, and the float32 path, goes to cuBLAS
through ``torch.mm``, as the reference's engine hands its products to a library
(src/paged_kv_serving/engine/model.py:249,258-259,264). Reduced-precision modes are switched
off: float32 products use true float32 multiply-adds (no TF32), bfloat16 products accumulate in
float32 without reduced-precision reductions.
"""

from __future__ import annotations

import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.ops import arena

__all__ = ["PendingNorm", "SILU_TCGEN05_MIN_ROWS", "TCGEN05_MIN_ROWS", "as_tensor", "linear", "linear_add_norm", "linear_rope_kv_store",
           "linear_silu_mul", "matmul"]

torch.backends.cuda.matmul.allow_tf32 = False
torch.backends.cudnn.allow_tf32 = False
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False

#: Activations with at least this many rows use the tcgen05 kernel (its tiles are 128 rows tall).
TCGEN05_MIN_ROWS = 128
#: The fused gate/up product (SiLU(gate) * up in the epilogue) takes portions of at least this many
#: rows; shorter ones go to cuBLAS followed by the activation kernel. Timed at the layer sizes of
#: 1-, 8- and 13-billion-parameter models, the fused kernel is ahead from about 1,500 rows on (2,048
#: rows, 8B: 337 against 384 us; 8,192 rows: 1,390 against 1,632) and behind below (544 rows, 13B:
#: 145 against 124 us; 256 rows, 8B: 69 against 61): with few row blocks its 128 x 256 tiles fill the
#: SMs' rounds unevenly and the library's wider two-SM tiles do more per byte of shared memory.
#: Tests set it to ``TCGEN05_MIN_ROWS`` to run the kernel at their sizes.
SILU_TCGEN05_MIN_ROWS = 1536
#: Set to False to send every product to cuBLAS (used by tests that compare the two).
USE_TCGEN05 = True
#: Which kernel takes the plain products (no fused epilogue) of prompt portions: "library" for
#: cuBLAS, "tcgen05" for the two-SM kernel of this package. Timed at 2,048 rows with the layer
#: sizes of an 8-billion-parameter model, cuBLAS is ahead on these by a tenth (fewer idle SMs in
#: the last wave of tiles), while the fused gate/up product is faster here than cuBLAS followed by
#: an activation kernel, so the library keeps the plain ones.
PLAIN_PRODUCT_KERNEL = "library"
#: Products with at most this many rows (decode steps) and a bfloat16 result go to the
#: weight-streaming kernel of ``csrc/gemm_small_m.cu`` (it takes up to 32 rows); 0 sends them to
#: cuBLAS. Inside a decode step of an 8-billion-parameter model the kernel is level with cuBLAS
#: plus the activation kernel at batch 8 and 3 to 4 % ahead at batch 1; from 16 rows on it falls
#: behind (it re-reads the activations for every 16 weight rows). The LM head (float32 result, one
#: long stream per step) stays with cuBLAS, which reaches the memory's copy rate there.
SMALL_M_ROWS = 8
#: Whether that kernel is launched as a programmatic dependent where the caller asks for it
#: (``chain=True``).
SMALL_M_CHAINED = True
#: Products of ``SMALL_M_ROWS + 1`` to this many rows go to the tcgen05 weight-streaming kernel of
#: ``csrc/gemm_stream.cu`` (tiles of 128 weight rows as the tall side of the MMA, weights through a
#: TMA ring, the fused residual / norm / activation epilogues that cuBLAS cannot carry); 0, the
#: default, leaves them with cuBLAS. Measured at the sizes of an 8-billion-parameter model: a ring
#: of 16 KB TMA boxes alone streams the gate/up weights in 35.6 us (6.6 TB/s), but every tile of
#: the product is shared by two or three blocks (112 pairs of tiles on 148 SMs) and settling the
#: partial accumulators through the workspace costs 4 us at the end of the kernel: 43 to 45 us at 8
#: and 16 rows, level with the kernel above (43) and cuBLAS + activation kernel (42). The smaller
#: products pay the same fixed cost on less work (output projection 12.5 us against 7.6 and 9.2).
#: Inside a decode step of 16 or 32 rows the kernel is slower than the cuBLAS path (4.23 against
#: 3.81 ms, 5.06 against 4.34 ms a step), and mixed with the kernel above in steps of up to 8 rows
#: it slows that kernel down (the two want opposite divisions of an SM's memory between L1 and
#: shared memory). What it needs to pay off is a cheaper settle (the blocks that share a tile as
#: one thread-block cluster, partial accumulators through distributed shared memory).
STREAM_ROWS = 0


class PendingNorm:
    """RMS-normalised rows that have not been divided by their root mean square yet: ``weighted``
    is the stream times the norm's weight (bfloat16), ``sumsq [parts, stride]`` the sums of squares
    of the stream per tile of columns and row (``gemm_small_m`` leaves tiles of 16 columns and a
    stride of 32, ``gemm_stream`` tiles of 128 columns and a stride of 128). ``linear`` and
    ``linear_silu_mul`` take it in place of a tensor and divide their result rows instead (a
    product is linear in its rows); anything else calls ``tensor()``."""

    __slots__ = ("weighted", "sumsq", "eps")

    def __init__(self, weighted: torch.Tensor, sumsq: torch.Tensor, eps: float) -> None:
        self.weighted, self.sumsq, self.eps = weighted, sumsq, float(eps)

    @property
    def shape(self):
        return self.weighted.shape

    @property
    def dtype(self):
        return self.weighted.dtype

    def tensor(self) -> torch.Tensor:
        return ops.finish_norm(self.weighted, self.sumsq, self.eps)


def as_tensor(x: "torch.Tensor | PendingNorm") -> torch.Tensor:
    return x.tensor() if isinstance(x, PendingNorm) else x


def _small_m(x: torch.Tensor, w_nk: torch.Tensor, epilogue: str) -> bool:
    return (USE_TCGEN05 and x.dtype == torch.bfloat16 and x.shape[0] <= SMALL_M_ROWS
            and ops.gemm_small_m_supports(x, w_nk, epilogue))


def _stream(x: torch.Tensor, w_nk: torch.Tensor, epilogue: str) -> bool:
    return (USE_TCGEN05 and x.dtype == torch.bfloat16 and SMALL_M_ROWS < x.shape[0] <= STREAM_ROWS
            and ops.gemm_stream_supports(x, w_nk, epilogue))


def _own_kernel(x: torch.Tensor, w_nk: torch.Tensor) -> bool:
    return (USE_TCGEN05 and x.dtype == torch.bfloat16 and x.shape[0] >= TCGEN05_MIN_ROWS
            and ops.gemm_tcgen05_supports(x, w_nk))


def matmul(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x [T, K] @ w [K, N]`` through cuBLAS; ``w`` may be a transposed view."""
    if not x.is_cuda:
        raise ValueError("matmul runs on the GPU only (there is no CPU path)")
    if x.dtype != w.dtype:
        raise TypeError(f"operands differ in type: {x.dtype} and {w.dtype}")
    if out_dtype is not None and out_dtype != x.dtype:
        return torch.mm(x, w, out_dtype=out_dtype)
    if arena.active() is not None:      # the product's rows change with every batch: memory of the step's own
        return torch.mm(x, w, out=arena.empty((x.shape[0], w.shape[1]), x.dtype, x.device))
    return torch.mm(x, w)


def linear(x: torch.Tensor, w_nk: torch.Tensor, out_dtype: torch.dtype | None = None,
           chain: bool = False) -> torch.Tensor:
    """``x [T, K] @ w_nk [N, K]^T``; ``out_dtype`` float32 keeps the float32 accumulator.

    ``chain``: launch the decode kernel as a programmatic dependent of the kernel before it on the
    stream, so that it requests its first weights while that kernel ends. Measured inside a decode
    step: this pays after a norm and after another product of this module (which lets its
    dependents start when its own reads are done). It must not follow a kernel that needs most of
    an SM's memory as shared memory (the attention kernels): an SM changes its division between
    L1 and shared memory only when idle, and a product whose blocks arrive beside such a kernel's
    keeps the small L1 and streams at half speed, and so do the products chained after it."""
    wants_f32 = out_dtype == torch.float32
    if isinstance(x, PendingNorm):
        if not wants_f32 and x.sumsq.shape[1] == 32 and _small_m(x.weighted, w_nk, "bf16"):
            return ops.gemm_small_m(x.weighted, w_nk, "bf16", chained=SMALL_M_CHAINED and chain,
                                    row_norm=(x.sumsq, x.eps))
        if not wants_f32 and _stream(x.weighted, w_nk, "bf16"):
            return ops.gemm_stream(x.weighted, w_nk, ops.status_word(w_nk.device), "bf16",
                                   chained=SMALL_M_CHAINED and chain, row_norm=(x.sumsq, x.eps))
        x = x.tensor()
    if not wants_f32 and _small_m(x, w_nk, "bf16"):
        return ops.gemm_small_m(x, w_nk, "bf16", chained=SMALL_M_CHAINED and chain)
    if not wants_f32 and _stream(x, w_nk, "bf16"):
        return ops.gemm_stream(x, w_nk, ops.status_word(w_nk.device), "bf16", chained=SMALL_M_CHAINED and chain)
    # rows of the output must start on 16-byte boundaries for the kernel's vector stores
    if (PLAIN_PRODUCT_KERNEL == "tcgen05" and w_nk.shape[0] % (4 if wants_f32 else 8) == 0
            and _own_kernel(x, w_nk)):
        return ops.gemm_tcgen05(x, w_nk, ops.status_word(x.device), "f32" if wants_f32 else "bf16")
    return matmul(x, w_nk.t(), out_dtype)


def linear_rope_kv_store(x: "torch.Tensor | PendingNorm", w_nk: torch.Tensor, positions: torch.Tensor,
                         cos: torch.Tensor | None, sin: torch.Tensor | None, k_pool: torch.Tensor, v_pool: torch.Tensor,
                         slots: torch.Tensor | None, n_heads: int, n_kv: int, head_dim: int, page_size: int,
                         chain: bool = False) -> torch.Tensor:
    """The fused query/key/value projection ``x @ w_nk^T`` followed by ``ops.rope_kv_store``: the
    queries rotated in the returned ``[T, (H + 2 KV) hd]`` matrix, keys (rotated) and values in the
    pools at ``slots``. For the few rows of a decode step one kernel does both."""
    fused_ok = head_dim % 16 == 0 and k_pool.dtype == torch.bfloat16
    if isinstance(x, PendingNorm):
        if fused_ok and x.sumsq.shape[1] == 32 and _small_m(x.weighted, w_nk, "bf16"):
            return ops.gemm_small_m(x.weighted, w_nk, chained=SMALL_M_CHAINED and chain,
                                    row_norm=(x.sumsq, x.eps),
                                    rope_kv=(positions, cos, sin, k_pool, v_pool, slots, n_heads, n_kv, head_dim, page_size))
        elif _stream(x.weighted, w_nk, "bf16"):
            # the product divides its rows itself; rotation and cache write follow as their own kernel
            qkv = linear(x, w_nk, chain=chain)
            ops.rope_kv_store(qkv, positions, cos, sin, k_pool, v_pool, slots, n_heads, n_kv, head_dim, page_size)
            return qkv
        x = x.tensor()
    if fused_ok and _small_m(x, w_nk, "bf16"):
        return ops.gemm_small_m(x, w_nk, chained=SMALL_M_CHAINED and chain,
                                rope_kv=(positions, cos, sin, k_pool, v_pool, slots, n_heads, n_kv, head_dim, page_size))
    qkv = linear(x, w_nk, chain=chain)
    ops.rope_kv_store(qkv, positions, cos, sin, k_pool, v_pool, slots, n_heads, n_kv, head_dim, page_size)
    return qkv


def linear_add_norm(x: torch.Tensor, w_nk: torch.Tensor, hidden: torch.Tensor, norm_weight: torch.Tensor, eps: float,
                    out_dtype: torch.dtype, chain: bool = False) -> "torch.Tensor | PendingNorm":
    """``hidden += x @ w_nk^T`` (the float32 stream, in place) and the RMS-normalised stream in
    ``out_dtype``. For the few rows of a decode step the weight-streaming kernel adds the product
    to the stream in its epilogue and leaves the norm as a ``PendingNorm`` for the product that
    reads it; otherwise it is the product followed by the add-and-norm kernel."""
    x = as_tensor(x)
    if out_dtype == torch.bfloat16 and w_nk.shape[0] % 32 == 0 and _small_m(x, w_nk, "bf16"):
        # the width of the stream is the inner size of the product that reads it: a multiple of 32
        weighted, sumsq = ops.gemm_small_m(x, w_nk, chained=SMALL_M_CHAINED and chain,
                                           residual=(hidden, norm_weight))
        return PendingNorm(weighted, sumsq, eps)
    if out_dtype == torch.bfloat16 and w_nk.shape[0] % 64 == 0 and _stream(x, w_nk, "bf16"):
        # (the stream's width is the inner size of the tcgen05 product that reads it: a multiple of 64)
        weighted, sumsq = ops.gemm_stream(x, w_nk, ops.status_word(w_nk.device), chained=SMALL_M_CHAINED and chain,
                                          residual=(hidden, norm_weight))
        return PendingNorm(weighted, sumsq, eps)
    return ops.add_rmsnorm(hidden, linear(x, w_nk, chain=chain), norm_weight, eps, out_dtype)


def linear_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor, ff: int, interleave: int, clip: float,
                    chain: bool = False) -> torch.Tensor:
    """``silu(x @ gate^T) * (x @ up^T)`` for gate and up rows held in one matrix (``interleave``
    as in ``ops.silu_mul``); ``[T, ff]``."""
    if isinstance(x, PendingNorm):
        if interleave == 128 and _stream(x.weighted, w_gate_up, "silu_mul"):
            return ops.gemm_stream(x.weighted, w_gate_up, ops.status_word(w_gate_up.device), "silu_mul", n_out=ff,
                                   clip=clip, chained=SMALL_M_CHAINED and chain, row_norm=(x.sumsq, x.eps))
        if interleave == 128 and x.sumsq.shape[1] == 32 and _small_m(x.weighted, w_gate_up, "silu_mul"):
            return ops.gemm_small_m(x.weighted, w_gate_up, "silu_mul", n_out=ff, clip=clip,
                                    chained=SMALL_M_CHAINED and chain, row_norm=(x.sumsq, x.eps))
        x = x.tensor()
    if interleave == 128 and _stream(x, w_gate_up, "silu_mul"):
        return ops.gemm_stream(x, w_gate_up, ops.status_word(w_gate_up.device), "silu_mul", n_out=ff, clip=clip,
                               chained=SMALL_M_CHAINED and chain)
    if interleave == 128 and _small_m(x, w_gate_up, "silu_mul"):
        return ops.gemm_small_m(x, w_gate_up, "silu_mul", n_out=ff, clip=clip,
                                chained=SMALL_M_CHAINED and chain)
    if interleave == 128 and w_gate_up.shape[0] % 256 == 0 and ff % 8 == 0 and x.shape[0] >= SILU_TCGEN05_MIN_ROWS \
            and _own_kernel(x, w_gate_up):
        # one SM per tile: with this many tiles the two-SM kernel's split of the last wave costs
        # more than it saves
        return ops.gemm_tcgen05(x, w_gate_up, ops.status_word(x.device), "silu_mul", n_out=ff, clip=clip,
                                pairs=False)
    return ops.silu_mul(matmul(x, w_gate_up.t()), clip, ff=ff, interleave=interleave)
