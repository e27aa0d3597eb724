"""Matrix products of the product path.

The reference's engine hands every matrix product to a library (NumPy/OpenBLAS,
src/paged_kv_serving/engine/model.py:249,258-259,264); here the library is cuBLAS through
``torch.mm``. Reduced-precision modes are switched off: float32 products use true float32
multiply-adds (no TF32), bfloat16 products accumulate in float32 without reduced-precision
reductions.
"""

from __future__ import annotations

import torch

__all__ = ["matmul"]

torch.backends.cuda.matmul.allow_tf32 = False
torch.backends.cudnn.allow_tf32 = False
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False


def matmul(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x [T, K] @ w [K, N]``; ``w`` may be a transposed view. ``out_dtype`` float32 keeps the
    float32 accumulator of a bfloat16 product."""
    if not x.is_cuda:
        raise ValueError("matmul runs on the GPU only (there is no CPU path)")
    if x.dtype != w.dtype:
        raise TypeError(f"operands differ in type: {x.dtype} and {w.dtype}")
    if out_dtype is not None and out_dtype != x.dtype:
        return torch.mm(x, w, out_dtype=out_dtype)
    return torch.mm(x, w)
