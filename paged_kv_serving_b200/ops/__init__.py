"""Python bindings of the hand-written CUDA kernels (``csrc/*.cu``), through ``ctypes``.

Every wrapper takes torch tensors that live on the GPU, checks what the kernel relies on
(dtype, contiguity, sizes), launches on torch's current stream and raises on a refused argument
or a failed launch. Nothing here falls back to a library or to the CPU.

Three kernels keep a workspace per device from launch to launch (partial tiles, arrival counters,
flags: ``gemm_small_m``, the two-SM ``gemm_tcgen05``, ``attention_decode_flat``). They are shared by
every caller in the process and serve one stream per device; see ``_one_stream``.
"""

from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_longlong, c_void_p

import torch

from paged_kv_serving_b200.ops.arena import empty as _empty
from paged_kv_serving_b200.ops.build import build_all, library, library_names

__all__ = [
    "add_rmsnorm", "attention_bf16_rows", "attention_bf16_supports", "attention_decode_bf16",
    "attention_decode_blocks_per_sm", "attention_decode_flat", "attention_decode_flat_blocks_per_sm",
    "attention_decode_flat_supports", "attention_decode_tma", "attention_decode_tma_blocks_per_sm",
    "attention_decode_tma_pushed_splits", "attention_decode_tma_supports",
    "attention_prefill_bf16", "attention_prefill_tcgen05", "attention_rows_per_block", "attention_tcgen05_narrow_boxes",
    "attention_tcgen05_rows",
    "attention_tcgen05_supports", "build_all", "copy_page", "dtype_code", "embedding_gather", "finish_norm", "gemm_small_m", "gemm_small_m_supports",
    "gemm_stream", "gemm_stream_supports", "gemm_tcgen05", "gemm_tcgen05_supports", "gemm_workspace",
    "launch_count", "library", "library_names", "paged_attention_generic", "raise_for_status", "reset_workspaces",
    "rope_kv_store", "sample", "silu_mul", "status_word", "wait_probe",
]

_CODES = {torch.float32: 0, torch.bfloat16: 1}
_ERRORS = {
    -2: "unsupported element type", -3: "refused size", -4: "refused alignment",
    -5: "size beyond the kernel's limit", -6: "device index beyond the kernel's table",
}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise TypeError(f"kernels take float32 or bfloat16 tensors, not {dtype}") from None


#: Number of kernel launches issued through this module since import (or the last reset).
LAUNCHES = {"count": 0}


def launch_count() -> int:
    return LAUNCHES["count"]


def _check(status: int, what: str) -> None:
    if status == 0:
        LAUNCHES["count"] += 1
        return
    if status < 0:
        raise ValueError(f"{what}: {_ERRORS.get(status, f'refused (code {status})')}")
    raise RuntimeError(f"{what}: CUDA error {status} at launch")


def _ptr(tensor: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if tensor is None else tensor.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(tensor: torch.Tensor, dtype: torch.dtype | None, name: str) -> None:
    if not tensor.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and tensor.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, found {tensor.dtype}")
    if not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


_SIGNATURES_SET: set[tuple[str, str]] = set()


def _fn(lib_name: str, fn_name: str, argtypes: list):
    lib = library(lib_name)
    fn = getattr(lib, fn_name)
    if (lib_name, fn_name) not in _SIGNATURES_SET:
        fn.argtypes = argtypes
        fn.restype = c_int
        _SIGNATURES_SET.add((lib_name, fn_name))
    return fn


# ---------------------------------------------------------------------------------------------


def embedding_gather(table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor,
                     fed_back: torch.Tensor | None = None, fed_back_at: torch.Tensor | None = None) -> torch.Tensor:
    """``table[ids]`` widened to float32. An id outside the table sets ``status[0]`` to 1.
    With ``fed_back`` (int32 ids on the device) and ``fed_back_at`` (one int32 per token), a token
    whose ``fed_back_at`` is not negative takes ``fed_back[fed_back_at]`` as its id."""
    _need(table, None, "table"); _need(ids, torch.int32, "ids"); _need(status, torch.int32, "status")
    if (fed_back is None) != (fed_back_at is None):
        raise ValueError("fed_back and fed_back_at go together")
    if fed_back is not None:
        _need(fed_back, torch.int32, "fed_back"); _need(fed_back_at, torch.int32, "fed_back_at")
        if fed_back_at.numel() != ids.numel():
            raise ValueError("fed_back_at needs one element per token")
    vocab, d = table.shape
    out = _empty((ids.numel(), d), torch.float32, table.device)
    fn = _fn("elementwise", "pkv_embedding_gather",
             [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), ids.numel(), d, vocab,
              _ptr(status), _ptr(fed_back), _ptr(fed_back_at), _stream()), "embedding_gather")
    return out


def add_rmsnorm(hidden: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: torch.Tensor | None = None) -> torch.Tensor:
    """``hidden += delta`` (in place, float32) and the RMS-normalised rows in ``out_dtype``.

    With ``rows`` only those rows are normalised and returned, and ``hidden`` is left untouched.
    """
    _need(hidden, torch.float32, "hidden"); _need(weight, torch.float32, "weight")
    n, d = hidden.shape
    if weight.numel() != d:
        raise ValueError(f"norm weight has {weight.numel()} elements, the stream is {d} wide")
    if delta is not None:
        _need(delta, None, "delta")
        if delta.shape != hidden.shape:
            raise ValueError("delta and hidden differ in shape")
    n_rows = n
    if rows is not None:
        _need(rows, torch.int32, "rows")
        n_rows = rows.numel()
    out = _empty((n_rows, d), out_dtype, hidden.device)
    fn = _fn("elementwise", "pkv_add_rmsnorm",
             [c_void_p, c_void_p, c_int, c_void_p, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(hidden), _ptr(delta), dtype_code(delta.dtype) if delta is not None else 0, _ptr(weight),
              float(eps), _ptr(out), dtype_code(out_dtype), _ptr(rows), n_rows, d, _stream()), "add_rmsnorm")
    return out


def copy_page(k_pool: torch.Tensor, v_pool: torch.Tensor, source: int, destination: int) -> None:
    """Copy page ``source`` onto page ``destination`` in every layer of both pools
    (``[layers, pages, ...]``, equal shapes and types): copy-on-write of a cache page in one launch."""
    _need(k_pool, None, "k_pool"); _need(v_pool, k_pool.dtype, "v_pool")
    if k_pool.shape != v_pool.shape or k_pool.dim() < 2:
        raise ValueError("the pools must be [layers, pages, ...] of equal shape")
    layers, pages = k_pool.shape[0], k_pool.shape[1]
    page_bytes = k_pool.stride(1) * k_pool.element_size()
    fn = _fn("elementwise", "pkv_copy_page",
             [c_void_p, c_void_p, c_int, c_longlong, c_longlong, c_longlong, c_longlong, c_longlong, c_void_p])
    _check(fn(_ptr(k_pool), _ptr(v_pool), layers, k_pool.stride(0) * k_pool.element_size(), page_bytes, pages,
              int(source), int(destination), _stream()), "copy_page")


def silu_mul(gate_up: torch.Tensor, clip: float, ff: int | None = None, interleave: int = 0) -> torch.Tensor:
    """``silu(gate) * up`` for a fused input ``[T, >= 2*ff]``; output ``[T, ff]``.

    ``interleave = 0``: the first ``ff`` columns are the gate, the next ``ff`` the up values.
    ``interleave = B``: blocks of ``B`` gate columns followed by the ``B`` matching up columns.
    """
    _need(gate_up, None, "gate_up")
    n, width = gate_up.shape
    if ff is None:
        ff = width // 2
    out = _empty((n, ff), gate_up.dtype, gate_up.device)
    fn = _fn("elementwise", "pkv_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(_ptr(gate_up), _ptr(out), dtype_code(gate_up.dtype), n, ff, width, int(interleave), float(clip),
              _stream()), "silu_mul")
    return out


_STATUS: dict[str, torch.Tensor] = {}


def _device_key(device: torch.device | str) -> str:
    """One name per device for the tables kept here: "cuda" means the current device, so that
    ``"cuda"`` and ``"cuda:0"`` find the same status word and workspaces."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return str(device)


def status_word(device: torch.device | str) -> torch.Tensor:
    """The int32 status word of a device: kernels record a code there instead of trapping
    (1: a token id outside the embedding table, 2: a kernel gave up a bounded wait, 3: a page, a
    cache slot or a position outside its range, which the kernel did not use)."""
    key = _device_key(device)
    if key not in _STATUS:
        _STATUS[key] = torch.zeros((1,), dtype=torch.int32, device=device)
    return _STATUS[key]


STATUS_MEANINGS = {1: "a token id outside the embedding table", 2: "a kernel gave up a bounded wait",
                   3: "a page, a cache slot or a position outside its range"}


def raise_for_status(code: int, device: torch.device | str) -> None:
    """What the host does with a status word it has read: nothing for 0; otherwise the word and
    the workspaces that kernels share from launch to launch are cleared (a kernel that gave up
    may have left counters or flags set, which would spoil every later launch) and the fault is
    raised. The results of the step that recorded the code are not to be used."""
    if not code:
        return
    torch.cuda.synchronize(device)
    status_word(device).zero_()
    reset_workspaces(device)
    raise RuntimeError(f"a kernel recorded a fault: {STATUS_MEANINGS.get(int(code), f'code {int(code)}')}")


def reset_workspaces(device: torch.device | str) -> None:
    """Zero the counters, flags and partial sums that kernels of this module keep on a device
    between launches (they are left zero by every launch that ends in order)."""
    key = _device_key(device)
    for kept in _DECODE_FLAT_SCRATCH.get(key, []):
        kept[1].zero_()
    for table in (_GEMM_WORKSPACE, _SMALL_M_WORKSPACE, _STREAM_WORKSPACE):
        if key in table:
            table[key].zero_()


_WORKSPACE_STREAM: dict[str, int] = {}


def _one_stream(device: torch.device | str) -> None:
    """The shared workspaces serve the launches of ONE stream per device: two launches that
    overlap would count each other's tiles. The first stream that uses them is remembered; a
    launch from another stream is refused unless it is being captured into a graph (a capture
    runs on a stream of its own and records launches, it runs none)."""
    key = _device_key(device)
    stream = torch.cuda.current_stream(device).cuda_stream
    known = _WORKSPACE_STREAM.setdefault(key, stream)
    if known != stream and not torch.cuda.is_current_stream_capturing():
        raise RuntimeError("the kernels' shared workspaces of this device belong to the stream that used them "
                           "first; launches from a second stream would race on their counters")


def wait_probe(status: torch.Tensor, limit_cycles: int) -> torch.Tensor:
    """Run one bounded wait that nothing will ever satisfy, with a limit of ``limit_cycles`` SM
    clock cycles: the wait gives up by itself and the kernel records code 2 in ``status`` as the
    tensor-core and TMA kernels do. Returns a device int that is 1 when the wait gave up. This is
    how the give-up path is exercised without faulting, trapping or hanging anything."""
    _need(status, torch.int32, "status")
    gave_up = torch.zeros((1,), dtype=torch.int32, device=status.device)
    fn = _fn("wait_probe", "pkv_wait_probe", [c_void_p, c_longlong, c_void_p, c_void_p])
    _check(fn(_ptr(status), int(limit_cycles), _ptr(gave_up), _stream()), "wait_probe")
    return gave_up


def rope_kv_store(qkv: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor | None, sin: torch.Tensor | None,
                  k_pool: torch.Tensor, v_pool: torch.Tensor, slots: torch.Tensor | None,
                  n_heads: int, n_kv: int, head_dim: int, page_size: int) -> None:
    """Rotate q and k of ``qkv [T, (H+2KV)*hd]`` by position (q in place) and write k, v to the
    pools ``[pages, KV, page_size, hd]`` at ``slots`` (``None``: rotate q only, store nothing).
    A slot outside the pools or a position outside the tables is not used: the kernel records
    code 3 in the device's status word, skips the store and rotates by position 0."""
    _need(qkv, None, "qkv"); _need(positions, torch.int32, "positions")
    _need(k_pool, None, "k_pool"); _need(v_pool, None, "v_pool")
    n = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise ValueError("qkv width does not match (n_heads + 2*n_kv) * head_dim")
    if cos is not None:
        _need(cos, torch.float32, "cos"); _need(sin, torch.float32, "sin")
        if cos.shape[1] != head_dim // 2:
            raise ValueError("rotary tables must be [positions, head_dim/2]")
    if slots is not None:
        _need(slots, torch.int32, "slots")
    fn = _fn("elementwise", "pkv_rope_kv_store",
             [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(qkv), dtype_code(qkv.dtype), _ptr(positions), _ptr(cos), _ptr(sin), _ptr(k_pool), _ptr(v_pool),
              dtype_code(k_pool.dtype), _ptr(slots), n, n_heads, n_kv, head_dim, page_size,
              0 if slots is None else 1, k_pool.shape[0] * page_size, 0 if cos is None else cos.shape[0],
              _ptr(status_word(qkv.device)), _stream()), "rope_kv_store")


def attention_rows_per_block() -> int:
    lib = library("attention_generic")
    lib.pkv_attention_generic_rows_per_block.restype = c_int
    return int(lib.pkv_attention_generic_rows_per_block())


def paged_attention_generic(qkv: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                            block_table: torch.Tensor, seq_starts: torch.Tensor, first_pos: torch.Tensor,
                            work_seq: torch.Tensor, work_row0: torch.Tensor, n_heads: int, n_kv: int,
                            head_dim: int, page_size: int, window: int, scale: float) -> torch.Tensor:
    """Causal attention of the (rotated) queries in ``qkv`` over the paged cache; ``[T, H*hd]``.
    A table entry that is neither a page of the pool nor -1 is read as no page (zeros) and
    recorded as code 3 in the device's status word."""
    _need(qkv, None, "qkv"); _need(k_pool, None, "k_pool"); _need(v_pool, None, "v_pool")
    for name, t in (("block_table", block_table), ("seq_starts", seq_starts), ("first_pos", first_pos),
                    ("work_seq", work_seq), ("work_row0", work_row0)):
        _need(t, torch.int32, name)
    n = qkv.shape[0]
    out = _empty((n, n_heads * head_dim), qkv.dtype, qkv.device)
    fn = _fn("attention_generic", "pkv_paged_attention_generic",
             [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
              c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(qkv), qkv.shape[1], _ptr(out), dtype_code(qkv.dtype), _ptr(k_pool), _ptr(v_pool),
              dtype_code(k_pool.dtype), _ptr(block_table), block_table.shape[1], _ptr(seq_starts), _ptr(first_pos),
              _ptr(work_seq), _ptr(work_row0), work_seq.numel(), n_heads, n_kv, head_dim, page_size, int(window),
              float(scale), k_pool.shape[0], _ptr(status_word(qkv.device)), _stream()), "paged_attention_generic")
    return out


def attention_bf16_supports(head_dim: int, q_row_stride: int) -> bool:
    """Whether the tensor-core bfloat16 attention kernels take this head size and row stride."""
    lib = library("attention_bf16")
    lib.pkv_attention_bf16_supports.restype = c_int
    lib.pkv_attention_bf16_supports.argtypes = [c_int, c_int]
    return bool(lib.pkv_attention_bf16_supports(int(head_dim), int(q_row_stride)))


def attention_bf16_rows() -> tuple[int, int]:
    """``(query rows per prefill block, most rows of a decode entry per key/value head)``."""
    lib = library("attention_bf16")
    lib.pkv_attention_bf16_rows.restype = c_int
    lib.pkv_attention_bf16_rows.argtypes = [c_int]
    return int(lib.pkv_attention_bf16_rows(0)), int(lib.pkv_attention_bf16_rows(1))


def attention_tcgen05_supports(head_dim: int, page_size: int, q_row_stride: int) -> bool:
    """Whether the tcgen05 prefill attention takes these sizes (head 64 or 128, pages of 8k keys)."""
    if head_dim not in (64, 128) or page_size % 8:
        return False     # known without building the library for a model that cannot use it
    lib = library("attention_tcgen05")
    lib.pkv_attention_tcgen05_supports.restype = c_int
    lib.pkv_attention_tcgen05_supports.argtypes = [c_int, c_int, c_int]
    return bool(lib.pkv_attention_tcgen05_supports(int(head_dim), int(page_size), int(q_row_stride)))


def attention_tcgen05_narrow_boxes(on: bool) -> bool:
    """For comparisons and tests: make the tcgen05 prefill attention fetch one copy per page and
    64-column panel even where it can fetch a page in one copy (head size 128). Returns the
    previous setting."""
    lib = library("attention_tcgen05")
    lib.pkv_attention_tcgen05_narrow_boxes.restype = c_int
    lib.pkv_attention_tcgen05_narrow_boxes.argtypes = [c_int]
    return bool(lib.pkv_attention_tcgen05_narrow_boxes(int(bool(on))))


def attention_tcgen05_rows() -> int:
    lib = library("attention_tcgen05")
    lib.pkv_attention_tcgen05_rows.restype = c_int
    return int(lib.pkv_attention_tcgen05_rows())


def attention_prefill_tcgen05(qkv: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                              block_table: torch.Tensor, seq_starts: torch.Tensor, first_pos: torch.Tensor,
                              work_seq: torch.Tensor, work_q0: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                              page_size: int, window: int, scale: float, status: torch.Tensor) -> None:
    """Prefill attention on tcgen05 tensor cores with TMA page loads; writes the rows of its work
    items (blocks of 128 queries) into ``out``."""
    for name, t in (("qkv", qkv), ("out", out), ("k_pool", k_pool), ("v_pool", v_pool)):
        _need(t, torch.bfloat16, name)
    for name, t in (("block_table", block_table), ("seq_starts", seq_starts), ("first_pos", first_pos),
                    ("work_seq", work_seq), ("work_q0", work_q0), ("status", status)):
        _need(t, torch.int32, name)
    fn = _fn("attention_tcgen05", "pkv_attention_prefill_tcgen05",
             [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p,
              c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(fn(_ptr(qkv), qkv.shape[1], qkv.shape[0], _ptr(out), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0],
              _ptr(block_table), block_table.shape[1], _ptr(seq_starts), _ptr(first_pos), _ptr(work_seq),
              _ptr(work_q0), work_seq.numel(), n_heads, n_kv, head_dim, page_size, int(window), float(scale),
              _ptr(status), _stream()), "attention_prefill_tcgen05")


_DECODE_TMA_BLOCKS: dict[tuple[int, bool], int] = {}


def attention_decode_tma_supports(head_dim: int, page_size: int, q_row_stride: int) -> bool:
    """Whether the TMA-fed decode attention takes these sizes (head 64 or 128, pages of 8k keys)."""
    if head_dim not in (64, 128) or page_size % 8:
        return False     # known without building the library for a model that cannot use it
    lib = library("attention_decode_tma")
    lib.pkv_attention_decode_tma_supports.restype = c_int
    lib.pkv_attention_decode_tma_supports.argtypes = [c_int, c_int, c_int]
    return bool(lib.pkv_attention_decode_tma_supports(int(head_dim), int(page_size), int(q_row_stride)))


def attention_decode_tma_blocks_per_sm(head_dim: int, deep_ring: bool) -> int:
    """Blocks of the TMA decode kernel per SM with the deep (six-stage) or shallow (three-stage) ring."""
    key = (head_dim, bool(deep_ring))
    if key not in _DECODE_TMA_BLOCKS:
        lib = library("attention_decode_tma")
        lib.pkv_attention_decode_tma_blocks_per_sm.restype = c_int
        lib.pkv_attention_decode_tma_blocks_per_sm.argtypes = [c_int, c_int]
        _DECODE_TMA_BLOCKS[key] = max(1, int(lib.pkv_attention_decode_tma_blocks_per_sm(int(head_dim), int(deep_ring))))
    return _DECODE_TMA_BLOCKS[key]


_DECODE_TMA_PUSHED: dict[tuple[int, int], int] = {}


def attention_decode_tma_pushed_splits(head_dim: int, rows: int) -> int:
    """Most splits that the TMA decode kernel merges the fast way (the other blocks of a cluster
    push their states into the first one) for entries of ``rows`` (token, head in group) rows."""
    key = (int(head_dim), int(rows))
    if key not in _DECODE_TMA_PUSHED:
        lib = library("attention_decode_tma")
        lib.pkv_attention_decode_tma_pushed_splits.restype = c_int
        lib.pkv_attention_decode_tma_pushed_splits.argtypes = [c_int, c_int]
        _DECODE_TMA_PUSHED[key] = int(lib.pkv_attention_decode_tma_pushed_splits(*key))
    return _DECODE_TMA_PUSHED[key]


def attention_decode_tma(qkv: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                         block_table: torch.Tensor, seq_starts: torch.Tensor, first_pos: torch.Tensor,
                         work_seq: torch.Tensor, max_entry_tokens: int, n_heads: int, n_kv: int, head_dim: int,
                         page_size: int, window: int, scale: float, num_splits: int, status: torch.Tensor,
                         deep_ring: bool = True) -> None:
    """Split-KV decode attention with TMA page loads into a ring of stages (at most 8 splits,
    merged inside a thread-block cluster); writes the rows of its entries into ``out``.
    ``deep_ring``: six stages and one block per SM (few blocks), else three stages and two."""
    for name, t in (("qkv", qkv), ("out", out), ("k_pool", k_pool), ("v_pool", v_pool)):
        _need(t, torch.bfloat16, name)
    for name, t in (("block_table", block_table), ("seq_starts", seq_starts), ("first_pos", first_pos),
                    ("work_seq", work_seq), ("status", status)):
        _need(t, torch.int32, name)
    fn = _fn("attention_decode_tma", "pkv_attention_decode_tma",
             [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(qkv), qkv.shape[1], _ptr(out), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(block_table),
              block_table.shape[1], _ptr(seq_starts), _ptr(first_pos), _ptr(work_seq), work_seq.numel(),
              int(max_entry_tokens), n_heads, n_kv, head_dim, page_size, int(window), float(scale), int(num_splits),
              int(bool(deep_ring)), _ptr(status), _stream()), "attention_decode_tma")


_DECODE_FLAT_BLOCKS: dict[int, int] = {}
_DECODE_FLAT_SCRATCH: dict[str, list[tuple[torch.Tensor, torch.Tensor]]] = {}


def attention_decode_flat_supports(head_dim: int, page_size: int, q_row_stride: int) -> bool:
    """Whether the even-shares decode kernel takes these sizes (answered without building it)."""
    return attention_decode_tma_supports(head_dim, page_size, q_row_stride)


def attention_decode_flat_blocks_per_sm(head_dim: int) -> int:
    """Blocks of the even-shares decode kernel that one SM holds."""
    if head_dim not in _DECODE_FLAT_BLOCKS:
        lib = library("attention_decode_flat")
        lib.pkv_attention_decode_flat_blocks_per_sm.restype = c_int
        lib.pkv_attention_decode_flat_blocks_per_sm.argtypes = [c_int]
        _DECODE_FLAT_BLOCKS[head_dim] = max(1, int(lib.pkv_attention_decode_flat_blocks_per_sm(int(head_dim))))
    return _DECODE_FLAT_BLOCKS[head_dim]


def _decode_flat_scratch(device: torch.device, floats: int, pairs: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Workspace and arrival counters of ``attention_decode_flat`` on a device. Counters are zeroed
    once and left zero by every launch. A buffer that has become too small is replaced but kept
    alive, since captured graphs may still point at it."""
    _one_stream(device)
    key = _device_key(device)
    kept = _DECODE_FLAT_SCRATCH.setdefault(key, [])
    if not kept or kept[-1][0].numel() < floats or kept[-1][1].numel() < pairs:
        kept.append((torch.empty((max(floats, 1 << 21),), dtype=torch.float32, device=device),
                     torch.zeros((max(pairs, 1 << 18),), dtype=torch.int32, device=device)))
    return kept[-1]


def attention_decode_flat(qkv: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                          block_table: torch.Tensor, seq_starts: torch.Tensor, first_pos: torch.Tensor,
                          work_seq: torch.Tensor, unit_starts: torch.Tensor, max_entry_tokens: int, n_heads: int,
                          n_kv: int, head_dim: int, page_size: int, window: int, scale: float, blocks: int,
                          status: torch.Tensor) -> None:
    """Decode attention over even shares of the step's keys: the 64-key tiles of all entries in
    ``work_seq`` and all kv heads, laid end to end, are cut into ``blocks`` equal ranges, one per
    block; parts of one (entry, head) are added up by the block that finishes last.
    ``unit_starts [entries + 1]``: the number of tiles of the entries before each entry, a tile
    being 64 key positions counted from position 0 (entry i has tiles ``key_lo // 64`` to
    ``(key_hi - 1) // 64`` with ``key_hi`` its context length after this step and ``key_lo`` the
    first position inside the window of its first query). Writes the rows of its entries into ``out``."""
    for name, t in (("qkv", qkv), ("out", out), ("k_pool", k_pool), ("v_pool", v_pool)):
        _need(t, torch.bfloat16, name)
    for name, t in (("block_table", block_table), ("seq_starts", seq_starts), ("first_pos", first_pos),
                    ("work_seq", work_seq), ("unit_starts", unit_starts), ("status", status)):
        _need(t, torch.int32, name)
    n_work = work_seq.numel()
    if unit_starts.numel() != n_work + 1:
        raise ValueError("unit_starts needs one more element than there are entries")
    lib = library("attention_decode_flat")
    lib.pkv_attention_decode_flat_workspace_floats.restype = c_longlong
    lib.pkv_attention_decode_flat_workspace_floats.argtypes = [c_int, c_int]
    floats = int(lib.pkv_attention_decode_flat_workspace_floats(int(head_dim), int(blocks)))
    workspace, counters = _decode_flat_scratch(qkv.device, floats, n_work * n_kv)
    fn = _fn("attention_decode_flat", "pkv_attention_decode_flat",
             [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
              c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_longlong, c_void_p,
              c_longlong, c_void_p, c_void_p])
    _check(fn(_ptr(qkv), qkv.shape[1], _ptr(out), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(block_table),
              block_table.shape[1], _ptr(seq_starts), _ptr(first_pos), _ptr(work_seq), _ptr(unit_starts), n_work,
              int(max_entry_tokens), n_heads, n_kv, head_dim, page_size, int(window), float(scale), int(blocks),
              _ptr(workspace), workspace.numel(), _ptr(counters), counters.numel(), _ptr(status), _stream()),
           "attention_decode_flat")


_DECODE_BLOCKS: dict[int, int] = {}


def attention_decode_blocks_per_sm(head_dim: int) -> int:
    """Decode-attention blocks that fit on one SM at this head size (for sizing the key splits)."""
    if head_dim not in _DECODE_BLOCKS:
        lib = library("attention_bf16")
        lib.pkv_attention_decode_blocks_per_sm.restype = c_int
        lib.pkv_attention_decode_blocks_per_sm.argtypes = [c_int]
        _DECODE_BLOCKS[head_dim] = max(1, int(lib.pkv_attention_decode_blocks_per_sm(int(head_dim))))
    return _DECODE_BLOCKS[head_dim]


def attention_prefill_bf16(qkv: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                           block_table: torch.Tensor, seq_starts: torch.Tensor, first_pos: torch.Tensor,
                           work_seq: torch.Tensor, work_q0: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                           page_size: int, window: int, scale: float) -> None:
    """Tensor-core attention for runs of queries; writes the rows of its work items into ``out``."""
    for name, t in (("qkv", qkv), ("out", out), ("k_pool", k_pool), ("v_pool", v_pool)):
        _need(t, torch.bfloat16, name)
    for name, t in (("block_table", block_table), ("seq_starts", seq_starts), ("first_pos", first_pos),
                    ("work_seq", work_seq), ("work_q0", work_q0)):
        _need(t, torch.int32, name)
    fn = _fn("attention_bf16", "pkv_attention_prefill_bf16",
             [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(qkv), qkv.shape[1], _ptr(out), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
              block_table.shape[1], _ptr(seq_starts), _ptr(first_pos), _ptr(work_seq), _ptr(work_q0),
              work_seq.numel(), n_heads, n_kv, head_dim, page_size, int(window), float(scale), k_pool.shape[0],
              _ptr(status_word(qkv.device)), _stream()), "attention_prefill_bf16")


def attention_decode_bf16(qkv: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                          block_table: torch.Tensor, seq_starts: torch.Tensor, first_pos: torch.Tensor,
                          work_seq: torch.Tensor, max_entry_tokens: int, n_heads: int, n_kv: int, head_dim: int,
                          page_size: int, window: int, scale: float, num_splits: int,
                          scratch: torch.Tensor | None) -> None:
    """Split-KV tensor-core attention for entries of a few rows. With ``num_splits > 1`` the
    partial results pass through ``scratch`` (float32, ``T * H * num_splits * (hd + 2)`` values)."""
    for name, t in (("qkv", qkv), ("out", out), ("k_pool", k_pool), ("v_pool", v_pool)):
        _need(t, torch.bfloat16, name)
    for name, t in (("block_table", block_table), ("seq_starts", seq_starts), ("first_pos", first_pos),
                    ("work_seq", work_seq)):
        _need(t, torch.int32, name)
    total_rows = qkv.shape[0] * n_heads
    if num_splits > 8:     # up to 8 splits merge inside a thread-block cluster and need no scratch
        _need(scratch, torch.float32, "scratch")
        if scratch.numel() < total_rows * num_splits * (head_dim + 2):
            raise ValueError("attention scratch is too small for this many splits")
    fn = _fn("attention_bf16", "pkv_attention_decode_bf16",
             [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_longlong, c_int, c_void_p,
              c_void_p])
    _check(fn(_ptr(qkv), qkv.shape[1], _ptr(out), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
              block_table.shape[1], _ptr(seq_starts), _ptr(first_pos), _ptr(work_seq), work_seq.numel(),
              int(max_entry_tokens), n_heads, n_kv, head_dim, page_size, int(window), float(scale), int(num_splits),
              _ptr(scratch), total_rows, k_pool.shape[0], _ptr(status_word(qkv.device)), _stream()),
           "attention_decode_bf16")
    if num_splits > 8:
        LAUNCHES["count"] += 1   # the merge kernel


def gemm_tcgen05_supports(a: torch.Tensor, b_nk: torch.Tensor) -> bool:
    """Whether the hand-written tcgen05 product takes these operands (bfloat16, K contiguous,
    16-byte aligned rows)."""
    if a.dtype != torch.bfloat16 or b_nk.dtype != torch.bfloat16 or a.stride(1) != 1 or b_nk.stride(1) != 1:
        return False
    lib = library("gemm_tcgen05")
    lib.pkv_gemm_tcgen05_supports.restype = c_int
    lib.pkv_gemm_tcgen05_supports.argtypes = [c_longlong, c_longlong, c_int, c_int, c_int]
    return bool(lib.pkv_gemm_tcgen05_supports(a.data_ptr(), b_nk.data_ptr(), a.stride(0), b_nk.stride(0), a.shape[1]))


GEMM_EPILOGUES = {"bf16": 0, "f32": 1, "silu_mul": 2}
_GEMM_WORKSPACE: dict[str, torch.Tensor] = {}


def gemm_workspace(device: torch.device | str) -> torch.Tensor:
    """The workspace of the two-SM tcgen05 product on a device (partial accumulators and flags of
    its stream-K hand-over), allocated and zeroed once. Launches on one stream share it."""
    _one_stream(device)
    key = _device_key(device)
    if key not in _GEMM_WORKSPACE:
        lib = library("gemm_tcgen05")
        lib.pkv_gemm_tcgen05_workspace_bytes.restype = c_longlong
        with torch.cuda.device(device):
            size = int(lib.pkv_gemm_tcgen05_workspace_bytes())
        _GEMM_WORKSPACE[key] = torch.zeros((size,), dtype=torch.uint8, device=device)
    return _GEMM_WORKSPACE[key]


def gemm_tcgen05(a: torch.Tensor, b_nk: torch.Tensor, status: torch.Tensor, epilogue: str = "bf16",
                 n_out: int = 0, clip: float = 60.0, pairs: bool = True) -> torch.Tensor:
    """``a [M, K] @ b_nk [N, K]^T`` on the tcgen05 tensor cores (bfloat16 in, float32 accumulate).

    ``epilogue``: ``"bf16"`` / ``"f32"`` store the product; ``"silu_mul"`` expects the rows of
    ``b_nk`` interleaved in blocks of 128 gate rows and 128 up rows and stores
    ``silu(gate) * up`` as ``[M, n_out]``. ``status`` receives an error code if a block gave up.
    ``pairs``: with more than 128 rows, let pairs of SMs share each tile (tcgen05 cta_group::2) and
    deal the work out stream-K fashion; partial tiles pass through ``gemm_workspace``.
    """
    if epilogue not in GEMM_EPILOGUES:
        raise ValueError(f"unknown epilogue {epilogue!r}")
    for name, t in (("a", a), ("b_nk", b_nk)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.stride(1) != 1:
            raise ValueError(f"{name} must be a bfloat16 CUDA matrix with contiguous rows")
    _need(status, torch.int32, "status")
    m, k = a.shape
    n = b_nk.shape[0]
    if b_nk.shape[1] != k:
        raise ValueError("inner sizes differ")
    if epilogue == "silu_mul":
        out = _empty((m, n_out), torch.bfloat16, a.device)
    else:
        out = _empty((m, n), torch.float32 if epilogue == "f32" else torch.bfloat16, a.device)
    fn = _fn("gemm_tcgen05", "pkv_gemm_tcgen05",
             [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
              c_void_p, c_longlong, c_void_p, c_void_p])
    workspace = gemm_workspace(a.device) if pairs and m > 128 else None
    _check(fn(_ptr(a), a.stride(0), _ptr(b_nk), b_nk.stride(0), _ptr(out), out.stride(0), m, n, k,
              GEMM_EPILOGUES[epilogue], int(n_out), float(clip), _ptr(workspace),
              workspace.numel() if workspace is not None else 0, _ptr(status), _stream()), "gemm_tcgen05")
    return out


SMALL_M_MAX_ROWS = {"bf16": 32, "f32": 32, "silu_mul": 32}


def gemm_small_m_supports(a: torch.Tensor, b_nk: torch.Tensor, epilogue: str = "bf16") -> bool:
    """Whether the weight-streaming product for few rows takes these operands: bfloat16, at most
    ``SMALL_M_MAX_ROWS[epilogue]`` rows, an inner size that is a multiple of 32, contiguous
    weights and 16-byte aligned rows."""
    return (a.dtype == torch.bfloat16 and b_nk.dtype == torch.bfloat16 and a.dim() == 2 and b_nk.dim() == 2
            and 0 < a.shape[0] <= SMALL_M_MAX_ROWS[epilogue] and a.shape[1] % 32 == 0 and a.stride(1) == 1
            and a.stride(0) % 8 == 0 and b_nk.is_contiguous() and a.data_ptr() % 16 == 0 and b_nk.data_ptr() % 16 == 0
            and (epilogue != "silu_mul" or b_nk.shape[0] % 256 == 0))


_SMALL_M_WORKSPACE: dict[str, torch.Tensor] = {}


def _small_m_workspace(device: torch.device) -> torch.Tensor:
    """Partial sums and tile counters of ``gemm_small_m`` on a device: allocated and zeroed once,
    left zero by every launch, shared by the launches of a stream."""
    _one_stream(device)
    key = _device_key(device)
    if key not in _SMALL_M_WORKSPACE:
        lib = library("gemm_small_m")
        lib.pkv_gemm_small_m_workspace_bytes.restype = c_longlong
        _SMALL_M_WORKSPACE[key] = torch.zeros((int(lib.pkv_gemm_small_m_workspace_bytes()),), dtype=torch.uint8, device=device)
    return _SMALL_M_WORKSPACE[key]


def gemm_small_m(a: torch.Tensor, b_nk: torch.Tensor, epilogue: str = "bf16", n_out: int = 0, clip: float = 60.0,
                 chained: bool = True, residual: tuple[torch.Tensor, torch.Tensor] | None = None,
                 row_norm: tuple[torch.Tensor, float] | None = None, rope_kv: tuple | None = None):
    """``a [M, K] @ b_nk [N, K]^T`` for the few rows of a decode step: the weights stream from
    memory through registers into ``mma.sync`` (bfloat16 in, float32 accumulate), every weight
    read once. Epilogues as in ``gemm_tcgen05``. ``chained`` launches the kernel as a programmatic
    dependent of the one before it on the stream, so that it requests its first weights while
    that kernel is still running; it reads ``a`` only after that kernel has finished.

    ``residual = (hidden, norm_weight)`` (instead of an epilogue): the product is added to the
    float32 stream ``hidden [M, N]`` in place; returned are ``hidden * norm_weight`` in bfloat16 and
    the sums of squares of the new stream per 16-column tile and row, ``[ceil(N / 16), 32]``.
    ``row_norm = (sumsq, eps)`` with such sums: ``a`` is taken to be such a weighted stream and the
    rows of the result are divided by ``sqrt(sum / K + eps)``. The two together are a residual add,
    an RMS norm and the next product in two launches instead of three.

    ``rope_kv = (positions, cos, sin, k_pool, v_pool, slots, n_heads, n_kv, head_dim, page_size)``
    (instead of an epilogue): ``b_nk`` is a fused query/key/value projection; what
    ``rope_kv_store`` would do to the product happens in the epilogue, and the result ``[M, N]``
    holds the rotated queries (its key and value columns are not written)."""
    if residual is not None:
        epilogue = "residual"
    if rope_kv is not None:
        epilogue = "rope_kv"
    if epilogue not in GEMM_EPILOGUES and epilogue not in ("residual", "rope_kv"):
        raise ValueError(f"unknown epilogue {epilogue!r}")
    for name, t in (("a", a), ("b_nk", b_nk)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.stride(1) != 1:
            raise ValueError(f"{name} must be a bfloat16 CUDA matrix with contiguous rows")
    if not b_nk.is_contiguous():
        raise ValueError("b_nk must be contiguous")
    m, k = a.shape
    n = b_nk.shape[0]
    if b_nk.shape[1] != k:
        raise ValueError("inner sizes differ")
    hidden = weight = sumsq_out = sumsq_in = None
    parts, eps = 0, 0.0
    if residual is not None:
        hidden, weight = residual
        _need(hidden, torch.float32, "hidden"); _need(weight, torch.float32, "norm weight")
        if hidden.shape != (m, n) or weight.numel() != n:
            raise ValueError("the residual epilogue needs a stream and a norm weight as wide as the product")
        sumsq_out = _empty((-(-n // 16), 32), torch.float32, a.device)
    if row_norm is not None:
        sumsq_in, eps = row_norm
        _need(sumsq_in, torch.float32, "sums of squares")
        if sumsq_in.dim() != 2 or sumsq_in.shape[1] != 32:
            raise ValueError("sums of squares must be [parts, 32]")
        parts = sumsq_in.shape[0]
    positions = cos = sin = k_pool = v_pool = slots = None
    n_heads = n_kv = head_dim = page_size = 0
    if rope_kv is not None:
        positions, cos, sin, k_pool, v_pool, slots, n_heads, n_kv, head_dim, page_size = rope_kv
        _need(positions, torch.int32, "positions"); _need(k_pool, torch.bfloat16, "k_pool"); _need(v_pool, torch.bfloat16, "v_pool")
        if cos is not None:
            _need(cos, torch.float32, "cos"); _need(sin, torch.float32, "sin")
            if cos.shape[1] != head_dim // 2:
                raise ValueError("rotary tables must be [positions, head_dim/2]")
        if slots is not None:
            _need(slots, torch.int32, "slots")
        if n != (n_heads + 2 * n_kv) * head_dim or positions.numel() < m:
            raise ValueError("the projection's rows do not match (n_heads + 2*n_kv) * head_dim, or positions are missing")
    if epilogue == "silu_mul":
        out = _empty((m, n_out), torch.bfloat16, a.device)
    else:
        out = _empty((m, n), torch.float32 if epilogue == "f32" else torch.bfloat16, a.device)
    fn = _fn("gemm_small_m", "pkv_gemm_small_m",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
              c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
              c_void_p, c_void_p])
    workspace = _small_m_workspace(a.device)
    num_slots = k_pool.shape[0] * int(page_size) if k_pool is not None else 0
    max_pos = cos.shape[0] if cos is not None else 0
    code = {"residual": 3, "rope_kv": 4}.get(epilogue) or GEMM_EPILOGUES[epilogue]
    _check(fn(_ptr(a), _ptr(b_nk), _ptr(out), m, n, k, a.stride(0), code, int(n_out), float(clip),
              1 if chained else 0, _ptr(workspace), workspace.numel(), _ptr(hidden), _ptr(weight), _ptr(sumsq_out),
              _ptr(sumsq_in), parts, k, float(eps), _ptr(positions), _ptr(cos), _ptr(sin), _ptr(k_pool), _ptr(v_pool),
              _ptr(slots), int(n_heads), int(n_kv), int(head_dim), int(page_size), num_slots, max_pos,
              _ptr(status_word(a.device)) if rope_kv is not None else None, _stream()), "gemm_small_m")
    return (out, sumsq_out) if residual is not None else out


STREAM_MAX_ROWS = 128
_STREAM_WORKSPACE: dict[str, torch.Tensor] = {}


def gemm_stream_supports(a: torch.Tensor, b_nk: torch.Tensor, epilogue: str = "bf16") -> bool:
    """Whether the tcgen05 weight-streaming product takes these operands: bfloat16, 1 to 128 rows, an
    inner size that is a multiple of 64, contiguous weights, 16-byte aligned rows (and, for the fused
    activation, gate and up rows interleaved in blocks of 128)."""
    return (a.dtype == torch.bfloat16 and b_nk.dtype == torch.bfloat16 and a.dim() == 2 and b_nk.dim() == 2
            and 0 < a.shape[0] <= STREAM_MAX_ROWS and a.shape[1] % 64 == 0 and a.stride(1) == 1 and a.stride(0) % 8 == 0
            and b_nk.is_contiguous() and a.data_ptr() % 16 == 0 and b_nk.data_ptr() % 16 == 0
            and (epilogue != "silu_mul" or b_nk.shape[0] % 256 == 0))


def _stream_workspace(device: torch.device) -> torch.Tensor:
    """Partial accumulators and tile counters of ``gemm_stream`` on a device: allocated and zeroed
    once, left zero by every launch, shared by the launches of a stream."""
    _one_stream(device)
    key = _device_key(device)
    if key not in _STREAM_WORKSPACE:
        lib = library("gemm_stream")
        lib.pkv_gemm_stream_workspace_bytes.restype = c_longlong
        lib.pkv_gemm_stream_workspace_bytes.argtypes = [c_int]
        size = int(lib.pkv_gemm_stream_workspace_bytes(STREAM_MAX_ROWS))
        _STREAM_WORKSPACE[key] = torch.zeros((size,), dtype=torch.uint8, device=device)
    return _STREAM_WORKSPACE[key]


def gemm_stream(a: torch.Tensor, b_nk: torch.Tensor, status: torch.Tensor, epilogue: str = "bf16", n_out: int = 0,
                clip: float = 60.0, chained: bool = True, residual: tuple[torch.Tensor, torch.Tensor] | None = None,
                row_norm: tuple[torch.Tensor, float] | None = None):
    """``a [M, K] @ b_nk [N, K]^T`` for 1 to 128 rows on the tcgen05 tensor cores with the operands
    swapped: tiles of 128 weight rows are the tall side of the MMA, the weights stream through a
    TMA ring, every weight is read once. Epilogues ``"bf16"``, ``"f32"``, ``"silu_mul"`` as in
    ``gemm_tcgen05``.

    ``residual = (hidden, norm_weight)``: the product is added to the float32 stream ``hidden
    [M, N]`` in place; returned are ``hidden * norm_weight`` in bfloat16 and the sums of squares of
    the new stream per 128-column tile and row, ``[ceil(N / 128), 128]``. ``row_norm = (sumsq,
    eps)`` with such sums ``[parts, stride]`` (this kernel's or ``gemm_small_m``'s): the rows of the
    result are divided by ``sqrt(sum / K + eps)``."""
    if residual is not None:
        epilogue = "residual"
    if epilogue not in GEMM_EPILOGUES and epilogue != "residual":
        raise ValueError(f"unknown epilogue {epilogue!r}")
    for name, t in (("a", a), ("b_nk", b_nk)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.stride(1) != 1:
            raise ValueError(f"{name} must be a bfloat16 CUDA matrix with contiguous rows")
    if not b_nk.is_contiguous():
        raise ValueError("b_nk must be contiguous")
    _need(status, torch.int32, "status")
    m, k = a.shape
    n = b_nk.shape[0]
    if b_nk.shape[1] != k:
        raise ValueError("inner sizes differ")
    hidden = weight = sumsq_out = sumsq_in = None
    parts, in_stride, eps = 0, 0, 0.0
    if residual is not None:
        hidden, weight = residual
        _need(hidden, torch.float32, "hidden"); _need(weight, torch.float32, "norm weight")
        if hidden.shape != (m, n) or weight.numel() != n:
            raise ValueError("the residual epilogue needs a stream and a norm weight as wide as the product")
        sumsq_out = _empty((-(-n // 128), 128), torch.float32, a.device)
    if row_norm is not None:
        sumsq_in, eps = row_norm
        _need(sumsq_in, torch.float32, "sums of squares")
        if sumsq_in.dim() != 2 or sumsq_in.shape[1] < m:
            raise ValueError("sums of squares must be [parts, at least as many columns as rows]")
        parts, in_stride = sumsq_in.shape
    if epilogue == "silu_mul":
        out = _empty((m, n_out), torch.bfloat16, a.device)
    else:
        out = _empty((m, n), torch.float32 if epilogue == "f32" else torch.bfloat16, a.device)
    fn = _fn("gemm_stream", "pkv_gemm_stream",
             [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_longlong,
              c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    workspace = _stream_workspace(a.device)
    code = 3 if epilogue == "residual" else GEMM_EPILOGUES[epilogue]
    _check(fn(_ptr(a), a.stride(0), _ptr(b_nk), _ptr(out), m, n, k, code, int(n_out), float(clip), 1 if chained else 0,
              _ptr(workspace), workspace.numel(), _ptr(hidden), _ptr(weight), _ptr(sumsq_out),
              sumsq_out.shape[1] if sumsq_out is not None else 0, _ptr(sumsq_in), parts, in_stride, k, float(eps),
              _ptr(status), _stream()), "gemm_stream")
    return (out, sumsq_out) if residual is not None else out


def finish_norm(xw: torch.Tensor, sumsq: torch.Tensor, eps: float) -> torch.Tensor:
    """The RMS-normalised rows from the two pieces that ``gemm_small_m(..., residual=...)`` or
    ``gemm_stream(..., residual=...)`` leaves (``sumsq [parts, stride]``):
    ``xw / sqrt(sum(sumsq) / width + eps)``, bfloat16."""
    _need(xw, torch.bfloat16, "xw"); _need(sumsq, torch.float32, "sums of squares")
    rows, d = xw.shape
    out = _empty(xw.shape, xw.dtype, xw.device)
    fn = _fn("elementwise", "pkv_finish_norm", [c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(xw), _ptr(sumsq), sumsq.shape[0], sumsq.shape[1], float(eps), _ptr(out), rows, d, _stream()), "finish_norm")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, uniform: torch.Tensor,
           greedy_below: float, probs: torch.Tensor | None = None, status: torch.Tensor | None = None,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """One token id per row of ``logits [R, V]`` (float32); ``uniform`` is float64, one per row.
    With ``status`` (the device's status word) the result has ``R + 1`` elements and the last is
    the word's value after every earlier kernel on the stream has finished. ``out`` (int32, at
    least that many elements) receives the result in place of a fresh tensor."""
    _need(logits, torch.float32, "logits"); _need(temperature, torch.float32, "temperature")
    _need(top_p, torch.float32, "top_p"); _need(uniform, torch.float64, "uniform")
    rows, vocab = logits.shape
    if probs is None:
        probs = torch.empty((rows, vocab), dtype=torch.float32, device=logits.device)
    else:
        _need(probs, torch.float32, "probs")
        if probs.numel() < rows * vocab:
            raise ValueError("probs scratch is smaller than the logits")
    if status is not None:
        _need(status, torch.int32, "status")
    count = rows + (status is not None)
    if out is None:
        out = torch.empty((count,), dtype=torch.int32, device=logits.device)
    else:
        _need(out, torch.int32, "out")
        if out.numel() < count:
            raise ValueError("the output buffer is smaller than the rows to sample")
        out = out[:count]
    fn = _fn("sampling", "pkv_sample",
             [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p,
              c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), _ptr(temperature), _ptr(top_p), _ptr(uniform), _ptr(probs), _ptr(out),
              rows, vocab, float(greedy_below), _ptr(status), _stream()), "sample")
    return out
