"""Each kernel alone against a plain float32 reference, at other sizes than the engine's tests
use (``-m gpu``). Inputs are made so that faults show: a far key that dominates the softmax,
queries at page and window edges, unused slots filled with NaN."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_model

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tol(dtype, scale=1.0):
    return 2e-5 * scale if dtype == "float32" else 2e-2 * scale


def dev(array, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(array)).cuda()
    return t.to(dtype) if dtype is not None else t


def as_np(tensor):
    return tensor.float().cpu().numpy()


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_gather(dtype):
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(0)
    table = rng.standard_normal((1000, 200)).astype(np.float32)
    table_d = dev(table, DTYPES[dtype])
    ids = rng.integers(0, 1000, size=77).astype(np.int32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.embedding_gather(table_d, dev(ids), status)
    assert out.dtype == torch.float32
    assert np.array_equal(as_np(out), as_np(table_d)[ids])
    assert int(status.item()) == 0
    bad = ids.copy()
    bad[5] = 1000
    ops.embedding_gather(table_d, dev(bad), status)
    assert int(status.item()) == 1                      # recorded, and nothing outside the table was read


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 1000, 1001, 4096, 11008, 16384, 20000])
def test_add_rmsnorm(dtype, width):
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(width)
    hidden = (rng.standard_normal((9, width)) * 3).astype(np.float32)
    delta = rng.standard_normal((9, width)).astype(np.float32)
    weight = (1 + 0.2 * rng.standard_normal(width)).astype(np.float32)
    delta_d = dev(delta, DTYPES[dtype])
    delta_seen = as_np(delta_d)
    hidden_d = dev(hidden)
    out = ops.add_rmsnorm(hidden_d, delta_d, dev(weight), 1e-5, DTYPES[dtype])
    summed = hidden + delta_seen
    assert np.allclose(as_np(hidden_d), summed, atol=1e-6)          # the stream is updated in float32
    assert np.abs(as_np(out) - plain_model.rms_norm(summed, weight, 1e-5)).max() <= tol(dtype, 4)
    # no delta: the stream stays; rows: only those rows, stream untouched
    before = as_np(hidden_d).copy()
    rows = np.array([7, 0, 3], dtype=np.int32)
    picked = ops.add_rmsnorm(hidden_d, delta_d, dev(weight), 1e-5, DTYPES[dtype], rows=dev(rows))
    assert np.array_equal(as_np(hidden_d), before)
    want = plain_model.rms_norm(before[rows] + delta_seen[rows], weight, 1e-5)
    assert np.abs(as_np(picked) - want).max() <= tol(dtype, 4)
    plain = ops.add_rmsnorm(hidden_d, None, dev(weight), 1e-5, torch.float32)
    assert np.abs(as_np(plain) - plain_model.rms_norm(before, weight, 1e-5)).max() <= 2e-5
    assert np.array_equal(as_np(hidden_d), before)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("ff", [300, 301, 304, 14336])
def test_silu_mul(dtype, ff):
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(1)
    x = (rng.standard_normal((13, 2 * ff)) * 4).astype(np.float32)
    x[0, :4] = [-100.0, 100.0, -60.0, 60.0]
    x_d = dev(x, DTYPES[dtype])
    seen = as_np(x_d)
    out = ops.silu_mul(x_d, 60.0)
    want = plain_model.silu(seen[:, :ff]) * seen[:, ff:]
    assert np.isfinite(as_np(out)).all()
    assert np.abs(as_np(out) - want).max() <= tol(dtype, np.abs(want).max())
    # the interleaved layout: blocks of 8 (and of 128) gate columns, each followed by its up columns
    for block in (8, 128):
        padded = -(-ff // block) * block
        wide = np.zeros((13, 2 * padded), dtype=np.float32)
        cols = np.arange(ff)
        wide[:, (cols // block) * 2 * block + cols % block] = seen[:, :ff]
        wide[:, (cols // block) * 2 * block + block + cols % block] = seen[:, ff:]
        again = ops.silu_mul(dev(wide, DTYPES[dtype]), 60.0, ff=ff, interleave=block)
        assert np.array_equal(as_np(again), as_np(out))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv, hd", [(5, 5, 48), (7, 1, 20), (32, 8, 128), (4, 2, 8)])
def test_rope_kv_store(dtype, heads, kv, hd):
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(2)
    page, pages, tokens = 4, 9, 11
    cos, sin = plain_model.rope_tables(64, hd, 1234.5)
    qkv = rng.standard_normal((tokens, (heads + 2 * kv) * hd)).astype(np.float32)
    positions = rng.integers(0, 64, size=tokens).astype(np.int32)
    slots = rng.permutation(pages * page)[:tokens].astype(np.int32)
    slots[3] = -1
    qkv_d = dev(qkv, DTYPES[dtype])
    seen = as_np(qkv_d).copy()
    k_pool = torch.full((pages, kv, page, hd), float("nan"), dtype=DTYPES[dtype], device="cuda")
    v_pool = torch.full((pages, kv, page, hd), float("nan"), dtype=DTYPES[dtype], device="cuda")
    ops.rope_kv_store(qkv_d, dev(positions), dev(cos), dev(sin), k_pool, v_pool, dev(slots), heads, kv, hd, page)
    q = seen[:, :heads * hd].reshape(tokens, heads, hd)
    k = seen[:, heads * hd:(heads + kv) * hd].reshape(tokens, kv, hd)
    v = seen[:, (heads + kv) * hd:].reshape(tokens, kv, hd)
    q_rot = plain_model.apply_rope(q, positions, cos, sin)
    k_rot = plain_model.apply_rope(k, positions, cos, sin)
    got_q = as_np(qkv_d)[:, :heads * hd].reshape(tokens, heads, hd)
    assert np.abs(got_q - q_rot).max() <= tol(dtype, 4)
    assert np.array_equal(as_np(qkv_d)[:, heads * hd:], seen[:, heads * hd:])      # k, v columns are only read
    kp, vp = as_np(k_pool), as_np(v_pool)
    written = np.zeros((pages, page), dtype=bool)
    for t in range(tokens):
        if slots[t] < 0:
            continue
        p, o = divmod(int(slots[t]), page)
        written[p, o] = True
        assert np.abs(kp[p, :, o] - k_rot[t]).max() <= tol(dtype, 4)
        assert np.abs(vp[p, :, o] - v[t]).max() <= tol(dtype, 1e-3)
    untouched = np.broadcast_to(~written[:, None, :], (pages, kv, page))
    assert np.isnan(kp[untouched]).all() and np.isnan(vp[untouched]).all()        # nothing else was touched
    # without tables: q untouched, k stored unrotated; without slots: nothing stored
    qkv_d2 = dev(qkv, DTYPES[dtype])
    ops.rope_kv_store(qkv_d2, dev(positions), None, None, k_pool, v_pool, dev(slots), heads, kv, hd, page)
    assert np.array_equal(as_np(qkv_d2), seen)
    p, o = divmod(int(slots[0]), page)
    assert np.array_equal(as_np(k_pool)[p, :, o], k[0])


def _attention_case(rng, *, heads, kv, hd, page, window, contexts, queries, dtype, spike=True, fast=False, splits=1,
                    tcgen05=False, deep_ring=True, flat_blocks=None, corrupt=None, expect_status=0):
    """Random sequences already in the cache (``contexts`` tokens each), of which the last
    ``queries`` tokens are this step's queries. Returns device inputs and the plain answer.
    ``corrupt = (sequence, table entry, value)`` puts ``value`` (no page of the pool) into that
    sequence's block table; the plain answer then has zeros for the keys and values of that page,
    which is how a kernel must read an entry it cannot use."""
    from paged_kv_serving_b200 import ops

    torch_dtype = DTYPES[dtype]
    total_pages = sum(-(-c // page) for c in contexts) + 3
    order = rng.permutation(total_pages)
    k_pool = torch.full((total_pages, kv, page, hd), float("nan"), dtype=torch_dtype, device="cuda")
    v_pool = torch.full((total_pages, kv, page, hd), float("nan"), dtype=torch_dtype, device="cuda")
    tables, q_rows, wants, starts, firsts = [], [], [], [0], []
    width = max(-(-c // page) for c in contexts)
    used = 0
    for context, n_q in zip(contexts, queries):
        q = rng.standard_normal((context, heads, hd)).astype(np.float32)
        k = rng.standard_normal((context, kv, hd)).astype(np.float32)
        v = rng.standard_normal((context, kv, hd)).astype(np.float32)
        if spike and context > 40:
            # one far key stands out for the last query: dropping or misplacing it changes the answer
            far = 3 if window is None else max(0, context - window)
            k[far, :, :] = 0.0
            k[far, :, 0] = 6.0
            q[context - 1, :, 0] = 6.0
        q = torch.from_numpy(q).to(torch_dtype).float().numpy()
        k = torch.from_numpy(k).to(torch_dtype).float().numpy()
        v = torch.from_numpy(v).to(torch_dtype).float().numpy()
        n_pages = -(-context // page)
        table = order[used:used + n_pages]
        used += n_pages
        for position in range(context):
            p, o = table[position // page], position % page
            k_pool[p, :, o] = torch.from_numpy(k[position]).to(torch_dtype).cuda()
            v_pool[p, :, o] = torch.from_numpy(v[position]).to(torch_dtype).cuda()
        tables.append(np.concatenate([table, np.full(width - n_pages, -1)]))
        if corrupt is not None and corrupt[0] == len(tables) - 1:
            tables[-1][corrupt[1]] = corrupt[2]
            k[corrupt[1] * page:(corrupt[1] + 1) * page] = 0.0
            v[corrupt[1] * page:(corrupt[1] + 1) * page] = 0.0
        full = plain_model.causal_attention(q, k, v, 1.0 / math.sqrt(hd), window=window)
        wants.append(full[context - n_q:].reshape(n_q, heads * hd))
        q_rows.append(q[context - n_q:].reshape(n_q, heads * hd))
        starts.append(starts[-1] + n_q)
        firsts.append(context - n_q)
    q_all = np.concatenate(q_rows)
    qkv = np.concatenate([q_all, np.full((q_all.shape[0], 2 * kv * hd), np.nan, dtype=np.float32)], axis=1)
    group = heads // kv
    if fast:
        block_rows, decode_rows = ops.attention_bf16_rows()
        if tcgen05:
            block_rows = ops.attention_tcgen05_rows()
        out = torch.full((q_all.shape[0], heads * hd), float("nan"), dtype=torch_dtype, device="cuda")
        small = [s for s, n_q in enumerate(queries) if n_q * group <= decode_rows]
        large = [(s, q0) for s, n_q in enumerate(queries) if n_q * group > decode_rows for q0 in range(0, n_q, block_rows)]
        common = (dev(np.stack(tables).astype(np.int32)), dev(np.asarray(starts, dtype=np.int32)),
                  dev(np.asarray(firsts, dtype=np.int32)))
        qkv_d = dev(qkv, torch_dtype)
        if large and tcgen05:
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            ops.attention_prefill_tcgen05(qkv_d, out, k_pool, v_pool, *common,
                                          dev(np.asarray([s for s, _ in large], dtype=np.int32)),
                                          dev(np.asarray([q for _, q in large], dtype=np.int32)),
                                          heads, kv, hd, page, window or 0, 1.0 / math.sqrt(hd), status)
            assert int(status.item()) == expect_status
        elif large:
            ops.attention_prefill_bf16(qkv_d, out, k_pool, v_pool, *common,
                                       dev(np.asarray([s for s, _ in large], dtype=np.int32)),
                                       dev(np.asarray([q for _, q in large], dtype=np.int32)),
                                       heads, kv, hd, page, window or 0, 1.0 / math.sqrt(hd))
        if small and flat_blocks:
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            hi = np.asarray([contexts[s] for s in small])
            lo = np.asarray([max(0, contexts[s] - queries[s] - window + 1) if window else 0 for s in small])
            units = np.concatenate([[0], np.cumsum((hi - 1) // 64 - lo // 64 + 1)])
            for _ in range(2):      # twice: the arrival counters must be back at zero
                out[:] = float("nan")
                ops.attention_decode_flat(qkv_d, out, k_pool, v_pool, *common, dev(np.asarray(small, dtype=np.int32)),
                                          dev(units.astype(np.int32)), max(queries[s] for s in small), heads, kv, hd,
                                          page, window or 0, 1.0 / math.sqrt(hd), flat_blocks, status)
            assert int(status.item()) == expect_status
        elif small and tcgen05 and ops.attention_decode_tma_supports(hd, page, qkv.shape[1]):
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            ops.attention_decode_tma(qkv_d, out, k_pool, v_pool, *common, dev(np.asarray(small, dtype=np.int32)),
                                     max(queries[s] for s in small), heads, kv, hd, page, window or 0,
                                     1.0 / math.sqrt(hd), splits, status, deep_ring=deep_ring)
            assert int(status.item()) == expect_status
        elif small:
            scratch = torch.full((q_all.shape[0] * heads * splits * (hd + 2),), float("nan"), device="cuda")
            ops.attention_decode_bf16(qkv_d, out, k_pool, v_pool, *common, dev(np.asarray(small, dtype=np.int32)),
                                      max(queries[s] for s in small), heads, kv, hd, page, window or 0,
                                      1.0 / math.sqrt(hd), splits, scratch if splits > 8 else None)
        return as_np(out), np.concatenate(wants)
    rows_per_block = ops.attention_rows_per_block()
    work_seq, work_row0 = [], []
    for s, n_q in enumerate(queries):
        for row0 in range(0, n_q * group, rows_per_block):
            work_seq.append(s)
            work_row0.append(row0)
    out = ops.paged_attention_generic(
        dev(qkv, torch_dtype), k_pool, v_pool, dev(np.stack(tables).astype(np.int32)),
        dev(np.asarray(starts, dtype=np.int32)), dev(np.asarray(firsts, dtype=np.int32)),
        dev(np.asarray(work_seq, dtype=np.int32)), dev(np.asarray(work_row0, dtype=np.int32)),
        heads, kv, hd, page, window or 0, 1.0 / math.sqrt(hd))
    return as_np(out), np.concatenate(wants)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv, hd, page", [(8, 1, 16, 1), (6, 2, 48, 4), (3, 3, 128, 16), (16, 2, 256, 8),
                                                   (9, 3, 80, 5)])
def test_paged_attention_generic(dtype, heads, kv, hd, page):
    rng = np.random.default_rng(hd + page)
    got, want = _attention_case(rng, heads=heads, kv=kv, hd=hd, page=page, window=None,
                                contexts=[300, 1, 65, 33, 128], queries=[1, 1, 65, 2, 17], dtype=dtype)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol(dtype, 2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 32, 33, 100])
def test_paged_attention_window_edges(dtype, window):
    rng = np.random.default_rng(window)
    got, want = _attention_case(rng, heads=4, kv=2, hd=32, page=8, window=window,
                                contexts=[200, 64, 31], queries=[1, 64, 31], dtype=dtype)
    assert np.abs(got - want).max() <= tol(dtype, 2)


@pytest.mark.parametrize("splits", [1, 3, 8, 11])
@pytest.mark.parametrize("heads, kv, hd, page", [(8, 1, 16, 1), (6, 2, 48, 4), (3, 3, 128, 16), (32, 8, 128, 16),
                                                   (16, 2, 64, 8), (9, 3, 80, 5), (4, 4, 112, 3), (8, 4, 32, 16),
                                                   (10, 2, 96, 7)])
def test_attention_bf16_tensor_core_kernels(heads, kv, hd, page, splits):
    """The prefill kernel (long runs of queries, block edges at 64 and 65 queries, a run that
    starts deep inside the context) and the split-KV decode kernel (one to a few queries) in
    one ragged batch, against the plain implementation."""
    rng = np.random.default_rng(hd * page + splits)
    got, want = _attention_case(rng, heads=heads, kv=kv, hd=hd, page=page, window=None,
                                contexts=[300, 1, 65, 33, 128, 200, 64, 513], queries=[1, 1, 65, 2, 17, 150, 64, 1],
                                dtype="bfloat16", fast=True, splits=splits)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol("bfloat16", 2)


@pytest.mark.parametrize("narrow", [False, True])
@pytest.mark.parametrize("heads, kv, hd, page", [(32, 8, 128, 16), (3, 3, 128, 8), (16, 2, 64, 8), (4, 4, 64, 32),
                                                   (6, 1, 128, 128), (5, 5, 128, 64), (4, 2, 128, 32)])
def test_attention_tcgen05_prefill(heads, kv, hd, page, narrow):
    """The tcgen05/TMA prefill kernel: runs of 17 to 513 queries, block edges at 128 and 129
    queries, a run deep inside its context, partial last pages filled with NaN, one far key that
    dominates the last query; short entries go to the decode kernel in the same batch. With head
    size 128 a page arrives as one copy over both 64-column panels, or (``narrow``) as one copy
    per panel."""
    from paged_kv_serving_b200 import ops

    assert ops.attention_tcgen05_supports(hd, page, (heads + 2 * kv) * hd)
    assert not ops.attention_tcgen05_supports(48, 16, 144) and not ops.attention_tcgen05_supports(128, 4, 384)
    if narrow and hd != 128:
        pytest.skip("head size 64 has one panel: the two forms are the same")
    rng = np.random.default_rng(hd + page)
    before = ops.attention_tcgen05_narrow_boxes(narrow)
    try:
        got, want = _attention_case(rng, heads=heads, kv=kv, hd=hd, page=page, window=None,
                                    contexts=[300, 1, 129, 33, 128, 700, 513, 1000], queries=[100, 1, 129, 17, 128, 150, 513, 2],
                                    dtype="bfloat16", fast=True, splits=2, tcgen05=True)
    finally:
        ops.attention_tcgen05_narrow_boxes(before)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol("bfloat16", 2)


@pytest.mark.parametrize("deep_ring", [True, False])
@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("heads, kv, hd, page", [(32, 8, 128, 16), (3, 3, 128, 8), (16, 2, 64, 8), (4, 4, 64, 32),
                                                   (8, 1, 128, 64)])
def test_attention_decode_tma(heads, kv, hd, page, splits, deep_ring):
    """The TMA-fed decode kernel alone: one to a few queries per entry over contexts from 1 to
    1500 keys (more tiles than ring stages), partial last pages filled with NaN, a far key that
    dominates, splits merged inside a cluster."""
    from paged_kv_serving_b200 import ops

    assert ops.attention_decode_tma_supports(hd, page, (heads + 2 * kv) * hd)
    group = heads // kv
    few = max(1, 16 // group)
    rng = np.random.default_rng(hd + page + splits)
    got, want = _attention_case(rng, heads=heads, kv=kv, hd=hd, page=page, window=None,
                                contexts=[300, 1, 65, 1500, 128, 64, 513, 1000], queries=[1, 1, few, 1, min(few, 2), 1, 1, few],
                                dtype="bfloat16", fast=True, splits=splits, tcgen05=True, deep_ring=deep_ring)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol("bfloat16", 2)


@pytest.mark.parametrize("blocks", [1, 3, 7, 40, 296, 5000])
@pytest.mark.parametrize("heads, kv, hd, page", [(32, 8, 128, 16), (8, 8, 128, 64), (12, 4, 64, 8), (16, 1, 64, 32)])
def test_attention_decode_flat(heads, kv, hd, page, blocks):
    """The even-shares decode kernel alone, with ranges that begin and end inside an (entry,
    head) pair, cover several pairs, or are empty: contexts from 1 to 1500 keys, partial last
    pages filled with NaN, a far key that dominates; run twice on the same counters."""
    from paged_kv_serving_b200 import ops

    assert ops.attention_decode_flat_supports(hd, page, (heads + 2 * kv) * hd)
    group = heads // kv
    few = max(1, 16 // group)
    rng = np.random.default_rng(hd + page + blocks)
    got, want = _attention_case(rng, heads=heads, kv=kv, hd=hd, page=page, window=None,
                                contexts=[300, 1, 65, 1500, 128, 64, 513, 1000], queries=[1, 1, few, 1, min(few, 2), 1, 1, few],
                                dtype="bfloat16", fast=True, flat_blocks=blocks)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol("bfloat16", 2)


@pytest.mark.parametrize("window", [1, 63, 64, 65, 300])
def test_attention_decode_flat_window_edges(window):
    rng = np.random.default_rng(window)
    got, want = _attention_case(rng, heads=4, kv=2, hd=64, page=8, window=window,
                                contexts=[400, 128, 31, 640, 65], queries=[1, 2, 1, 8, 1],
                                dtype="bfloat16", fast=True, flat_blocks=5)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol("bfloat16", 2)


@pytest.mark.parametrize("window", [1, 63, 64, 65, 300])
def test_attention_decode_tma_window_edges(window):
    rng = np.random.default_rng(window)
    got, want = _attention_case(rng, heads=4, kv=2, hd=64, page=8, window=window,
                                contexts=[400, 128, 31, 640, 65], queries=[1, 2, 1, 8, 1],
                                dtype="bfloat16", fast=True, splits=2, tcgen05=True)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol("bfloat16", 2)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("window", [1, 63, 128, 129, 300])
def test_attention_tcgen05_prefill_window_edges(window, hd):
    rng = np.random.default_rng(window)
    got, want = _attention_case(rng, heads=4, kv=2, hd=hd, page=8, window=window,
                                contexts=[400, 128, 31, 640], queries=[200, 128, 31, 300],
                                dtype="bfloat16", fast=True, splits=2, tcgen05=True)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol("bfloat16", 2)


@pytest.mark.parametrize("window", [1, 7, 63, 64, 65, 100])
def test_attention_bf16_tensor_core_kernels_window_edges(window):
    rng = np.random.default_rng(window)
    got, want = _attention_case(rng, heads=4, kv=2, hd=32, page=8, window=window,
                                contexts=[200, 64, 31, 140, 300], queries=[1, 64, 31, 3, 130],
                                dtype="bfloat16", fast=True, splits=2)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol("bfloat16", 2)


@pytest.mark.parametrize("kernel", ["generic", "mma", "tma", "flat", "tcgen05"])
def test_attention_kernels_at_a_long_context(kernel):
    """One sequence of 40,000 cached tokens (2,500 pages in shuffled order): the last token's
    decode step, and for the prefill kernel the last 128 positions as one portion. One key near
    the beginning and one near the end stand out for every query, so a tile that is dropped, read
    twice or taken from the wrong page changes the answer; the plain answer is computed for the
    queried rows only."""
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(40)
    heads, kv, hd, page, context = 4, 2, 128, 16, 40_000
    n_q = 128 if kernel == "tcgen05" else 1
    pages = context // page
    order = rng.permutation(pages + 5)[:pages]
    k = rng.standard_normal((context, kv, hd)).astype(np.float32) * 0.5
    v = rng.standard_normal((context, kv, hd)).astype(np.float32)
    q = rng.standard_normal((n_q, heads, hd)).astype(np.float32) * 0.5
    for far in (37, context - 300):
        k[far] = 0.0
        k[far, :, 0] = 5.0
    q[:, :, 0] = 5.0
    k, v, q = (torch.from_numpy(t).to(torch.bfloat16).float().numpy() for t in (k, v, q))
    k_pool = torch.zeros((pages + 5, kv, page, hd), dtype=torch.bfloat16, device="cuda")
    v_pool = torch.zeros_like(k_pool)
    k_pool[torch.from_numpy(order).cuda()] = torch.from_numpy(k).to(torch.bfloat16).cuda().view(pages, page, kv, hd).transpose(1, 2)
    v_pool[torch.from_numpy(order).cuda()] = torch.from_numpy(v).to(torch.bfloat16).cuda().view(pages, page, kv, hd).transpose(1, 2)
    scale = 1.0 / math.sqrt(hd)
    want = np.zeros((n_q, heads, hd), dtype=np.float32)
    for row in range(n_q):
        visible = context - n_q + row + 1
        for h in range(heads):
            scores = (k[:visible, h // (heads // kv)] @ q[row, h]) * np.float32(scale)
            weights = np.exp(scores - scores.max())
            want[row, h] = (weights / weights.sum()) @ v[:visible, h // (heads // kv)]
    want = want.reshape(n_q, heads * hd)
    qkv = np.concatenate([q.reshape(n_q, heads * hd), np.zeros((n_q, 2 * kv * hd), dtype=np.float32)], axis=1)
    qkv_d = dev(qkv, torch.bfloat16)
    table, starts, first = dev(order[None, :].astype(np.int32)), dev(np.asarray([0, n_q], dtype=np.int32)), \
        dev(np.asarray([context - n_q], dtype=np.int32))
    out = torch.full((n_q, heads * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    one = dev(np.asarray([0], dtype=np.int32))
    if kernel == "generic":
        rows = ops.attention_rows_per_block()
        work = np.arange(0, n_q * (heads // kv), rows, dtype=np.int32)
        out = ops.paged_attention_generic(qkv_d, k_pool, v_pool, table, starts, first, dev(np.zeros_like(work)), dev(work),
                                          heads, kv, hd, page, 0, scale)
    elif kernel == "mma":
        ops.attention_decode_bf16(qkv_d, out, k_pool, v_pool, table, starts, first, one, 1, heads, kv, hd, page, 0, scale, 8, None)
    elif kernel == "tma":
        ops.attention_decode_tma(qkv_d, out, k_pool, v_pool, table, starts, first, one, 1, heads, kv, hd, page, 0, scale, 8, status)
    elif kernel == "flat":
        units = dev(np.asarray([0, context // 64], dtype=np.int32))
        ops.attention_decode_flat(qkv_d, out, k_pool, v_pool, table, starts, first, one, units, 1, heads, kv, hd, page, 0, scale,
                                  64, status)
    else:
        ops.attention_prefill_tcgen05(qkv_d, out, k_pool, v_pool, table, starts, first, one, one, heads, kv, hd, page, 0, scale,
                                      status)
    assert int(status.item()) == 0
    got = as_np(out)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol("bfloat16", 2)


@pytest.mark.parametrize("kernel", ["tma", "flat", "tcgen05"])
def test_more_pools_than_the_kernels_remember_tensor_maps_for(kernel):
    """The TMA kernels keep the tensor maps of the pools they have seen (a few hundred). A process
    that has used more pools than that (many engines, one after the other) must still read keys
    from the key pool and values from the value pool: 700 pairs of small pools, one launch each,
    every answer checked."""
    from paged_kv_serving_b200 import ops

    heads, kv, hd, page = 2, 1, 64, 16
    n_q = 32 if kernel == "tcgen05" else 1
    context = 32
    scale = 1.0 / math.sqrt(hd)
    generator = torch.Generator(device="cuda").manual_seed(9)
    table = dev(np.asarray([[1, 0]], dtype=np.int32))
    starts, first = dev(np.asarray([0, n_q], dtype=np.int32)), dev(np.asarray([context - n_q], dtype=np.int32))
    one = dev(np.asarray([0], dtype=np.int32))
    units = dev(np.asarray([0, 1], dtype=np.int32))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    keep = []
    worst = 0.0
    for _ in range(700):
        k_pool = torch.randn((2, kv, page, hd), device="cuda", generator=generator).to(torch.bfloat16)
        v_pool = torch.randn((2, kv, page, hd), device="cuda", generator=generator).to(torch.bfloat16)
        keep.append((k_pool, v_pool))                      # alive, so that every pool has an address of its own
        qkv = torch.randn((n_q, (heads + 2 * kv) * hd), device="cuda", generator=generator).to(torch.bfloat16)
        out = torch.zeros((n_q, heads * hd), dtype=torch.bfloat16, device="cuda")
        if kernel == "tma":
            ops.attention_decode_tma(qkv, out, k_pool, v_pool, table, starts, first, one, 1, heads, kv, hd, page, 0, scale, 1, status)
        elif kernel == "flat":
            ops.attention_decode_flat(qkv, out, k_pool, v_pool, table, starts, first, one, units, 1, heads, kv, hd, page, 0, scale,
                                      1, status)
        else:
            ops.attention_prefill_tcgen05(qkv, out, k_pool, v_pool, table, starts, first, one, one, heads, kv, hd, page, 0, scale,
                                          status)
        keys = torch.cat([k_pool[1, 0], k_pool[0, 0]]).float()            # logical order: page 1, then page 0
        values = torch.cat([v_pool[1, 0], v_pool[0, 0]]).float()
        q = qkv[:, :heads * hd].float().view(n_q, heads, hd)
        scores = torch.einsum("qhd,kd->qhk", q, keys) * scale
        positions = torch.arange(context, device="cuda")
        visible = positions[None, :] <= (context - n_q + torch.arange(n_q, device="cuda"))[:, None]
        scores = scores.masked_fill(~visible[:, None, :], float("-inf"))
        want = torch.einsum("qhk,kd->qhd", torch.softmax(scores, dim=-1), values).reshape(n_q, heads * hd)
        worst = max(worst, float((out.float() - want).abs().max()))
    assert int(status.item()) == 0
    assert worst <= tol("bfloat16", 2), worst


@pytest.mark.parametrize("seed", range(3))
def test_attention_kernels_on_random_shapes(seed):
    """Seeded draws of head counts, groupings, head sizes, page sizes, windows, context lengths,
    query counts and split counts (also more splits than key tiles): each goes to the kernel that
    takes it (float32-arithmetic, mma.sync, or the TMA / tcgen05 pair, the even-shares decode
    kernel for steps that hold decode entries only) and is compared with the plain attention."""
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(500 + seed)
    ran = set()
    for _ in range(25):
        kv = int(rng.choice([1, 2, 3, 4, 8]))
        group = int(rng.choice([1, 2, 3, 4, 8]))
        heads = kv * group
        kind = str(rng.choice(["generic", "mma", "tensor"]))
        if kind == "generic":
            hd, page, dtype = 2 * int(rng.integers(1, 65)), int(rng.integers(1, 40)), str(rng.choice(["float32", "bfloat16"]))
        elif kind == "mma":
            hd, page, dtype = 16 * int(rng.integers(1, 9)), int(rng.choice([1, 2, 3, 4, 5, 8, 16, 24, 32])), "bfloat16"
        else:
            hd, page, dtype = int(rng.choice([64, 128])), int(rng.choice([8, 16, 32, 64, 128])), "bfloat16"
        window = None if rng.random() < 0.6 else int(rng.integers(1, 200))
        contexts = [int(rng.integers(1, 260)) for _ in range(int(rng.integers(1, 5)))]
        queries = [int(min(c, rng.choice([1, 1, 1, 2, 3, int(rng.integers(1, c + 1))]))) for c in contexts]
        case = dict(heads=heads, kv=kv, hd=hd, page=page, window=window, contexts=contexts, queries=queries, dtype=dtype,
                    spike=bool(rng.integers(0, 2)))
        splits = int(rng.integers(1, 9))
        if kind == "generic":
            got, want = _attention_case(rng, **case)
        elif kind == "mma":
            got, want = _attention_case(rng, fast=True, splits=splits, **case)
        else:
            only_decode = all(q * group <= 16 for q in queries)
            flat = int(rng.integers(1, 300)) if only_decode and rng.random() < 0.5 and \
                ops.attention_decode_flat_supports(hd, page, (heads + 2 * kv) * hd) else None
            got, want = _attention_case(rng, fast=True, tcgen05=True, splits=splits, deep_ring=bool(rng.integers(0, 2)),
                                        flat_blocks=flat, **case)
            kind = "even shares" if flat else kind
        ran.add(kind)
        assert np.isfinite(got).all(), case
        assert np.abs(got - want).max() <= tol(dtype, 2), (case, splits)
    assert {"generic", "mma", "tensor"} <= ran


def test_attention_refuses_what_it_cannot_do():
    from paged_kv_serving_b200 import ops

    z = torch.zeros((1, 3 * 258), device="cuda")
    pool = torch.zeros((1, 1, 1, 258), device="cuda")
    i = torch.zeros((1, 1), dtype=torch.int32, device="cuda")
    one = torch.zeros((2,), dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="limit"):
        ops.paged_attention_generic(z, pool, pool, i, one, one[:1], one[:1], one[:1], 1, 1, 258, 1, 0, 1.0)
    with pytest.raises(ValueError, match="size"):
        ops.paged_attention_generic(z, pool, pool, i, one, one[:1], one[:1], one[:1], 3, 2, 6, 1, 0, 1.0)
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops.silu_mul(torch.zeros(2, 4), 60.0)
    assert not ops.attention_bf16_supports(24, 72) and not ops.attention_bf16_supports(256, 768)
    assert ops.attention_bf16_supports(48, 144)
    b = torch.zeros((1, 3 * 24), dtype=torch.bfloat16, device="cuda")
    pool_b = torch.zeros((1, 1, 1, 24), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="limit"):
        ops.attention_prefill_bf16(b, b[:, :24].contiguous(), pool_b, pool_b, i, one, one[:1], one[:1], one[:1],
                                   1, 1, 24, 1, 0, 1.0)


@pytest.mark.parametrize("m, n, k", [(128, 256, 64), (1, 520, 136), (200, 1000, 72), (300, 96, 4096), (2048, 1024, 200), (1000, 4000, 1032), (2100, 2304, 72), (520, 6400, 136),
                                     (130, 1320, 120),
                                     (4200, 520, 4096)])      # row blocks walked in groups (32 and a last one of 1), 3 column blocks
@pytest.mark.parametrize("pairs", [True, False])
@pytest.mark.parametrize("epilogue", ["bf16", "f32"])
def test_gemm_tcgen05(m, n, k, epilogue, pairs):
    """The hand-written tcgen05/TMA product against a float32 product of the same bfloat16
    operands: tails in every dimension (rows, columns, inner size), one row, many tiles."""
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(m + n + k)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    b = torch.from_numpy(rng.standard_normal((n, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert ops.gemm_tcgen05_supports(a, b)
    out = ops.gemm_tcgen05(a, b, status, epilogue, pairs=pairs)
    want = a.double() @ b.double().t()
    assert int(status.item()) == 0
    scale = float(want.abs().max())
    bound = 1e-5 * scale if epilogue == "f32" else 2 ** -8 * scale
    assert float((out.double() - want).abs().max()) <= bound
    # a strided view of a wider matrix (rows 16-byte aligned) is taken as it is
    wide = torch.zeros((m, k + 8), dtype=torch.bfloat16, device="cuda")
    wide[:, :k] = a
    again = ops.gemm_tcgen05(wide[:, :k], b, status, epilogue, pairs=pairs)
    assert torch.equal(again, out)


@pytest.mark.parametrize("pairs", [True, False])
@pytest.mark.parametrize("m, ff, k", [(128, 128, 64), (257, 200, 120), (2048, 1000, 256), (3, 384, 72), (600, 3000, 520),
                                      (2048, 14336, 4096)])     # more tiles than SMs: every block takes several
def test_gemm_tcgen05_silu_mul_epilogue(m, ff, k, pairs):
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(ff)
    blocks = -(-ff // 128)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    gate = torch.from_numpy(rng.standard_normal((ff, k)).astype(np.float32) * 0.3).cuda().to(torch.bfloat16)
    up = torch.from_numpy(rng.standard_normal((ff, k)).astype(np.float32) * 0.3).cuda().to(torch.bfloat16)
    fused = torch.zeros((blocks, 2, 128, k), dtype=torch.bfloat16, device="cuda")
    for b in range(blocks):
        rows = min(128, ff - 128 * b)
        fused[b, 0, :rows] = gate[128 * b:128 * b + rows]
        fused[b, 1, :rows] = up[128 * b:128 * b + rows]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.gemm_tcgen05(a, fused.view(-1, k), status, "silu_mul", n_out=ff, pairs=pairs)
    g, u = (a.float() @ gate.float().t()).cpu().numpy(), (a.float() @ up.float().t()).cpu().numpy()
    want = plain_model.silu(g) * u
    assert int(status.item()) == 0 and out.shape == (m, ff)
    assert np.abs(as_np(out) - want).max() <= 2 ** -8 * np.abs(want).max() + 1e-6


def test_products_on_random_shapes():
    """Seeded draws of row counts, widths and inner sizes for the three product kernels and their
    fused activation epilogues, against float64 products of the same operands."""
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(77)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ran = {"few rows": 0, "streamed": 0, "tcgen05": 0, "few rows + activation": 0, "streamed + activation": 0,
           "tcgen05 + activation": 0}

    def check(kind, out, want, bound, what):
        ran[kind] += 1
        assert float((out.double() - want).abs().max()) <= bound and int(status.item()) == 0, (kind, what)

    def fused(ff, k):
        blocks = -(-ff // 128)
        gate = (torch.randn(ff, k, device="cuda") * 0.3).to(torch.bfloat16)
        up = (torch.randn(ff, k, device="cuda") * 0.3).to(torch.bfloat16)
        both = torch.zeros((blocks, 2, 128, k), dtype=torch.bfloat16, device="cuda")
        for b in range(blocks):
            rows = min(128, ff - 128 * b)
            both[b, 0, :rows] = gate[128 * b:128 * b + rows]
            both[b, 1, :rows] = up[128 * b:128 * b + rows]
        return gate, up, both.view(-1, k)

    def activation(a, gate, up):
        g, u = (a.float() @ gate.float().t()).cpu().numpy(), (a.float() @ up.float().t()).cpu().numpy()
        return torch.from_numpy(plain_model.silu(g) * u).cuda().double()

    torch.manual_seed(77)
    for _ in range(120):
        m, k = int(rng.integers(1, 33)), 32 * int(rng.integers(1, 200))
        n = int(rng.integers(1, 12000)) if rng.random() < 0.8 else int(rng.integers(9000, 40000))
        a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        b = torch.randn(n, k, device="cuda").to(torch.bfloat16)
        want = a.double() @ b.double().t()
        scale = float(want.abs().max()) + 1e-9
        for epilogue in ("bf16", "f32"):
            if ops.gemm_small_m_supports(a, b, epilogue):
                out = ops.gemm_small_m(a, b, epilogue, chained=bool(rng.integers(0, 2)))
                check("few rows", out, want, (1e-5 if epilogue == "f32" else 2 ** -8) * scale * max(1.0, (k / 2048) ** 0.5), (m, n, k))
        if k % 64 == 0 and ops.gemm_stream_supports(a, b, "bf16"):
            check("streamed", ops.gemm_stream(a, b, status, "bf16", chained=bool(rng.integers(0, 2))), want, 2 ** -8 * scale, (m, n, k))
        m2, k2, n2 = int(rng.integers(1, 3000)), 8 * int(rng.integers(8, 300)), 8 * int(rng.integers(1, 800))
        a2 = torch.randn(m2, k2, device="cuda").to(torch.bfloat16)
        b2 = torch.randn(n2, k2, device="cuda").to(torch.bfloat16)
        if ops.gemm_tcgen05_supports(a2, b2):
            want2 = a2.double() @ b2.double().t()
            for pairs in (True, False):
                check("tcgen05", ops.gemm_tcgen05(a2, b2, status, "bf16", pairs=pairs), want2,
                      2 ** -8 * (float(want2.abs().max()) + 1e-9), (m2, n2, k2, pairs))
        ff, k3, m3 = int(rng.integers(1, 4000)), 64 * int(rng.integers(1, 40)), int(rng.integers(1, 33))
        gate, up, w = fused(ff, k3)
        a3 = torch.randn(m3, k3, device="cuda").to(torch.bfloat16)
        want3 = activation(a3, gate, up)
        bound3 = 2 ** -8 * float(want3.abs().max()) + 1e-6
        if ops.gemm_small_m_supports(a3, w, "silu_mul"):
            check("few rows + activation", ops.gemm_small_m(a3, w, "silu_mul", n_out=ff), want3, bound3, (m3, ff, k3))
        if ops.gemm_stream_supports(a3, w, "silu_mul"):
            check("streamed + activation", ops.gemm_stream(a3, w, status, "silu_mul", n_out=ff), want3, bound3, (m3, ff, k3))
        if ff % 8 == 0:
            a4 = torch.randn(int(rng.integers(128, 700)), k3, device="cuda").to(torch.bfloat16)
            if ops.gemm_tcgen05_supports(a4, w):
                want4 = activation(a4, gate, up)
                check("tcgen05 + activation", ops.gemm_tcgen05(a4, w, status, "silu_mul", n_out=ff, pairs=bool(rng.integers(0, 2))),
                      want4, 2 ** -8 * float(want4.abs().max()) + 1e-6, (a4.shape[0], ff, k3))
    assert all(count > 0 for count in ran.values()), ran


def test_gemm_tcgen05_refuses_unaligned_operands():
    from paged_kv_serving_b200 import ops

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = torch.zeros((4, 36), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((16, 36), dtype=torch.bfloat16, device="cuda")
    assert not ops.gemm_tcgen05_supports(a, b)                  # rows of 72 bytes do not start on 16-byte boundaries
    with pytest.raises(ValueError, match="alignment"):
        ops.gemm_tcgen05(a, b, status)
    assert not ops.gemm_tcgen05_supports(a.float(), b.float())  # bfloat16 only
    a = torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((12, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="alignment"):          # 12 bfloat16 columns: output rows of 24 bytes
        ops.gemm_tcgen05(a, b, status, "bf16")
    assert ops.gemm_tcgen05(a, b, status, "f32").shape == (4, 12)


@pytest.mark.parametrize("chained", [True, False])
@pytest.mark.parametrize("m, n, k", [(1, 16, 32), (3, 331, 96), (8, 520, 4096), (9, 100, 160), (16, 1000, 2048), (17, 72, 1792),
                                     (32, 4096, 320), (25, 250, 64), (31, 6144, 512),
                                     # more than two waves of tiles with a nearly empty last one: even ranges of
                                     # (tile, chunk) units, tiles shared between blocks through the workspace
                                     (8, 9600, 512), (2, 16032, 128), (20, 9616, 96),
                                     # the inner size of a down projection
                                     (4, 4096, 14336), (16, 5120, 13824)])
@pytest.mark.parametrize("epilogue", ["bf16", "f32"])
def test_gemm_small_m(m, n, k, epilogue, chained):
    """The weight-streaming product of decode steps against a float64 product of the same
    operands: every row-count bucket and its edge, weight rows that are no multiple of 16, inner
    sizes that leave warps without work or with uneven shares; a row's result does not change
    with the rows beside it."""
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(m * 7 + n + k)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    b = torch.from_numpy(rng.standard_normal((n, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    assert ops.gemm_small_m_supports(a, b, epilogue)
    out = ops.gemm_small_m(a, b, epilogue, chained=chained)
    want = a.double() @ b.double().t()
    scale = float(want.abs().max())
    bound = 1e-5 * scale if epilogue == "f32" else 2 ** -8 * scale
    assert out.shape == (m, n) and float((out.double() - want).abs().max()) <= bound
    alone = ops.gemm_small_m(a[m - 1:], b, epilogue, chained=chained)
    assert torch.equal(alone[0], out[m - 1])
    wide = torch.zeros((m, k + 8), dtype=torch.bfloat16, device="cuda")
    wide[:, :k] = a
    assert torch.equal(ops.gemm_small_m(wide[:, :k], b, epilogue, chained=chained), out)


@pytest.mark.parametrize("m, ff, k", [(1, 128, 32), (8, 200, 96), (13, 1000, 256), (32, 392, 2048), (20, 3000, 544),
                                      # feed-forward widths of 8- and 13-billion-parameter models: 896 tiles are cut
                                      # into even ranges (shared tiles, workspace counters), 864 run one per block
                                      (8, 14336, 4096), (5, 13824, 5120), (16, 14336, 512), (32, 9728, 256)])
def test_gemm_small_m_silu_mul_epilogue(m, ff, k):
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(ff + m)
    blocks = -(-ff // 128)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    gate = torch.from_numpy(rng.standard_normal((ff, k)).astype(np.float32) * 0.3).cuda().to(torch.bfloat16)
    up = torch.from_numpy(rng.standard_normal((ff, k)).astype(np.float32) * 0.3).cuda().to(torch.bfloat16)
    fused = torch.zeros((blocks, 2, 128, k), dtype=torch.bfloat16, device="cuda")
    for b in range(blocks):
        rows = min(128, ff - 128 * b)
        fused[b, 0, :rows] = gate[128 * b:128 * b + rows]
        fused[b, 1, :rows] = up[128 * b:128 * b + rows]
    out = ops.gemm_small_m(a, fused.view(-1, k), "silu_mul", n_out=ff)
    g, u = (a.float() @ gate.float().t()).cpu().numpy(), (a.float() @ up.float().t()).cpu().numpy()
    want = plain_model.silu(g) * u
    assert out.shape == (m, ff)
    assert np.abs(as_np(out) - want).max() <= 2 ** -8 * np.abs(want).max() + 1e-6
    # again on the same workspace: every counter was left at zero, and the sums do not depend on timing
    assert torch.equal(ops.gemm_small_m(a, fused.view(-1, k), "silu_mul", n_out=ff), out)


@pytest.mark.parametrize("m, d, k, n", [(1, 64, 32, 48), (5, 352, 96, 100), (8, 4096, 512, 256), (13, 992, 64, 520),
                                        (32, 256, 2048, 72),
                                        # a stream wide enough for even ranges; the inner sizes of down projections
                                        (8, 9600, 64, 48), (8, 4096, 14336, 256), (3, 5120, 13824, 64)])
def test_gemm_small_m_residual_epilogue_and_row_norm(m, d, k, n):
    """Residual add, RMS norm and the next product in two launches: the first product adds itself
    to the float32 stream and leaves the stream times the norm's weight with per-tile sums of
    squares; the second divides its rows by the root mean square. Against the plain formulas,
    twice in a row on the same stream; the small kernel that completes the norm by itself too."""
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(m + d)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    b = torch.from_numpy(rng.standard_normal((d, k)).astype(np.float32) * 0.2).cuda().to(torch.bfloat16)
    nxt = torch.from_numpy(rng.standard_normal((n, d)).astype(np.float32) * 0.2).cuda().to(torch.bfloat16)
    weight = torch.from_numpy((1 + 0.1 * rng.standard_normal(d)).astype(np.float32)).cuda()
    stream = torch.from_numpy(rng.standard_normal((m, d)).astype(np.float32)).cuda()
    eps = 1e-5
    for _ in range(2):
        before = as_np(stream)
        weighted, sumsq = ops.gemm_small_m(a, b, residual=(stream, weight))
        product = (a.double() @ b.double().t()).cpu().numpy()
        want_stream = before + product
        # float32 accumulation: the rounding of a sum grows with the root of its length
        assert np.abs(as_np(stream) - want_stream).max() <= 2e-6 * max(1.0, (k / 2048) ** 0.5) * np.abs(want_stream).max()
        assert sumsq.shape == (-(-d // 16), 32)
        assert np.allclose(as_np(sumsq)[:, :m].sum(axis=0), (want_stream ** 2).sum(axis=1), rtol=1e-5)
        want_normed = plain_model.rms_norm(want_stream.astype(np.float32), as_np(weight), eps)
        normed = ops.finish_norm(weighted, sumsq, eps)
        assert np.abs(as_np(normed) - want_normed).max() <= 2 ** -7 * np.abs(want_normed).max() + 1e-6
        got = ops.gemm_small_m(weighted, nxt, "f32", row_norm=(sumsq, eps))
        want = want_normed.astype(np.float64) @ as_np(nxt).astype(np.float64).T
        assert np.abs(as_np(got) - want).max() <= 2 ** -7 * np.abs(want).max() + 1e-5


@pytest.mark.parametrize("m, h, kv, hd, k, page", [(1, 2, 1, 16, 32, 4), (5, 3, 3, 32, 96, 8), (8, 8, 2, 64, 256, 16),
                                                    (8, 32, 8, 128, 512, 16), (20, 6, 2, 48, 160, 16),
                                                    # 40 + 2 * 40 heads of 128: 960 tiles, cut into even ranges
                                                    (8, 40, 40, 128, 256, 16)])
def test_gemm_small_m_rotary_and_cache_epilogue(m, h, kv, hd, k, page):
    """The fused projection whose epilogue rotates queries and keys and writes keys and values into
    the paged pools, against the projection followed by the plain rotation; one row is not
    stored (slot -1), and a second call without slots leaves the pools alone."""
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(m + h + hd)
    n = (h + 2 * kv) * hd
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    w = torch.from_numpy(rng.standard_normal((n, k)).astype(np.float32) * 0.3).cuda().to(torch.bfloat16)
    cos, sin = plain_model.rope_tables(64, hd, 10000.0)
    positions = rng.integers(0, 64, size=m).astype(np.int32)
    pages = 2 * m // page + 3
    slots = rng.permutation(pages * page)[:m].astype(np.int32)
    if m > 1:
        slots[1] = -1
    k_pool = torch.zeros((pages, kv, page, hd), dtype=torch.bfloat16, device="cuda")
    v_pool = torch.zeros_like(k_pool)
    out = ops.gemm_small_m(a, w, rope_kv=(dev(positions), dev(cos), dev(sin), k_pool, v_pool, dev(slots), h, kv, hd, page))
    product = (a.double() @ w.double().t()).cpu().numpy().astype(np.float32)
    q = plain_model.apply_rope(product[:, :h * hd].reshape(m, h, hd), positions, cos, sin)
    kk = plain_model.apply_rope(product[:, h * hd:(h + kv) * hd].reshape(m, kv, hd), positions, cos, sin)
    vv = product[:, (h + kv) * hd:].reshape(m, kv, hd)
    bound = 2 ** -7 * np.abs(product).max()
    assert np.abs(as_np(out)[:, :h * hd].reshape(m, h, hd) - q).max() <= bound
    got_k, got_v = as_np(k_pool), as_np(v_pool)
    for row in range(m):
        if slots[row] < 0:
            continue
        pg, off = divmod(int(slots[row]), page)
        assert np.abs(got_k[pg, :, off] - kk[row]).max() <= bound
        assert np.abs(got_v[pg, :, off] - vv[row]).max() <= bound
    written = np.zeros((pages, page), dtype=bool)
    for sl in slots[slots >= 0]:
        written[divmod(int(sl), page)] = True
    untouched = ~written[:, None, :].repeat(kv, axis=1)
    assert not got_k[untouched].any() and not got_v[untouched].any(), "only the named slots are written"
    before = k_pool.clone()
    again = ops.gemm_small_m(a, w, rope_kv=(dev(positions), dev(cos), dev(sin), k_pool, v_pool, None, h, kv, hd, page))
    assert torch.equal(k_pool, before) and torch.equal(again[:, :h * hd], out[:, :h * hd])


def test_gemm_small_m_refusals():
    from paged_kv_serving_b200 import ops

    a = torch.zeros((4, 40), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((16, 40), dtype=torch.bfloat16, device="cuda")
    assert not ops.gemm_small_m_supports(a, b)                     # inner size no multiple of 32
    with pytest.raises(ValueError, match="size"):
        ops.gemm_small_m(a, b)
    a = torch.zeros((33, 64), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((512, 64), dtype=torch.bfloat16, device="cuda")
    assert not ops.gemm_small_m_supports(a, b)                     # at most 32 rows
    with pytest.raises(ValueError, match="limit"):
        ops.gemm_small_m(a, b)
    assert not ops.gemm_small_m_supports(a, b, "silu_mul")
    with pytest.raises(ValueError, match="limit"):
        ops.gemm_small_m(a, b, "silu_mul", n_out=256)
    assert not ops.gemm_small_m_supports(a[:4].float(), b.float())


def test_sampling_kernel_greedy_ties_and_distribution():
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(3)
    vocab = 1237
    logits = rng.standard_normal((6, vocab)).astype(np.float32) * 2
    logits[0, [900, 17, 400]] = 9.0                       # a tie: the lowest id wins
    logits[1, vocab - 1] = 50.0
    temperature = np.array([0.0, 1e-6, 0.8, 1.3, 0.8, 0.5], dtype=np.float32)
    top_p = np.array([1.0, 0.3, 1.0, 0.9, 0.35, 1.0], dtype=np.float32)
    logits_d = dev(logits)
    for trial in range(40):
        u = rng.random(6)
        ids = ops.sample(logits_d, dev(temperature), dev(top_p), dev(u), 1e-5).cpu().numpy()
        assert ids[0] == 17 and ids[1] == vocab - 1
        for row in range(2, 6):
            want = plain_model.sample_token(logits[row], float(temperature[row]), float(top_p[row]), float(u[row]))
            if ids[row] != want:
                # allowed only when the draw sits on a boundary of the cumulative distribution
                p = plain_model.sample_distribution(logits[row], float(temperature[row]), float(top_p[row]))
                cum = np.cumsum(p, dtype=np.float64)
                draw = u[row] * cum[-1]
                assert min(abs(cum[ids[row]] - draw), abs(cum[want] - draw)) < 1e-6, (trial, row, ids[row], want)


def test_sampling_kernel_nucleus_keeps_the_crossing_token_and_ties_by_id():
    from paged_kv_serving_b200 import ops

    vocab = 64
    logits = np.full((2, vocab), -30.0, dtype=np.float32)
    logits[0, [5, 9, 11, 40]] = np.log([0.4, 0.3, 0.2, 0.1]).astype(np.float32)
    logits[1, :8] = 0.0                                     # eight equal tokens: ids 0..3 reach 0.5
    temperature = np.array([1.0, 1.0], dtype=np.float32)
    top_p = np.array([0.65, 0.5], dtype=np.float32)
    seen = [set(), set()]
    for u in np.linspace(0.0005, 0.9995, 200):
        ids = ops.sample(dev(logits), dev(temperature), dev(top_p), dev(np.array([u, u])), 1e-5).cpu().numpy()
        for row in range(2):
            want = plain_model.sample_token(logits[row], 1.0, float(top_p[row]), float(u))
            assert ids[row] == want
            seen[row].add(int(ids[row]))
    assert seen[0] == {5, 9} and seen[1] == {0, 1, 2, 3}


def test_sampling_kernel_large_vocabulary():
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(5)
    vocab = 128256
    logits = (rng.standard_normal((3, vocab)) * 3).astype(np.float32)
    temperature = np.array([0.0, 0.7, 0.7], dtype=np.float32)
    top_p = np.array([1.0, 1.0, 0.8], dtype=np.float32)
    u = np.array([0.0, 0.37, 0.93])
    ids = ops.sample(dev(logits), dev(temperature), dev(top_p), dev(u), 1e-5).cpu().numpy()
    assert ids[0] == int(np.argmax(logits[0]))
    for row in (1, 2):
        want = plain_model.sample_token(logits[row], 0.7, float(top_p[row]), float(u[row]))
        if ids[row] != want:
            p = plain_model.sample_distribution(logits[row], 0.7, float(top_p[row]))
            cum = np.cumsum(p, dtype=np.float64)
            assert min(abs(cum[ids[row]] - u[row] * cum[-1]), abs(cum[want] - u[row] * cum[-1])) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layers, pages, kv, page, hd", [(3, 7, 2, 4, 6), (1, 4, 1, 3, 2), (5, 9, 8, 16, 128)])
def test_copy_page_copies_one_page_of_every_layer_and_nothing_else(layers, pages, kv, page, hd, dtype):
    """Copy-on-write of a cache page: one launch for both pools and all layers; pages whose bytes
    are no multiple of 16 take the narrow path."""
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(layers + hd)
    k_pool = torch.from_numpy(rng.standard_normal((layers, pages, kv, page, hd)).astype(np.float32)).cuda().to(dtype)
    v_pool = torch.from_numpy(rng.standard_normal((layers, pages, kv, page, hd)).astype(np.float32)).cuda().to(dtype)
    want_k, want_v = k_pool.clone(), v_pool.clone()
    want_k[:, pages - 2] = want_k[:, 1]
    want_v[:, pages - 2] = want_v[:, 1]
    ops.copy_page(k_pool, v_pool, 1, pages - 2)
    assert torch.equal(k_pool, want_k) and torch.equal(v_pool, want_v)
    with pytest.raises(ValueError, match="size"):
        ops.copy_page(k_pool, v_pool, 1, pages)          # outside the pool
    with pytest.raises(ValueError, match="size"):
        ops.copy_page(k_pool, v_pool, 2, 2)              # onto itself


@pytest.mark.parametrize("chained", [True, False])
@pytest.mark.parametrize("m, n, k", [(1, 128, 64), (3, 331, 192), (8, 520, 4096), (9, 100, 320), (16, 1000, 2048), (17, 72, 1792),
                                     (32, 4096, 320), (33, 250, 64), (64, 6144, 512), (65, 3000, 256), (100, 9600, 512),
                                     (128, 1024, 1024), (8, 28672, 4096), (4, 4096, 14336)])
@pytest.mark.parametrize("epilogue", ["bf16", "f32"])
def test_gemm_stream(m, n, k, epilogue, chained):
    """The tcgen05 weight-streaming product (weights as the tall operand, 1 to 128 rows) against a
    float64 product of the same operands: every row-count bucket and its edge, weight rows that
    are no multiple of 128, few and many tiles (ranges that begin and end inside a tile, settled
    through the workspace), long inner sizes; a row's result does not change with the rows beside
    it; twice on the same workspace."""
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(m * 7 + n + k)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    b = torch.from_numpy(rng.standard_normal((n, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert ops.gemm_stream_supports(a, b, epilogue)
    out = ops.gemm_stream(a, b, status, epilogue, chained=chained)
    want = a.double() @ b.double().t()
    scale = float(want.abs().max())
    bound = 1e-5 * scale if epilogue == "f32" else 2 ** -8 * scale
    assert int(status.item()) == 0
    assert out.shape == (m, n) and float((out.double() - want).abs().max()) <= bound
    assert torch.equal(ops.gemm_stream(a, b, status, epilogue, chained=chained), out)
    alone = ops.gemm_stream(a[m - 1:], b, status, epilogue, chained=chained)
    assert torch.equal(alone[0], out[m - 1])
    wide = torch.zeros((m, k + 8), dtype=torch.bfloat16, device="cuda")
    wide[:, :k] = a
    assert torch.equal(ops.gemm_stream(wide[:, :k], b, status, epilogue, chained=chained), out)
    assert int(status.item()) == 0


@pytest.mark.parametrize("m, ff, k", [(1, 128, 64), (8, 200, 192), (13, 1000, 256), (32, 392, 2048), (20, 3000, 576),
                                      (8, 14336, 4096), (64, 13824, 5120), (100, 1000, 512), (128, 2048, 256)])
def test_gemm_stream_silu_mul_epilogue(m, ff, k):
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(ff + m)
    blocks = -(-ff // 128)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    gate = torch.from_numpy(rng.standard_normal((ff, k)).astype(np.float32) * 0.3).cuda().to(torch.bfloat16)
    up = torch.from_numpy(rng.standard_normal((ff, k)).astype(np.float32) * 0.3).cuda().to(torch.bfloat16)
    fused = torch.zeros((blocks, 2, 128, k), dtype=torch.bfloat16, device="cuda")
    for b in range(blocks):
        rows = min(128, ff - 128 * b)
        fused[b, 0, :rows] = gate[128 * b:128 * b + rows]
        fused[b, 1, :rows] = up[128 * b:128 * b + rows]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.gemm_stream(a, fused.view(-1, k), status, "silu_mul", n_out=ff)
    g, u = (a.float() @ gate.float().t()).cpu().numpy(), (a.float() @ up.float().t()).cpu().numpy()
    want = plain_model.silu(g) * u
    assert int(status.item()) == 0 and out.shape == (m, ff)
    assert np.abs(as_np(out) - want).max() <= 2 ** -8 * np.abs(want).max() + 1e-6
    assert torch.equal(ops.gemm_stream(a, fused.view(-1, k), status, "silu_mul", n_out=ff), out)


@pytest.mark.parametrize("m, d, k, n", [(1, 128, 64, 48), (5, 352, 192, 100), (8, 4096, 512, 256), (13, 992, 64, 520),
                                        (32, 256, 2048, 72), (8, 4096, 14336, 256), (64, 5120, 13824, 64), (100, 640, 256, 333),
                                        (128, 384, 128, 128)])
def test_gemm_stream_residual_epilogue_and_row_norm(m, d, k, n):
    """Residual add, RMS norm and the next product in two launches, as with the kernel for few
    rows: the first product adds itself to the float32 stream and leaves the stream times the
    norm's weight with per-tile sums of squares; the second divides its rows by the root mean
    square. Against the plain formulas, twice in a row on the same stream."""
    from paged_kv_serving_b200 import ops

    rng = np.random.default_rng(m + d)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    b = torch.from_numpy(rng.standard_normal((d, k)).astype(np.float32) * 0.2).cuda().to(torch.bfloat16)
    d_pad = -(-d // 64) * 64
    nxt = torch.zeros((n, d_pad), dtype=torch.bfloat16, device="cuda")
    nxt[:, :d] = torch.from_numpy(rng.standard_normal((n, d)).astype(np.float32) * 0.2).cuda().to(torch.bfloat16)
    weight = torch.from_numpy((1 + 0.1 * rng.standard_normal(d)).astype(np.float32)).cuda()
    stream = torch.from_numpy(rng.standard_normal((m, d)).astype(np.float32)).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    eps = 1e-5
    for _ in range(2):
        before = as_np(stream)
        weighted, sumsq = ops.gemm_stream(a, b, status, residual=(stream, weight))
        product = (a.double() @ b.double().t()).cpu().numpy()
        want_stream = before + product
        assert np.abs(as_np(stream) - want_stream).max() <= 2e-6 * max(1.0, (k / 2048) ** 0.5) * np.abs(want_stream).max()
        assert sumsq.shape == (-(-d // 128), 128)
        assert np.allclose(as_np(sumsq)[:, :m].sum(axis=0), (want_stream ** 2).sum(axis=1), rtol=1e-5)
        want_normed = plain_model.rms_norm(want_stream.astype(np.float32), as_np(weight), eps)
        if d % 64 == 0:
            got = ops.gemm_stream(weighted, nxt, status, "f32", row_norm=(sumsq, eps))
            # row_norm divides by sqrt(sum / K + eps) with K the inner size of the product that reads it
            want = want_normed.astype(np.float64) @ as_np(nxt)[:, :d].astype(np.float64).T
            assert np.abs(as_np(got) - want).max() <= 2 ** -7 * np.abs(want).max() + 1e-5
    assert int(status.item()) == 0
