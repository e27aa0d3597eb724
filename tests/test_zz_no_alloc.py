"""The sampling entry point for callers that cannot allocate device memory (``-m gpu``).

Some users of the kernel library cannot call cudaMalloc where they sample: code that runs under
an allocator it does not own, a serving process whose pools are frozen, a plain C host program.
``pkv_sample_static_scratch`` does for them what ``pkv_sample`` does, with the work area that
``pkv_sample`` takes from its caller replaced by an array inside the library image. This test
calls it the way such a user would, through the exported C symbol with raw device pointers, and
checks it against the ordinary entry point on two calls in a row (the second call finds the
first call's leftovers in the shared work area and must not be disturbed by them).

The file sorts after every other test file on purpose: a run that stops at the first failure
has then already run everything else.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_FLOATS = 1 << 20     # PKV_SAMPLE_STATIC_FLOATS in csrc/sampling_noalloc.h


def _entry_point():
    from paged_kv_serving_b200 import ops

    fn = ops.library("sampling").pkv_sample_static_scratch
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p]
    return fn


def _call(fn, logits, temperature, top_p, uniform):
    out = torch.full((logits.shape[0],), -1, dtype=torch.int32, device="cuda")
    status = fn(logits.data_ptr(), logits.stride(0), temperature.data_ptr(), top_p.data_ptr(), uniform.data_ptr(),
                out.data_ptr(), logits.shape[0], logits.shape[1], 1e-5, torch.cuda.current_stream().cuda_stream)
    return status, out


def test_static_scratch_sampling_matches_the_ordinary_entry_point_twice_in_a_row():
    from paged_kv_serving_b200 import ops

    fn = _entry_point()
    rng = np.random.default_rng(21)
    for rows, vocab in ((6, 1237), (3, 50021)):          # two calls in a row, different shapes
        logits = torch.from_numpy((rng.standard_normal((rows, vocab)) * 2.5).astype(np.float32)).cuda()
        temperature = torch.tensor([0.0, 0.7, 1.3, 0.9, 0.7, 1.0][:rows], dtype=torch.float32, device="cuda")
        top_p = torch.tensor([1.0, 1.0, 0.9, 0.35, 0.6, 1.0][:rows], dtype=torch.float32, device="cuda")
        uniform = torch.from_numpy(rng.random(rows)).cuda()
        want = ops.sample(logits, temperature, top_p, uniform, 1e-5)
        status, got = _call(fn, logits, temperature, top_p, uniform)
        assert status == 0
        torch.cuda.synchronize()
        # the same kernel on the same inputs: the ids are equal, not merely close
        assert torch.equal(got, want), (got.tolist(), want.tolist())
        assert int(got[0]) == int(torch.argmax(logits[0]))


def test_static_scratch_sampling_refuses_more_than_its_work_area_holds():
    fn = _entry_point()
    rows, vocab = 9, 128256                              # 1,154,304 floats > 1,048,576
    assert rows * vocab > STATIC_FLOATS
    logits = torch.zeros((rows, vocab), dtype=torch.float32, device="cuda")
    ones = torch.ones((rows,), dtype=torch.float32, device="cuda")
    uniform = torch.zeros((rows,), dtype=torch.float64, device="cuda")
    status, out = _call(fn, logits, ones, ones, uniform)
    torch.cuda.synchronize()
    assert status == -5
    assert (out == -1).all()                             # nothing was launched
    status, out = _call(fn, logits[:8], ones[:8], ones[:8], uniform[:8])   # 8 rows fit exactly
    torch.cuda.synchronize()
    assert status == 0 and (out == 0).all()
