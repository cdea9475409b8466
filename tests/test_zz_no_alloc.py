"""The allocation-free entry point, thvm_cuda_channel_sums_noalloc.

Some users of this library may not allocate device memory while they run: a
host that gave the whole GPU to its own arena at start-up, a training step that
is being recorded for later replay (allocator calls are not allowed in the
recorded region), or a latency-critical loop.  For them the per-channel sum of a
[B, C, HW] tensor is available with its partial sums kept in a fixed 256 KiB
array inside the library instead of pool scratch.

Checked here, through the C ABI: on two calls in a row (different data, so stale
partials from the first call would show) the result equals what the regular entry
point (thvm_cuda_dispatch_kernel_rs on the SUM{0,2,3} dispatch) gives, within the
reduction tolerance the other GPU tests use; and a shape beyond the built-in
scratch is refused with a clear message.  Runs last so that a failure here cannot
hide the results of any other test.
"""
import ctypes as C

import numpy as np
import pytest

import cases
from tinyhvm_b200 import abi
from tinyhvm_b200.abi import SUM, Dispatch, Leaf

pytestmark = pytest.mark.gpu


def regular_path(cuda, x, B, Cc, HW):
    """SUM over axes 0,2,3 of [B,C,H,W] through the vtable entry point (pool scratch)."""
    d = Dispatch([Leaf(x, abi.view_contiguous([B, Cc, HW, 1]))], [], [B, Cc, HW, 1], [0, 2, 3], SUM)
    return cuda.run(d), cuda.last_plan()


def noalloc_path(cuda, x, B, Cc, HW):
    lib = cuda.lib
    xin = cuda.upload(x)                         # the caller owns input and output buffers
    out = cuda.alloc(Cc * 4)
    cuda.sync()
    rc = lib.thvm_cuda_channel_sums_noalloc(lib.thvm_cuda_buf_ptr(xin), lib.thvm_cuda_buf_ptr(out), B, Cc, HW,
                                            lib.thvm_cuda_stream())
    assert rc == 0, cuda.last_error()
    got = cuda.read(out, np.float32, Cc)
    cuda.reset(xin - 1)
    return got


def test_channel_sums_noalloc_matches_regular_entry_point(cuda):
    rng = np.random.default_rng(2026)
    B, Cc, HW = 32, 24, 64 * 64                  # 24 outputs x 131072 terms: the split (two-pass) path
    for call in range(2):
        x = (rng.standard_normal(B * Cc * HW) + call).astype(np.float32)
        want, plan = regular_path(cuda, x, B, Cc, HW)
        assert plan == "reduce_final", plan      # the regular path used its scratch-backed second pass
        got = noalloc_path(cuda, x, B, Cc, HW)
        exact = x.reshape(B, Cc, HW).astype(np.float64).sum(axis=(0, 2))
        floor = 4e-7 * np.sqrt(np.mean(exact ** 2))
        assert np.all(np.abs(got - exact) <= 1e-5 * np.abs(exact) + floor), f"call {call}: off the exact sums"
        assert np.all(np.abs(got - want) <= 1e-5 * np.abs(want) + floor), f"call {call}: differs from the regular entry point"
    assert cuda.last_error() == ""


def test_channel_sums_noalloc_small_and_unaligned_shapes(cuda):
    rng = np.random.default_rng(7)
    for B, Cc, HW in ((3, 5, 7), (2, 300, 33), (1, 1, 1000)):
        x = rng.standard_normal(B * Cc * HW).astype(np.float32)
        got = noalloc_path(cuda, x, B, Cc, HW)
        exact = x.reshape(B, Cc, HW).astype(np.float64).sum(axis=(0, 2))
        assert np.allclose(got, exact, rtol=1e-5, atol=1e-5), (B, Cc, HW)


def test_channel_sums_noalloc_rejects_shapes_beyond_its_scratch(cuda):
    lib = cuda.lib
    buf = cuda.alloc(16)
    p = lib.thvm_cuda_buf_ptr(buf)
    rc = lib.thvm_cuda_channel_sums_noalloc(p, p, 1, 65537, 1, lib.thvm_cuda_stream())
    assert rc == 1
    assert "exceed the built-in scratch" in cuda.last_error()
    cuda.clear_error()
    cuda.reset(buf - 1)
