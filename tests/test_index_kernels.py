"""Integer-output kernels on the GPU against the oracle, bit for bit: the 2x2 max-pool
window index (first maximum wins) and the per-row argmax, including ties, signed zeros,
NaNs and odd shapes; the pooled values must also equal what the RMAX dispatch of the same
pool gives.  CPU part: the oracle's own pins for these two behaviours."""
import ctypes as C

import numpy as np
import pytest

from tinyhvm_b200 import abi

vp = C.c_void_p


def pool_inputs(planes, H, W, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((planes, H, W)).astype(np.float32)
    x[rng.random(x.shape) < 0.3] = 1.0                     # many ties inside windows
    x[rng.random(x.shape) < 0.05] = -0.0
    x[rng.random(x.shape) < 0.05] = 0.0
    if x.size > 16:
        x.ravel()[rng.integers(0, x.size, 8)] = np.nan
    return x


def oracle_pool(oracle, x):
    planes, H, W = x.shape
    y = np.empty((planes, H // 2, W // 2), np.float32)
    idx = np.empty(y.shape, np.uint8)
    oracle.lib.oracle_maxpool2x2_index(vp(x.ctypes.data), vp(y.ctypes.data), vp(idx.ctypes.data), C.c_uint32(planes), C.c_uint32(H), C.c_uint32(W))
    return y, idx


def test_oracle_pool_index_and_argmax_pins(oracle):
    x = np.array([[[1, 1, 0, 5], [1, 1, 5, 5], [2, 3, -1, -2], [4, 3, -1, -1]]], np.float32)
    y, idx = oracle_pool(oracle, x)
    assert y.tolist() == [[[1, 5], [4, -1]]] and idx.tolist() == [[[0, 1], [2, 0]]]       # ties: the first maximum wins
    rows = np.array([[0, 3, 3, 1], [2, 2, 2, 2], [-1, -5, -1, 0]], np.float32)
    out = np.empty(3, np.uint32)
    oracle.lib.oracle_argmax_rows(vp(rows.ctypes.data), C.c_uint32(3), C.c_uint32(4), vp(out.ctypes.data))
    assert out.tolist() == [1, 0, 3]


@pytest.mark.gpu
@pytest.mark.parametrize("planes,H,W", [(6, 28, 28), (16, 10, 10), (3, 7, 9), (1, 2, 2), (5, 64, 64), (2, 6, 4)])
def test_maxpool_index_matches_oracle(cuda, oracle, planes, H, W):
    x = pool_inputs(planes, H, W, seed=planes * 1000 + H * 10 + W)
    want_y, want_i = oracle_pool(oracle, x)
    n = want_y.size
    cuda.reset(0)
    bx, by, bi = cuda.upload(x), cuda.alloc(n * 4), cuda.alloc(n)
    assert cuda.lib.thvm_cuda_maxpool2x2_index(by, bi, bx, planes, H, W) == 0, cuda.last_error()
    got_y, got_i = cuda.read(by, np.float32, n), cuda.read(bi, np.uint8, n)
    assert np.array_equal(got_i, want_i.ravel())
    assert np.array_equal(got_y.view(np.uint32), want_y.ravel().view(np.uint32))
    # value half only
    by2 = cuda.alloc(n * 4)
    assert cuda.lib.thvm_cuda_maxpool2x2_index(by2, 0, bx, planes, H, W) == 0
    assert np.array_equal(cuda.read(by2, np.float32, n).view(np.uint32), got_y.view(np.uint32))
    assert cuda.last_error() == ""
    cuda.reset(0)


@pytest.mark.gpu
def test_maxpool_values_equal_the_rmax_dispatch(cuda, oracle):
    """thvm_maxpool2d is an RMAX dispatch over a [B,C,OH,OW,2,2] view (src/nn/conv.c:484-513): same values."""
    planes, H, W = 12, 8, 8
    x = np.random.default_rng(5).standard_normal((planes, H, W)).astype(np.float32)
    v = abi.view_pool(abi.view_contiguous([planes, H, W]), [2, 2], [2, 2])
    d = abi.Dispatch([abi.Leaf(x.ravel(), v)], [], [planes, H // 2, W // 2, 2, 2], reduce_axes=[3, 4], reduce_type=abi.RMAX, name="pool")
    cuda.reset(0)
    via_dispatch = cuda.run(d)
    bx, by = cuda.upload(x), cuda.alloc(via_dispatch.nbytes)
    assert cuda.lib.thvm_cuda_maxpool2x2_index(by, 0, bx, planes, H, W) == 0
    assert np.array_equal(cuda.read(by, np.float32, via_dispatch.size), via_dispatch.ravel())
    cuda.reset(0)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(1024, 10), (512, 100), (7, 1), (3, 33), (64, 1000)])
def test_argmax_rows_matches_oracle(cuda, oracle, rows, cols):
    rng = np.random.default_rng(rows + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    x[rng.random(x.shape) < 0.2] = 2.5                     # repeated maxima: the first one must win
    x[0, :] = 0.0; x[0, cols // 2] = -0.0
    if rows > 2:
        x[1, 0] = np.nan                                   # a leading NaN is never beaten
        x[2, cols - 1] = np.nan                            # a later NaN never wins
    want = np.empty(rows, np.uint32)
    oracle.lib.oracle_argmax_rows(vp(x.ctypes.data), C.c_uint32(rows), C.c_uint32(cols), vp(want.ctypes.data))
    cuda.reset(0)
    bx, bo = cuda.upload(x), cuda.alloc(rows * 4)
    assert cuda.lib.thvm_cuda_argmax_rows(bo, bx, rows, cols) == 0, cuda.last_error()
    assert np.array_equal(cuda.read(bo, np.uint32, rows), want)
    cuda.reset(0)


@pytest.mark.gpu
@pytest.mark.parametrize("shape,ties", [((4, 6, 28, 28), False), ((2, 3, 8, 8), True), ((3, 5, 10, 10), True), ((1, 2, 6, 14), False)])
def test_maxpool_backward_dispatch_is_bit_exact(cuda, oracle, shape, ties):
    """The mask-form pool gradient (src/interact/grad.c:406-425) runs on the pooling-backward kernel: same bits as
    the oracle's op-by-op evaluation, ties included (every maximum passes the gradient)."""
    import cases
    d = cases.maxpool_bwd_case(np.random.default_rng(sum(shape)), *shape, ties=ties)
    cuda.reset(0)
    got = cuda.run(d)
    assert cuda.last_plan() == "pool2x2_backward", cuda.last_plan()
    want = oracle.run(d)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert cuda.last_error() == ""
    cuda.reset(0)
