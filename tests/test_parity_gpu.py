"""Parity of the CUDA path with the oracle, through the C ABI, on a B200.

Tolerances (from the stated target): integer / index outputs bit-exact; f32
elementwise bit-exact unless the chain holds EXP or LOG (device libm differs
from glibc in the last ulp: 1e-5 relative); reductions 1e-5 relative to the exact (double-accumulated) sum of the
f32 terms, which the oracle reports beside its own left-to-right f32 sum;
MUL+SUM contractions (matmul / conv) 1e-4 on the same measure.  Sums that cancel
to near zero get an absolute floor of 4e-7 x the RMS of the output tensor.
"""
import numpy as np
import pytest

import cases
from test_oracle_pins import all_cases, dtype_cast_dispatches, golden_case_list, golden_dispatches, run_chain, same, GOLDEN
from tinyhvm_b200 import abi
from tinyhvm_b200.abi import EXP, F16, F32, I32, LOG, MUL, SUM, U32

pytestmark = pytest.mark.gpu


def as_float(arr, dtype):
    if dtype == F16:
        return arr.view(np.float16).astype(np.float64)
    return arr.astype(np.float64)


def is_contraction(d):
    return d.reduce_type == SUM and len(d.ops) == 1 and d.ops[0][0] == MUL and len(d.leaves) == 2


def check(d, got, want, strict_serial=False, oracle=None):
    """Compare one dispatch's output with the oracle's under the stated tolerances.

    A re-ordered f32 SUM and the oracle's left-to-right f32 SUM are both
    roundings of the same exact sum of f32 terms.  The oracle can report that
    exact sum (accumulated in double); the CUDA result must then lie within
    1e-5 relative (1e-4 for contractions) of the EXACT sum, and within the same
    bound plus the oracle's own distance from the exact sum of the ORACLE."""
    inexact_ops = any(o[0] in (EXP, LOG) for o in d.ops)
    red_n = int(np.prod([d.full[a] for a in d.reduce_axes])) if d.reduce_type else 1
    reordered = d.reduce_type == SUM and d.out_dtype == F32 and (red_n > 64 or not strict_serial)
    if not inexact_ops and not reordered:
        assert same(got, want), f"{d.name}: not bit-exact"
        return
    g, w = as_float(got, d.out_dtype), as_float(want, d.out_dtype)
    finite = np.isfinite(w)
    assert np.array_equal(np.isnan(g), np.isnan(w)) or d.out_dtype != F32 or inexact_ops, f"{d.name}: NaN pattern differs"
    if d.out_dtype in (I32, U32):
        # only reached with EXP/LOG in the chain: a value that sits on an integer
        # boundary may truncate differently after a 1-ulp libm difference
        assert np.mean(g != w) <= 0.02, f"{d.name}: {np.mean(g != w):.3f} of the integer outputs differ"
        return
    rtol = 1e-4 if is_contraction(d) else 1e-5
    if d.out_dtype == F16:
        rtol = 1e-3                                                             # one half-precision ulp
    err = np.abs(g[finite] - w[finite])
    bound = rtol * np.abs(w[finite]) + 1e-30
    exact = None
    if reordered and oracle is not None and not d.post_start:
        _, exact = oracle.run_with_wide_sums(d)
    if exact is not None and np.all(np.isfinite(exact[finite])):
        ex = exact[finite]
        # absolute floor for outputs that cancel to near zero: a few f32 ulps of the output
        # scale; 1e-5 of it for contractions, whose 3xTF32 products carry ~2^-21 each
        floor = (1e-5 if is_contraction(d) else 4e-7) * np.sqrt(np.mean(ex ** 2))
        if not inexact_ops:          # with EXP/LOG the device terms themselves differ in the last ulp
            e_exact = np.abs(g[finite] - ex)
            b_exact = rtol * np.abs(ex) + floor + 1e-30
            assert np.all(e_exact <= b_exact), f"{d.name}: {np.max(e_exact / b_exact):.2f}x over rtol {rtol} against the exact sum"
        bound = bound + np.abs(w[finite] - ex) + floor
    else:
        rms = float(np.sqrt(np.mean(w[finite] ** 2))) if finite.any() else 0.0
        bound = bound + rtol * rms
    assert np.all(err <= bound), f"{d.name}: max excess {np.max(err / bound):.2f}x over rtol {rtol}"
    assert np.array_equal(g[~finite], w[~finite], equal_nan=True) or inexact_ops, d.name


@pytest.mark.parametrize("generic", [False, True], ids=["auto", "generic"])
def test_named_and_fuzzed_dispatches(cuda, oracle, generic):
    cuda.force_generic(generic)
    try:
        plans = {}
        for d in all_cases():
            got, want = cuda.run(d), oracle.run(d)
            check(d, got, want, strict_serial=generic, oracle=oracle)
            plans[cuda.last_plan()] = plans.get(cuda.last_plan(), 0) + 1
        print("plans used:", plans)
        assert cuda.last_error() == ""
    finally:
        cuda.force_generic(False)


def test_reference_golden_vectors_on_gpu(cuda):
    for name, chain, want, tol in golden_dispatches():
        got = run_chain(cuda, chain)
        assert np.allclose(got, want, rtol=max(tol, 1e-6), atol=max(tol, 1e-6)), (name, got, want)
    for name, d, want in dtype_cast_dispatches():
        assert same(cuda.run(d), want), name


def test_committed_fixtures_on_gpu(cuda, oracle):
    z = np.load(GOLDEN / "boundary_cases.npz")
    for key, d in golden_case_list():
        check(d, cuda.run(d), z[key], oracle=oracle)


def test_pool_contract(cuda):
    """ids ascend from the floor, fresh buffers are zero, pool_reset rewinds the counter,
    decref below the persistent floor is ignored (src/backend/cpu/pool.c:14-26)."""
    lib = cuda.lib
    a = cuda.alloc(64)
    b = cuda.alloc(1 << 20)
    assert b == a + 1
    assert not cuda.read(b, np.uint8, 1 << 20).any()
    x = np.arange(1 << 18, dtype=np.float32)
    cuda.write(b, x)
    assert np.array_equal(cuda.read(b, np.float32, 1 << 18), x)
    big = np.arange(3 << 20, dtype=np.float32)            # > 1 MiB: direct (unstaged) path
    c = cuda.upload(big)
    assert np.array_equal(cuda.read(c, np.float32, big.size), big)
    d = cuda.alloc(big.nbytes)
    lib.thvm_cuda_buf_copy(d, c, big.nbytes)
    assert np.array_equal(cuda.read(d, np.float32, big.size), big)
    lib.thvm_cuda_pool_set_persistent(a)
    lib.thvm_cuda_buf_decref(a)
    assert lib.thvm_cuda_buf_bytes(a) == 64                # persistent: still live
    lib.thvm_cuda_buf_incref(b); lib.thvm_cuda_buf_decref(b)
    assert lib.thvm_cuda_buf_bytes(b) == 1 << 20
    lib.thvm_cuda_buf_decref(b)
    assert lib.thvm_cuda_buf_bytes(b) == 0                 # freed at refcount 0
    lib.thvm_cuda_pool_set_persistent(0)
    cuda.reset(a - 1)
    assert cuda.alloc(16) == a                             # counter rewound
    cuda.reset(a - 1)
    # a kernel writes a small buffer, the host then overwrites its first element only: the rest comes from the device
    src = cuda.upload(np.arange(10, dtype=np.float32))
    small = cuda.alloc(40)
    lib.thvm_cuda_buf_copy(small, src, 40)                 # both host-only: stays a host copy
    vd = abi.view_contiguous([10])
    cuda.dispatch_ids(small, [src, src], abi.Dispatch([abi.Leaf(None, vd), abi.Leaf(None, vd)], [(abi.ADD, 0, 1)], [10]))
    cuda.write(small, np.array([100.0], dtype=np.float32))
    assert cuda.read(small, np.float32, 10).tolist() == [100.0] + [2.0 * i for i in range(1, 10)]
    cuda.reset(a - 1)
    # reads past the end of a buffer return zeros
    e = cuda.upload(np.ones(4, dtype=np.float32))
    assert cuda.read(e, np.float32, 8).tolist() == [1, 1, 1, 1, 0, 0, 0, 0]
    cuda.reset(e - 1)


def test_out_of_range_load_is_caught_not_faulted(cuda):
    """A view that addresses past its buffer reads 0 and raises the status word
    (the CPU backend would read out of bounds)."""
    v = abi.view_contiguous([8])
    d = abi.Dispatch([abi.Leaf(np.ones(4, dtype=np.float32), v)], [], [8])
    got = cuda.run(d)
    assert got.tolist() == [1, 1, 1, 1, 0, 0, 0, 0]
    assert "out of bounds" in cuda.last_error()
    cuda.clear_error()


def test_single_op_forms(cuda, oracle):
    """op_unary / op_binary / op_mm / op_reduce / contiguify / adam_step against the oracle."""
    import ctypes as C
    lib, ol = cuda.lib, oracle.lib
    rng = np.random.default_rng(5)
    vp = C.c_void_p
    x = rng.standard_normal(6 * 7).astype(np.float32)
    y = rng.standard_normal(6 * 7).astype(np.float32)
    dv = abi.view_contiguous([6, 7])
    tv = abi.view_permute(abi.view_contiguous([7, 6]), [1, 0])
    first = cuda.alloc(16)
    bx, by, bo = cuda.upload(x), cuda.upload(y), cuda.alloc(x.nbytes)
    for uop in (abi.NEG, abi.RELU, abi.SQRT, abi.EXP):
        lib.thvm_cuda_op_unary(uop, bo, C.byref(dv), F32, bx, C.byref(tv), F32)
        want = np.zeros_like(x)
        ol.oracle_op_unary(C.c_uint32(uop), vp(want.ctypes.data), C.byref(dv), C.c_uint32(F32), vp(x.ctypes.data), C.byref(tv), C.c_uint32(F32))
        got = cuda.read(bo, np.float32, x.size)
        assert np.allclose(got, want, rtol=1e-5, atol=0, equal_nan=True), uop
    for uop in (abi.ADD, abi.MUL, abi.DIV, abi.SUB, abi.MAX, abi.CMP):
        lib.thvm_cuda_op_binary(uop, bo, C.byref(dv), F32, bx, C.byref(tv), F32, by, C.byref(dv), F32)
        want = np.zeros_like(x)
        ol.oracle_op_binary(C.c_uint32(uop), vp(want.ctypes.data), C.byref(dv), C.c_uint32(F32), vp(x.ctypes.data), C.byref(tv),
                            C.c_uint32(F32), vp(y.ctypes.data), C.byref(dv), C.c_uint32(F32))
        assert same(cuda.read(bo, np.float32, x.size), want), uop
    # mm: [6,7] (transposed storage) @ [7,6]
    bv = abi.view_contiguous([7, 6])
    bm = cuda.alloc(36 * 4)
    lib.thvm_cuda_op_mm(bm, F32, bx, C.byref(tv), F32, by, C.byref(bv), F32, 6, 7, 6)
    want = np.zeros(36, dtype=np.float32)
    ol.oracle_op_mm(vp(want.ctypes.data), C.c_uint32(F32), vp(x.ctypes.data), C.byref(tv), C.c_uint32(F32), vp(y.ctypes.data),
                    C.byref(bv), C.c_uint32(F32), C.c_uint32(6), C.c_uint32(7), C.c_uint32(6))
    assert np.allclose(cuda.read(bm, np.float32, 36), want, rtol=1e-5, atol=1e-6)
    # reduce over the last dim
    br = cuda.alloc(6 * 4)
    for uop in (abi.SUM, abi.RMAX):
        lib.thvm_cuda_op_reduce(uop, br, 6, F32, bx, 42, F32, 7)
        want = np.zeros(6, dtype=np.float32)
        ol.oracle_op_reduce(C.c_uint32(uop), vp(want.ctypes.data), C.c_uint32(6), C.c_uint32(F32), vp(x.ctypes.data), C.c_uint32(F32), C.c_uint32(7))
        assert np.allclose(cuda.read(br, np.float32, 6), want, rtol=1e-6, atol=1e-6), uop
    # contiguify a transposed view
    lib.thvm_cuda_contiguify(bo, 42, bx, C.byref(tv))
    assert np.array_equal(cuda.read(bo, np.float32, 42), x.reshape(7, 6).T.ravel())
    # adam
    n = 1000
    p, g_, m, v = (rng.standard_normal(n).astype(np.float32) for _ in range(4))
    v = np.abs(v)
    ids = [cuda.upload(a) for a in (p, g_, m, v)]
    lib.thvm_cuda_adam_step(*ids, 1e-3, 0.9, 0.999, 1e-8, 0.1, 0.001, n)
    ol.oracle_adam_step(vp(p.ctypes.data), vp(g_.ctypes.data), vp(m.ctypes.data), vp(v.ctypes.data), C.c_float(1e-3), C.c_float(0.9),
                        C.c_float(0.999), C.c_float(1e-8), C.c_float(0.1), C.c_float(0.001), C.c_uint32(n))
    assert np.allclose(cuda.read(ids[0], np.float32, n), p, rtol=1e-6, atol=1e-7)
    assert same(cuda.read(ids[2], np.float32, n), m) and same(cuda.read(ids[3], np.float32, n), v)
    cuda.reset(first - 1)


def contraction_cases():
    rng = np.random.default_rng(77)
    return [
        cases.mm_case(rng, 128, 128, 128), cases.mm_case(rng, 200, 333, 150), cases.mm_case(rng, 256, 64, 512),
        cases.mm_case(rng, 130, 96, 260, ta=True), cases.mm_case(rng, 130, 96, 260, tb=True),
        cases.mm_case(rng, 64, 1024, 96), cases.mm_case(rng, 33, 4000, 40),            # few tiles, long K: split-K
        cases.conv_fprop_case(rng, 8, 16, 18, 18, 64, 3), cases.conv_fprop_case(rng, 4, 6, 14, 14, 32, 5),
        cases.conv_wgrad_case(rng, 8, 16, 18, 18, 32, 3),
        # CTA-pair kernel: >= 256 rows; 256-, 128- and 64-column tiles with ragged edges; long K (split); a wide, short
        # product computed as its transpose; convolutions with many output positions
        cases.mm_case(rng, 300, 96, 300), cases.mm_case(rng, 600, 64, 100, ta=True), cases.mm_case(rng, 512, 70, 40, tb=True),
        cases.mm_case(rng, 256, 2100, 256), cases.mm_case(rng, 40, 130, 700), cases.mm_case(rng, 1024, 256, 512),
        cases.conv_fprop_case(rng, 8, 16, 18, 18, 64, 3), cases.conv_wgrad_case(rng, 4, 32, 12, 12, 16, 3),
        # convolutions whose re-laid operands arrive by tile loads: 32 and 64 input channels, output widths 16 and 32
        cases.conv_fprop_case(rng, 2, 32, 18, 18, 64, 3), cases.conv_fprop_case(rng, 1, 64, 34, 34, 32, 3),
        cases.conv_fprop_case(rng, 4, 192, 10, 10, 32, 3), cases.conv_fprop_case(rng, 3, 32, 13, 21, 48, 3),   # long K (split), odd sizes
        cases.conv_fprop_case(rng, 2, 32, 18, 18, 256, 3), cases.conv_fprop_case(rng, 2, 64, 18, 18, 200, 3),  # two column tiles on the persistent kernel, the second ragged
        # weight gradients by tile loads over shifted copies: 32, 64 and 256 input channels (4, 2 and half a tap per CTA)
        cases.conv_wgrad_case(rng, 4, 32, 18, 18, 64, 3), cases.conv_wgrad_case(rng, 1, 64, 34, 34, 32, 3),
        cases.conv_wgrad_case(rng, 2, 256, 18, 18, 32, 3),
        cases.conv_wgrad_case(rng, 1, 32, 34, 66, 64, 3),          # output rows of 64: the gradient is read in place, two k-blocks per row
        # thin shapes on the CUDA-core kernels: many rows x few columns, and few outputs x very long K
        cases.conv_fprop_case(rng, 32, 1, 32, 32, 6, 5), cases.mm_case(rng, 5000, 40, 12), cases.mm_case(rng, 4100, 290, 27),
        cases.conv_wgrad_case(rng, 32, 1, 32, 32, 6, 5), cases.mm_case(rng, 10, 6000, 20), cases.mm_case(rng, 16, 9000, 150, ta=True),
        # a 3-channel first layer: K = 27 with 64 (four columns per load) and 50 output channels on the row kernel, its
        # weight gradient (27 x 64 outputs, long K) on the tiled slice kernel; 40 x 100 outputs do not tile: plain slice kernel
        cases.conv_fprop_case(rng, 2, 3, 50, 50, 64, 3), cases.conv_fprop_case(rng, 2, 3, 50, 50, 50, 3),
        cases.conv_wgrad_case(rng, 4, 3, 34, 34, 64, 3), cases.mm_case(rng, 40, 5000, 100),
    ]


def test_contraction_kernel(cuda, oracle):
    """MUL+SUM dispatches with separable operands run on the tcgen05 3xTF32 kernel
    and stay within 1e-4 of the exact sum (and of the oracle, up to its own rounding)."""
    plans = []
    for d in contraction_cases():
        got = cuda.run(d)
        plans.append(cuda.last_plan())
        assert cuda.last_error() == "", (d.name, cuda.last_error())
        check(d, got, oracle.run(d), oracle=oracle)
    print("plans:", plans)
    assert all(p.startswith("gemm") or p.startswith("contract_skinny") for p in plans), plans
    assert sum(p == "contract_skinny_rows" for p in plans) >= 5, plans
    assert any("splitk" in p for p in plans), plans
    assert sum(p.startswith("gemm_pair") or p.startswith("gemm_tma") for p in plans) >= 6, plans
    assert sum(p.startswith("gemm_tma") for p in plans) >= 4, plans


def test_read_back_variants(cuda):
    """buf_read_nosync hands back valid bytes on return (the reference reads metadata through it, src/interact/_.c:8-11),
    for host-written and for device-written buffers; buf_read_async delivers after thvm_cuda_sync and the library keeps a
    later overwrite of the buffer behind the copy."""
    import ctypes as C
    lib = cuda.lib
    cuda.reset(0)
    small = np.arange(8, dtype=np.float32)
    big = np.random.default_rng(3).standard_normal(1 << 20).astype(np.float32)
    bs, bb = cuda.upload(small), cuda.upload(big)
    out_s, out_b = np.zeros_like(small), np.zeros_like(big)
    lib.thvm_cuda_buf_read_nosync(bs, out_s.ctypes.data, out_s.nbytes)
    lib.thvm_cuda_buf_read_nosync(bb, out_b.ctypes.data, out_b.nbytes)
    assert np.array_equal(out_s, small) and np.array_equal(out_b, big)
    dst = cuda.alloc(big.nbytes)
    lib.thvm_cuda_buf_copy(dst, bb, big.nbytes)                       # device-written
    out_b[:] = 0
    lib.thvm_cuda_buf_read_nosync(dst, out_b.ctypes.data, out_b.nbytes)
    assert np.array_equal(out_b, big)
    out_a = np.zeros_like(big)
    lib.thvm_cuda_buf_read_async(dst, out_a.ctypes.data, out_a.nbytes)
    cuda.write(dst, np.zeros_like(big))                               # must not overtake the read-back
    lib.thvm_cuda_sync()
    assert np.array_equal(out_a, big)
    assert np.array_equal(cuda.read(dst, np.float32, big.size), np.zeros_like(big))
    cuda.reset(0)
    assert cuda.last_error() == ""


def test_layout_copy_kernels(cuda, oracle):
    """Padding materialised as ADD(pad(x), 0) (src/tensor/view/pad.c:2-16: a mask and a negative offset, never a copy)
    the opposite cut (SHRINK materialised) and the pool gradient's window-to-plane permute run on their own bandwidth
    kernels when the planes are contiguous;
    shapes those kernels decline (odd extents, permuted planes) fall to the general forms.  Bit for bit either way."""
    rng = np.random.default_rng(31)
    eligible = [(cases.pad_case(rng, 3, 5, 16, 16, 1), "pad_planes"), (cases.pad_case(rng, 2, 1, 28, 28, 2), "pad_planes"),
                (cases.pad_case(rng, 4, 64, 64, 64, 1), "pad_planes"), (cases.pad_case(rng, 1, 7, 9, 30, 1), "pad_planes"),
                (cases.permute_copy_case(rng, [2, 3, 4, 6, 2, 2], [0, 1, 2, 4, 3, 5]), "window_to_plane"),
                (cases.permute_copy_case(rng, [4, 64, 32, 32, 2, 2], [0, 1, 2, 4, 3, 5]), "window_to_plane"),
                (cases.permute_copy_case(rng, [5, 8, 2, 2], [0, 2, 1, 3]), "window_to_plane"),
                (cases.crop_case(rng, 3, 5, 16, 16, 1), "crop_planes"), (cases.crop_case(rng, 2, 64, 64, 64, 1), "crop_planes"),
                (cases.crop_case(rng, 2, 1, 28, 28, 2), "crop_planes"), (cases.crop_case(rng, 1, 7, 9, 32, 2, 1), "crop_planes")]
    declined = [cases.pad_case(rng, 2, 3, 5, 7, 2), cases.crop_case(rng, 2, 3, 5, 7, 2), cases.permute_copy_case(rng, [2, 3, 4, 5, 2, 2], [0, 1, 2, 4, 3, 5]),
                cases.permute_copy_case(rng, [2, 3, 4, 6, 2, 2], [1, 0, 2, 4, 3, 5])]
    for d, plan in eligible:
        got = cuda.run(d)
        assert cuda.last_plan() == plan, (d.name, cuda.last_plan())
        assert same(got, oracle.run(d)), d.name
    for d in declined:
        got = cuda.run(d)
        assert cuda.last_plan() not in ("pad_planes", "window_to_plane", "crop_planes"), (d.name, cuda.last_plan())
        assert same(got, oracle.run(d)), d.name
    assert cuda.last_error() == ""
