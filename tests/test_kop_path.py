"""The lowered-program path of the vtable (dispatch_uop_kernel).

Programs come from the reference's OWN lowerer (thvm_lower_kernel_uop, src/lower/_.c:765-973, linked into
oracle/_ref/libthvm_host_ref.so and reached through drv_lower_dispatch): a dispatch in dispatch_kernel_rs form goes
in, the KOP program the scheduler would hand to dispatch_uop_kernel (src/schedule/_.c:2343-2378) comes out.

CPU: the restated KOP interpreter of the oracle is pinned to the reference's (src/backend/cpu/uop.c:29-155) on those
programs, bit for bit.  Programs over padded (masked) views are left out of that comparison because the reference's
interpreter loads before it masks (src/lower/_.c:303-307, src/backend/cpu/uop.c:55-69) and walks off the buffer; for
them the oracle runs in checked mode (a load outside the buffer yields 0, the following MASK discards it), and must
then agree with the structured form of the same dispatch.

GPU: the device interpreter runs the same programs — including a convolution's padding materialised as
ADD(pad(x), 0), the load-before-mask case, and a max-pool RMAX — and is compared with the pinned oracle.
"""
import ctypes as C

import numpy as np
import pytest

import cases
import hostref
from test_host_dropin import needs_ref
from tinyhvm_b200 import abi
from tinyhvm_b200.abi import F32, SUM

_u32, _u64, _vp = C.c_uint32, C.c_uint64, C.c_void_p


def lower(d):
    """KOP program of a dispatch, made by the reference's lowerer; None if it declines."""
    L = hostref.lib()
    views, sts, ops, full, red, dts = d.c_args()
    k = abi.UOpKernel()
    rc = L.drv_lower_dispatch(views, C.cast(sts, _vp) if sts is not None else None, _u32(len(d.leaves)), ops, _u32(len(d.ops)),
                              C.byref(full), C.byref(red) if red is not None else None, dts, C.byref(k))
    return k if rc == 1 and k.n_ops > 0 else None


def unmasked_programs():
    rng = np.random.default_rng(21)
    return [cases.chain_fwd_case(rng, 8, 300), cases.chain_bwd_case(rng, 9, 77), cases.mm_case(rng, 12, 40, 9),
            cases.mm_case(rng, 6, 300, 5), cases.bias_relu_case(rng, 7, 13), cases.maxpool_case(rng, 2, 3, 8, 8, ties=True),
            cases.bn_stats_case(rng, 4, 5, 6, 6), cases.bn_var_case(rng, 4, 8, 6, 6), cases.conv_fprop_case(rng, 2, 3, 8, 8, 4, 3),
            cases.rowmax_case(rng, 16, 10), cases.softmax_sum_case(rng, 16, 10), cases.permute_copy_case(rng, [5, 7], [1, 0]),
            cases.bias_grad_case(rng, 40, 11)]


def masked_programs():
    rng = np.random.default_rng(22)
    return [cases.pad_case(rng, 2, 3, 8, 8, 1), cases.pad_case(rng, 1, 1, 28, 28, 2), cases.pad_case(rng, 3, 2, 5, 7, 2)]


@needs_ref
def test_oracle_kop_interpreter_is_pinned_to_the_reference_on_lowered_programs(oracle, ref):
    n_group = 0
    for d in unmasked_programs():
        k = lower(d)
        assert k is not None, d.name
        n_group += k.local_size > 0
        leaves = [np.ascontiguousarray(l.data) for l in d.leaves]
        got = oracle.uop_kernel(k, leaves, np.zeros(d.out_numel, np.float32), checked=False)
        ids = [ref.upload(x) for x in leaves]
        out = ref.lib.ref_buf_alloc(_u64(max(d.out_numel * 4, 4)))
        ref.lib.ref_dispatch_uop_kernel(_u32(out), (_u32 * len(ids))(*ids), _u32(len(ids)), C.byref(k))
        want = ref.read(out, np.float32, d.out_numel)
        ref.lib.ref_pool_reset(_u32(ids[0] - 1))
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"{d.name}: oracle and reference interpreters differ"
        # and the lowered program computes what the structured dispatch computes (same left-to-right accumulation)
        direct = oracle.run(d)
        assert np.allclose(got, direct, rtol=1e-5, atol=1e-6), d.name
    assert n_group >= 2, "no group-reduce program (reduce range >= 256) among the cases"


@needs_ref
def test_checked_oracle_runs_load_before_mask_programs(oracle):
    for d in masked_programs():
        k = lower(d)
        assert k is not None, d.name
        types = [k.ops[i].type for i in range(k.n_ops)]
        assert abi.KOP_MASK in types and types.index(abi.KOP_LOAD) < types.index(abi.KOP_MASK), "not the load-before-mask shape"
        leaves = [np.ascontiguousarray(l.data) for l in d.leaves]
        got = oracle.uop_kernel(k, leaves, np.zeros(d.out_numel, np.float32), checked=True)
        assert np.array_equal(got, oracle.run(d)), d.name


@needs_ref
@pytest.mark.gpu
def test_lowered_programs_on_the_device_interpreter(cuda, oracle):
    """Every program above, the padded ones included, through thvm_cuda_dispatch_uop_kernel: equal to the oracle
    (bit for bit without a reduce; sums run in the same order per output, so they are held to 1e-6)."""
    lib = cuda.lib
    for d in unmasked_programs() + masked_programs():
        k = lower(d)
        assert k is not None, d.name
        cuda.reset(0)
        ids = [cuda.upload(np.ascontiguousarray(l.data)) for l in d.leaves]
        out = cuda.alloc(max(d.out_numel * 4, 4))
        lib.thvm_cuda_dispatch_uop_kernel(out, (_u32 * len(ids))(*ids), len(ids), C.byref(k), 0)
        assert cuda.last_plan() == "uop_program"
        got = cuda.read(out, np.float32, d.out_numel)
        assert cuda.last_error() == "", (d.name, cuda.last_error())
        want = oracle.run(d)
        if d.reduce_type == 0 and not any(o[0] in (abi.EXP, abi.LOG) for o in d.ops):
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), d.name
        else:
            assert np.allclose(got, want, rtol=1e-5, atol=1e-6), d.name
    cuda.reset(0)


@pytest.mark.gpu
def test_device_interpreter_refuses_a_program_that_would_not_end(cuda):
    """Nested RANGEs whose trip counts multiply out beyond the step budget are refused on the host; nothing is launched."""
    k = abi.UOpKernel()
    ops = [(abi.KOP_RANGE, 0xFFFFFFFF), (abi.KOP_RANGE, 0xFFFFFFFF), (abi.KOP_ENDRANGE, 0), (abi.KOP_ENDRANGE, 0)]
    for i, (t, imm) in enumerate(ops):
        k.ops[i].type = t
        k.ops[i].imm.u = imm
    k.n_ops, k.n_bufs, k.n_leaves = len(ops), 1, 0
    k.grid[0] = k.grid[1] = k.grid[2] = 1
    cuda.reset(0)
    out = cuda.alloc(16)
    before = cuda.launches()
    cuda.lib.thvm_cuda_dispatch_uop_kernel(out, (_u32 * 1)(0), 0, C.byref(k), 0)
    assert "op executions per output exceed" in cuda.last_error()
    assert cuda.launches() == before
    cuda.clear_error()
    cuda.reset(0)
