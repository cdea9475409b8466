"""The reference's Python-facing C surface (the `py_*` functions of py/csrc/libthvm.m, which its ctypes layer
py/tinyhvm/_ffi.py binds and its Tensor class is written on) running on the CUDA backend.

oracle/_ref/libthvm_py_ref.so is that shim compiled from the reference checkout together with the CUDA hub
(oracle/ref_py.c).  The cases below are this repository's own, in the style of the reference's op tests
(py/tests/test_ops.py: small random tensors, one op or a short composition each, atol 1e-4): every case is built
through py_tensor / py_scalar / py_op (elementwise, SUM / RMAX with an axis operand, MM) / py_assign / the movement calls, realised with py_to_host, and compared with numpy — once on the
reference's CPU backend (which shows the case itself is right; runs without a GPU) and once on "cuda".
The reference's pure-Python Tensor package cannot travel to the GPU box, so the surface is driven through ctypes here.
"""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
SO = ROOT / "oracle" / "_ref" / "libthvm_py_ref.so"
needs_shim = pytest.mark.skipif(not SO.exists(), reason="oracle/_ref/libthvm_py_ref.so not built (no reference checkout at build time)")

NEG, EXP, LOG, RELU, SQRT, ADD, MUL, DIV, MAX, CMP, SUB, SUM, RMAX, MM = 3, 4, 5, 6, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17
_u32, _u64, _vp = C.c_uint32, C.c_uint64, C.c_void_p


class Surface:
    def __init__(self, device: str):
        import os
        os.environ.setdefault("THVM_CUDA_LIB", str(ROOT / "tinyhvm_b200" / "libthvm_cuda.so"))
        if device == "cpu":
            # the reference's lowered CPU interpreter loads before it masks and walks off padded buffers
            # (src/lower/_.c:303-307, src/backend/cpu/uop.c:55-69): its structured interpreter is used instead
            os.environ["THVM_NO_LOWER"] = "1"
        else:
            os.environ.pop("THVM_NO_LOWER", None)
        L = self.L = C.CDLL(str(SO))
        L.py_init_device.restype, L.py_init_device.argtypes = _vp, [C.c_char_p]
        L.py_free.argtypes = [_vp]
        L.py_tensor.restype, L.py_tensor.argtypes = _u64, [_vp, _vp, C.POINTER(_u32), _u32]
        L.py_op.restype, L.py_op.argtypes = _u64, [_vp, _u32, _u64, _u64]
        L.py_to_host.restype, L.py_to_host.argtypes = C.POINTER(C.c_float), [_vp, _u64]
        L.py_era.restype = _u64
        L.py_numel.restype, L.py_numel.argtypes = _u32, [_vp, _u64]
        for f in ("py_reshape", "py_expand", "py_permute", "py_pad"):
            getattr(L, f).restype, getattr(L, f).argtypes = _u64, [_vp, _u64, C.POINTER(_u32), _u32]
        L.py_scalar.restype, L.py_scalar.argtypes = _u64, [_vp, C.c_float]
        L.py_assign.restype, L.py_assign.argtypes = _u64, [_vp, _u64, _u64]
        L.py_conv2d.restype, L.py_conv2d.argtypes = _u64, [_vp, _u64, _u64, _u64, _u32, C.POINTER(_u32), C.POINTER(_u32)]
        L.py_maxpool2d.restype, L.py_maxpool2d.argtypes = _u64, [_vp, _u64, C.POINTER(_u32), C.POINTER(_u32)]
        self.ctx = L.py_init_device(device.encode())
        self.era = L.py_era()

    def close(self):
        self.L.py_free(self.ctx)

    @staticmethod
    def _arr(v):
        return (_u32 * len(v))(*[int(x) for x in v])

    def tensor(self, a):
        a = np.ascontiguousarray(a, dtype=np.float32)
        return self.L.py_tensor(self.ctx, a.ctypes.data, self._arr(a.shape), a.ndim)

    def un(self, uop, t): return self.L.py_op(self.ctx, uop, t, self.era)
    def reduce(self, uop, t, axis): return self.L.py_op(self.ctx, uop, t, self.L.py_scalar(self.ctx, float(axis)))   # as py/tinyhvm/tensor.py:301-312 does
    def matmul(self, a, b): return self.L.py_op(self.ctx, MM, a, b)
    def assign(self, dst, src): return self.L.py_assign(self.ctx, dst, src)
    def bin(self, uop, a, b): return self.L.py_op(self.ctx, uop, a, b)
    def reshape(self, t, dims): return self.L.py_reshape(self.ctx, t, self._arr(dims), len(dims))
    def expand(self, t, dims): return self.L.py_expand(self.ctx, t, self._arr(dims), len(dims))
    def permute(self, t, axes): return self.L.py_permute(self.ctx, t, self._arr(axes), len(axes))
    def pad(self, t, pairs): return self.L.py_pad(self.ctx, t, self._arr([x for p in pairs for x in p]), len(pairs))

    def host(self, t, shape):
        p = self.L.py_to_host(self.ctx, t)
        n = int(np.prod(shape))
        assert p, "py_to_host returned NULL"
        return np.ctypeslib.as_array(p, shape=(n,)).copy().reshape(shape)


def cases():
    rng = np.random.default_rng(5)
    r = lambda *s: rng.uniform(-2, 2, size=s).astype(np.float32)
    a, b, c = r(45, 65), r(45, 65), r(45, 65)
    out = []
    add = lambda name, build, want: out.append((name, build, want))
    for name, uop, f in (("add", ADD, np.add), ("sub", SUB, np.subtract), ("mul", MUL, np.multiply), ("maximum", MAX, np.maximum)):
        add(name, lambda S, uop=uop: S.bin(uop, S.tensor(a), S.tensor(b)), f(a, b))
    add("div", lambda S: S.bin(DIV, S.tensor(a), S.tensor(np.abs(b) + 0.5)), a / (np.abs(b) + 0.5))
    add("cmp_gt", lambda S: S.bin(CMP, S.tensor(a), S.tensor(b)), (a > b).astype(np.float32))
    add("neg", lambda S: S.un(NEG, S.tensor(a)), -a)
    add("relu", lambda S: S.un(RELU, S.tensor(a)), np.maximum(a, 0))
    add("exp", lambda S: S.un(EXP, S.tensor(a)), np.exp(a))
    add("log", lambda S: S.un(LOG, S.tensor(np.abs(a) + 0.1)), np.log(np.abs(a) + 0.1))
    add("sqrt", lambda S: S.un(SQRT, S.tensor(np.abs(a))), np.sqrt(np.abs(a)))
    add("fused_chain", lambda S: S.un(RELU, S.bin(ADD, S.bin(MUL, S.tensor(a), S.tensor(b)), S.tensor(c))), np.maximum(a * b + c, 0))
    add("broadcast_row", lambda S: S.bin(ADD, S.tensor(a), S.expand(S.reshape(S.tensor(b[0]), [1, 65]), [45, 65])), a + b[0][None, :])
    add("broadcast_scalar", lambda S: S.bin(MUL, S.tensor(a), S.expand(S.reshape(S.tensor(np.float32([2.5])), [1, 1]), [45, 65])), a * 2.5)
    add("permute_copy", lambda S: S.bin(ADD, S.permute(S.tensor(a), [1, 0]), S.tensor(np.zeros((65, 45), np.float32))), a.T)
    add("pad_then_op", lambda S: S.bin(ADD, S.pad(S.tensor(a), [(1, 2), (3, 0)]), S.tensor(np.zeros((48, 68), np.float32))), np.pad(a, ((1, 2), (3, 0))))
    w, bias = r(65, 30) / 2, r(30)
    add("sum_axis1", lambda S: S.reduce(SUM, S.tensor(a), 1), a.sum(1, keepdims=True))
    add("max_axis0", lambda S: S.reduce(RMAX, S.tensor(a), 0), a.max(0, keepdims=True))
    add("sum_all", lambda S: S.reduce(SUM, S.reduce(SUM, S.tensor(a), 1), 0), a.sum(dtype=np.float64).astype(np.float32).reshape(1, 1))
    add("matmul", lambda S: S.matmul(S.tensor(a), S.tensor(w)), a @ w)
    add("linear_relu", lambda S: S.un(RELU, S.bin(ADD, S.matmul(S.tensor(a), S.tensor(w)), S.expand(S.reshape(S.tensor(bias), [1, 30]), [45, 30]))),
        np.maximum(a @ w + bias, 0))
    sm = np.exp(a - a.max(1, keepdims=True))
    add("softmax", lambda S: S.bin(DIV, S.un(EXP, S.bin(SUB, S.tensor(a), S.expand(S.reduce(RMAX, S.tensor(a), 1), [45, 65]))),
                                   S.expand(S.reduce(SUM, S.un(EXP, S.bin(SUB, S.tensor(a), S.expand(S.reduce(RMAX, S.tensor(a), 1), [45, 65]))), 1), [45, 65])),
        sm / sm.sum(1, keepdims=True))
    add("assign", lambda S: S.assign(S.tensor(a), S.bin(ADD, S.tensor(a), S.tensor(b))), a + b)
    x4, w4, b4 = r(2, 3, 12, 12), r(5, 3, 3, 3) / 3, r(5)
    return out, (x4, w4, b4)


def conv_ref(x, w, b):
    B, Ci, H, W = x.shape
    Co, _, K, _ = w.shape
    O = H - K + 1
    y = np.zeros((B, Co, O, O), np.float64)
    for kh in range(K):
        for kw in range(K):
            y += np.einsum("bchw,oc->bohw", x[:, :, kh:kh + O, kw:kw + O].astype(np.float64), w[:, :, kh, kw].astype(np.float64))
    return (y + b[None, :, None, None]).astype(np.float32)


def run_all(device):
    S = Surface(device)
    try:
        ops, (x4, w4, b4) = cases()
        for name, build, want in ops:
            got = S.host(build(S), want.shape)
            assert np.allclose(got, want, atol=2e-4 if name == "sum_all" else 1e-4, rtol=1e-5), f"{device}: {name}"
        # nn surface: convolution without padding (+ bias) and 2x2 max-pool (src/nn/conv.c:390-513)
        one, zero = S._arr([1, 1]), S._arr([0, 0])
        y = S.L.py_conv2d(S.ctx, S.tensor(x4), S.tensor(w4), S.tensor(b4), 1, one, zero)
        assert np.allclose(S.host(y, (2, 5, 10, 10)), conv_ref(x4, w4, b4), atol=1e-4), f"{device}: conv2d"
        two = S._arr([2, 2])
        p = S.L.py_maxpool2d(S.ctx, S.tensor(x4), two, two)
        assert np.allclose(S.host(p, (2, 3, 6, 6)), x4.reshape(2, 3, 6, 2, 6, 2).max(axis=(3, 5)), atol=0), f"{device}: maxpool2d"
    finally:
        S.close()


@needs_shim
def test_py_surface_cases_on_the_reference_cpu_backend():
    run_all("cpu")


@needs_shim
@pytest.mark.gpu
def test_py_surface_cases_on_cuda():
    run_all("cuda")
