"""Loaders for the two checkers the tests compare against.

`Oracle`    — oracle/liboracle.so, the CPU restatement (built on demand with gcc).
`Reference` — oracle/_ref/libthvm_cpu_ref.so, the reference's own CPU backend,
              present only where the reference checkout was available at build time.
Both take a `tinyhvm_b200.abi.Dispatch` and return the output as a numpy array.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

from tinyhvm_b200 import abi

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"

_u32, _u64, _vp = C.c_uint32, C.c_uint64, C.c_void_p


def build_oracle() -> Path:
    so = ORACLE_DIR / "liboracle.so"
    src = ORACLE_DIR / "thvm_oracle.c"
    if not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(ORACLE_DIR), "liboracle.so"], check=True, capture_output=True)
    return so


class Oracle:
    def __init__(self):
        self.lib = C.CDLL(str(build_oracle()))
        self.lib.oracle_f32_to_f16.restype = C.c_uint16
        self.lib.oracle_f32_to_f16.argtypes = [C.c_float]
        self.lib.oracle_f16_to_f32.restype = C.c_float
        self.lib.oracle_f16_to_f32.argtypes = [C.c_uint16]
        self.lib.oracle_signature.restype = _u64

    def run(self, d: abi.Dispatch) -> np.ndarray:
        views, sts, ops, full, red, dts = d.c_args()
        n = len(d.leaves)
        bufs = [np.ascontiguousarray(l.data) for l in d.leaves]
        ptrs = (_vp * n)(*[b.ctypes.data for b in bufs])
        out = np.zeros(max(d.out_numel, 1), dtype=abi.NP_DTYPE[d.out_dtype])
        self.lib.oracle_dispatch_kernel_rs(
            _vp(out.ctypes.data), ptrs, views, C.cast(sts, _vp) if sts is not None else None, _u32(n),
            ops, _u32(len(d.ops)), C.byref(full), C.byref(red) if red is not None else None, dts, _u32(d.out_dtype))
        return out[:d.out_numel]

    def run_with_wide_sums(self, d: abi.Dispatch):
        """(f32 output, the same SUM accumulated in double): the second is the
        exact sum of the f32 terms, against which both summation orders are measured."""
        wide = np.zeros(max(d.out_numel, 1), dtype=np.float64)
        self.lib.oracle_set_wide_sums(_vp(wide.ctypes.data))
        try:
            out = self.run(d)
        finally:
            self.lib.oracle_set_wide_sums(None)
        return out, wide[:d.out_numel]

    def signature(self, d: abi.Dispatch) -> int:
        views, sts, ops, full, red, _ = d.c_args()
        return int(self.lib.oracle_signature(ops, _u32(len(d.ops)), views, C.cast(sts, _vp) if sts is not None else None,
                                             _u32(len(d.leaves)), C.byref(full), C.byref(red) if red is not None else None))

    def uop_kernel(self, k: abi.UOpKernel, leaves: list[np.ndarray], out: np.ndarray, checked: bool = True) -> np.ndarray:
        n = len(leaves)
        ptrs = (_vp * max(n, 1))(*[l.ctypes.data for l in leaves])
        caps = (_u64 * max(n, 1))(*[l.size for l in leaves])
        self.lib.oracle_dispatch_uop_kernel(_vp(out.ctypes.data), _u64(out.size if checked else 0), ptrs,
                                            caps if checked else None, _u32(n), C.byref(k))
        return out


class Reference:
    """The reference's CPU backend behind its own vtable (buffer ids, not pointers)."""

    def __init__(self, path: Path):
        self.lib = C.CDLL(str(path))
        self.lib.ref_buf_alloc.restype = _u32
        self.lib.ref_buf_alloc.argtypes = [_u64]
        self.lib.ref_buf_write.argtypes = [_u32, _vp, _u64]
        self.lib.ref_buf_read.argtypes = [_u32, _vp, _u64]
        self.lib.ref_signature.restype = _u64
        self.lib.ref_f32_to_f16.restype = C.c_uint16
        self.lib.ref_f32_to_f16.argtypes = [C.c_float]
        self.lib.ref_f16_to_f32.restype = C.c_float
        self.lib.ref_f16_to_f32.argtypes = [C.c_uint16]
        self.lib.ref_init()

    @classmethod
    def try_load(cls):
        so = ORACLE_DIR / "_ref" / "libthvm_cpu_ref.so"
        if not so.exists():
            try:
                import os
                ref = os.environ.get("THVM_REFERENCE") or str(ROOT.parent / "reference")
                subprocess.run(["make", "-C", str(ORACLE_DIR), "ref", f"REF={ref}"], check=True, capture_output=True)
            except Exception:
                return None
        return cls(so) if so.exists() else None

    def upload(self, arr: np.ndarray) -> int:
        arr = np.ascontiguousarray(arr)
        bid = self.lib.ref_buf_alloc(max(arr.nbytes, 4))
        if arr.nbytes:
            self.lib.ref_buf_write(bid, arr.ctypes.data, arr.nbytes)
        return bid

    def read(self, bid: int, dtype, count: int) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        self.lib.ref_buf_read(bid, out.ctypes.data, out.nbytes)
        return out

    def run(self, d: abi.Dispatch) -> np.ndarray:
        views, sts, ops, full, red, dts = d.c_args()
        ids = [self.upload(l.data) for l in d.leaves]
        out = self.lib.ref_buf_alloc(max(d.out_numel * abi.DTYPE_SIZE[d.out_dtype], 4))
        idarr = (_u32 * len(ids))(*ids)
        self.lib.ref_dispatch_kernel_rs(_u32(out), idarr, views, C.cast(sts, _vp) if sts is not None else None,
                                        _u32(len(ids)), ops, _u32(len(d.ops)), C.byref(full),
                                        C.byref(red) if red is not None else None, dts, _u32(d.out_dtype))
        res = self.read(out, abi.NP_DTYPE[d.out_dtype], d.out_numel)
        self.lib.ref_pool_reset(_u32(ids[0] - 1))
        return res

    def signature(self, d: abi.Dispatch) -> int:
        views, sts, ops, full, red, _ = d.c_args()
        return int(self.lib.ref_signature(ops, _u32(len(d.ops)), views, C.cast(sts, _vp) if sts is not None else None,
                                          _u32(len(d.leaves)), C.byref(full), C.byref(red) if red is not None else None))
