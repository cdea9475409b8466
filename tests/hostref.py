"""Loader for oracle/_ref/libthvm_host_ref.so: the reference's own host runtime
(reducer, fuser, scheduler, nn library) with its CPU backend and the CUDA hub,
plus the staged driver programs of oracle/ref_host.c.

`run(driver, device, *args)` executes one driver with thvm_init(device) and
returns {name: array} of every tensor the driver kept.  The library exists only
where it was built from a reference checkout; tests skip otherwise.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
SO = ROOT / "oracle" / "_ref" / "libthvm_host_ref.so"
_lib = None


def available() -> bool:
    return SO.exists()


def lib():
    global _lib
    if _lib is None:
        os.environ.setdefault("THVM_CUDA_LIB", str(ROOT / "tinyhvm_b200" / "libthvm_cuda.so"))
        _lib = C.CDLL(str(SO))
        _lib.drv_name.restype = C.c_char_p
        _lib.drv_data.restype = C.POINTER(C.c_float)
        _lib.drv_numel.restype = C.c_uint32
        _lib.drv_count.restype = C.c_uint32
        _lib.drv_seconds.restype = C.c_double
    return _lib


def _arg(a):
    if isinstance(a, np.ndarray):
        return C.c_void_p(a.ctypes.data)
    if isinstance(a, float):
        return C.c_float(a)
    if isinstance(a, int):
        return C.c_uint32(a)
    return a


def run(driver: str, device: str, *args) -> dict:
    L = lib()
    L.drv_clear()
    keepalive = [np.ascontiguousarray(a) if isinstance(a, np.ndarray) else a for a in args]
    rc = getattr(L, driver)(device.encode(), *[_arg(a) for a in keepalive])
    assert rc == 0, f"{driver} returned {rc}"
    out = {}
    for i in range(L.drv_count()):
        n = L.drv_numel(i)
        name = L.drv_name(i).decode()
        out[name] = np.ctypeslib.as_array(L.drv_data(i), shape=(n,)).copy() if n else np.zeros(0, np.float32)
    out["_seconds"] = L.drv_seconds()
    return out
