"""tinyhvm_b200 — B200 (sm_100a) backend for TinyHVM's realized-kernel path.

The product is `libthvm_cuda.so`, a C-ABI library whose entry points are the
slots of the reference's `Backend` vtable (include/thvm_cuda.h).  This package
is the thin Python host side used by the tests and the benchmark: it loads the
library with ctypes and drives it exactly as the reference's scheduler would
(buf_alloc / buf_write / dispatch_kernel_rs / buf_read).

There is no CPU fallback: `load()` raises if the library has not been built,
and `CudaBackend()` raises if no CUDA device answers.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import abi
from .abi import Dispatch, Leaf

_LIB_PATH = Path(__file__).resolve().parent / "libthvm_cuda.so"
_lib = None

_u32, _u64, _vp = C.c_uint32, C.c_uint64, C.c_void_p
_PV = C.POINTER(abi.View)

# name -> (restype, argtypes): every symbol include/thvm_cuda.h declares
SYMBOLS = {
    "thvm_cuda_init": (C.c_int, []),
    "thvm_cuda_shutdown": (None, []),
    "thvm_cuda_buf_alloc": (_u32, [_u64]),
    "thvm_cuda_buf_free": (None, [_u32]),
    "thvm_cuda_buf_incref": (None, [_u32]),
    "thvm_cuda_buf_decref": (None, [_u32]),
    "thvm_cuda_mem_checkpoint": (None, [C.POINTER(_u32), _u32]),
    "thvm_cuda_buf_mark_use": (None, [_u32]),
    "thvm_cuda_buf_write": (None, [_u32, _vp, _u64]),
    "thvm_cuda_buf_read": (None, [_u32, _vp, _u64]),
    "thvm_cuda_op_unary": (None, [_u32, _u32, _PV, _u32, _u32, _PV, _u32]),
    "thvm_cuda_op_binary": (None, [_u32, _u32, _PV, _u32, _u32, _PV, _u32, _u32, _PV, _u32]),
    "thvm_cuda_op_mm": (None, [_u32, _u32, _u32, _PV, _u32, _u32, _PV, _u32, _u32, _u32, _u32]),
    "thvm_cuda_op_reduce": (None, [_u32, _u32, _u32, _u32, _u32, _u32, _u32, _u32]),
    "thvm_cuda_dispatch_kernel_rs": (None, [_u32, C.POINTER(_u32), C.POINTER(_PV), _vp, _u32,
                                            C.POINTER(abi.FusedOp), _u32, C.POINTER(abi.Shape),
                                            C.POINTER(abi.ReduceSpec), _vp, _vp, _u32, C.POINTER(_u32), _u32]),
    "thvm_cuda_dispatch_uop_kernel": (None, [_u32, C.POINTER(_u32), _u32, C.POINTER(abi.UOpKernel), _u64]),
    "thvm_cuda_contiguify": (None, [_u32, _u32, _u32, _PV]),
    "thvm_cuda_buf_copy": (None, [_u32, _u32, _u64]),
    "thvm_cuda_buf_read_nosync": (None, [_u32, _vp, _u64]),
    "thvm_cuda_buf_read_async": (None, [_u32, _vp, _u64]),
    "thvm_cuda_adam_step": (None, [_u32, _u32, _u32, _u32] + [C.c_float] * 6 + [_u32]),
    "thvm_cuda_pool_reset": (None, [_u32]),
    "thvm_cuda_pool_set_persistent": (None, [_u32]),
    "thvm_cuda_begin_batch": (None, []),
    "thvm_cuda_end_batch": (None, []),
    "thvm_cuda_profile_report": (None, []),
    "thvm_cuda_profile_reset": (None, []),
    "thvm_cuda_last_error": (C.c_char_p, []),
    "thvm_cuda_clear_error": (None, []),
    "thvm_cuda_stream": (_vp, []),
    "thvm_cuda_sync": (None, []),
    "thvm_cuda_buf_ptr": (_vp, [_u32]),
    "thvm_cuda_buf_bytes": (_u64, [_u32]),
    "thvm_cuda_launch_count": (_u64, []),
    "thvm_cuda_last_plan": (C.c_char_p, []),
    "thvm_cuda_set_force_generic": (None, [C.c_int]),
    "thvm_cuda_plan_count": (_u64, []),
    "thvm_cuda_dp_unique_id": (C.c_int, [_vp]),
    "thvm_cuda_dp_init": (C.c_int, [C.c_int, C.c_int, _vp]),
    "thvm_cuda_dp_world": (C.c_int, []),
    "thvm_cuda_dp_rank": (C.c_int, []),
    "thvm_cuda_dp_allreduce_sum": (C.c_int, [C.POINTER(_u32), C.POINTER(_u64), _u32]),
    "thvm_cuda_dp_shutdown": (None, []),
    "thvm_cuda_dp_arena_create": (C.c_int, [_u64, _vp]),
    "thvm_cuda_dp_arena_attach": (C.c_int, [C.c_int, _vp]),
    "thvm_cuda_dp_sgd_step": (C.c_int, [C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u64), _u32, _u32]),
    "thvm_cuda_dp_arena_attach_silent": (C.c_int, [C.c_int]),
    "thvm_cuda_dp_set_poll_limit": (None, [_u64]),
    "thvm_cuda_capture_begin": (C.c_int, []),
    "thvm_cuda_capture_input": (C.c_int, [_u32, _vp, _u64]),
    "thvm_cuda_capture_end": (C.c_int, []),
    "thvm_cuda_graph_set_input": (C.c_int, [C.c_int, C.c_int, _vp]),
    "thvm_cuda_graph_prefetch_input": (C.c_int, [C.c_int, C.c_int, _vp]),
    "thvm_cuda_graph_launch": (C.c_int, [C.c_int]),
    "thvm_cuda_graph_result": (C.c_int, [C.c_int, C.c_int, _vp, _u64]),
    "thvm_cuda_graph_result_async": (C.c_int, [C.c_int, C.c_int, _vp, _u64]),
    "thvm_cuda_graph_counts": (C.c_int, [C.c_int, C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u64)]),
    "thvm_cuda_graph_nodes": (C.c_int, [C.c_int, C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u32)]),
    "thvm_cuda_graph_destroy": (None, [C.c_int]),
    "thvm_cuda_graph_memory": (C.c_int, [C.c_int, C.POINTER(_u64), C.POINTER(_u64), C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u64)]),
    "thvm_cuda_capture_input_sizes": (None, [C.POINTER(_u64), _u32]),
    "thvm_cuda_graph_input_bytes": (_u64, [C.c_int, C.c_int]),
    "thvm_cuda_maxpool2x2_index": (C.c_int, [_u32, _u32, _u32, _u32, _u32, _u32]),
    "thvm_cuda_argmax_rows": (C.c_int, [_u32, _u32, _u32, _u32]),
    "thvm_cuda_channel_sums_noalloc": (C.c_int, [_vp, _vp, _u32, _u32, _u32, _vp]),
    "thvm_cuda_signature": (_u64, [C.POINTER(abi.FusedOp), _u32, C.POINTER(_PV), _vp, _u32,
                                   C.POINTER(abi.Shape), C.POINTER(abi.ReduceSpec)]),
}


def load() -> C.CDLL:
    """dlopen libthvm_cuda.so and type every entry point.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(f"{_LIB_PATH} is missing: run `python -m tinyhvm_b200.build` (there is no CPU fallback)")
    lib = C.CDLL(str(_LIB_PATH))
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)          # AttributeError = the library does not match the header
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


class CudaBackend:
    """The vtable as a Python object; one per process (the library's state is global)."""

    def __init__(self):
        self.lib = load()
        if self.lib.thvm_cuda_init() != 0:
            raise RuntimeError("thvm_cuda_init failed: " + self.lib.thvm_cuda_last_error().decode())

    # -- buffers
    def alloc(self, nbytes: int) -> int:
        bid = self.lib.thvm_cuda_buf_alloc(nbytes)
        if bid == 0:
            raise MemoryError(self.last_error())
        return bid

    def write(self, bid: int, arr: np.ndarray) -> None:
        arr = np.ascontiguousarray(arr)
        self.lib.thvm_cuda_buf_write(bid, arr.ctypes.data, arr.nbytes)

    def read(self, bid: int, dtype, count: int) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        self.lib.thvm_cuda_buf_read(bid, out.ctypes.data, out.nbytes)
        return out

    def upload(self, arr: np.ndarray) -> int:
        bid = self.alloc(max(arr.nbytes, 1))
        if arr.nbytes:
            self.write(bid, arr)
        return bid

    def reset(self, keep: int = 0) -> None:
        self.lib.thvm_cuda_pool_reset(keep)

    # -- compute
    def dispatch_ids(self, out_id: int, leaf_ids, d: Dispatch) -> None:
        views, sts, ops, full, red, dts = d.c_args()
        ids = (C.c_uint32 * len(leaf_ids))(*leaf_ids)
        self.lib.thvm_cuda_dispatch_kernel_rs(
            out_id, ids, views, C.cast(sts, C.c_void_p) if sts is not None else None, len(leaf_ids),
            ops, len(d.ops), C.byref(full), C.byref(red) if red is not None else None,
            None, None, 0, dts, d.out_dtype)

    def run(self, d: Dispatch) -> np.ndarray:
        """Upload the leaves, dispatch, read the output back (the call sequence of
        src/schedule/_.c:2279-2378 followed by src/ops/_.c:317)."""
        ids = [self.upload(l.data) for l in d.leaves]
        n_out = d.out_numel
        out = self.alloc(max(n_out * abi.DTYPE_SIZE[d.out_dtype], 1))
        self.dispatch_ids(out, ids, d)
        res = self.read(out, abi.NP_DTYPE[d.out_dtype], n_out)
        self.reset(min(ids + [out]) - 1)      # frees these buffers and rewinds the id counter
        return res

    # -- diagnostics
    def last_error(self) -> str:
        return self.lib.thvm_cuda_last_error().decode()

    def clear_error(self) -> None:
        self.lib.thvm_cuda_clear_error()

    def last_plan(self) -> str:
        return self.lib.thvm_cuda_last_plan().decode()

    def sync(self) -> None:
        self.lib.thvm_cuda_sync()

    def launches(self) -> int:
        return int(self.lib.thvm_cuda_launch_count())

    def force_generic(self, on: bool) -> None:
        self.lib.thvm_cuda_set_force_generic(1 if on else 0)

    def shutdown(self) -> None:
        self.lib.thvm_cuda_shutdown()
