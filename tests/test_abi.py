"""CPU-side checks of the C ABI: the library loads without a GPU, exports every
symbol include/thvm_cuda.h declares, and the ctypes mirrors have the C layout."""
import ctypes as C
import re
from pathlib import Path

import tinyhvm_b200
from tinyhvm_b200 import abi

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "thvm_cuda.h").read_text()
    return sorted(set(re.findall(r"\b(thvm_cuda_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = tinyhvm_b200.load()
    names = declared_symbols()
    assert len(names) >= 36
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/thvm_cuda.h but not exported"
    assert set(names) == set(tinyhvm_b200.SYMBOLS), set(names) ^ set(tinyhvm_b200.SYMBOLS)


def test_struct_layouts():
    assert C.sizeof(abi.Shape) == 36
    assert C.sizeof(abi.View) == 212
    assert abi.View.mask_begin.offset == 80 and abi.View.compound_masks.offset == 148 and abi.View.mod_size.offset == 180
    assert C.sizeof(abi.Tracker) == 852
    assert C.sizeof(abi.FusedOp) == 16
    assert C.sizeof(abi.ReduceSpec) == 36 and abi.ReduceSpec.is_reduce2.offset == 28
    assert C.sizeof(abi.KOp) == 20
    assert C.sizeof(abi.UOpKernel) == 512 * 20 + 12 + 64 * 212 + 64 * 4 + 32 + 4 + 36 + 12 + 12 + 12


def test_no_device_means_loud_failure():
    """Without a CUDA device init reports failure; it never silently computes on the CPU."""
    import torch
    if torch.cuda.is_available():
        return
    lib = tinyhvm_b200.load()
    assert lib.thvm_cuda_init() != 0
    assert b"no CUDA device" in lib.thvm_cuda_last_error()


def test_view_algebra_canonical_forms():
    v = abi.view_contiguous([2, 1, 3])
    assert abi.view_strides(v) == [3, 0, 1] and v.numel == 6 and v.contiguous == 1
    p = abi.view_pad(abi.view_contiguous([2, 3]), [1, 2], [1, 0])
    assert abi.view_dims(p) == [4, 5] and p.offset == -(1 * 3 + 2 * 1) and p.has_mask == 1
    assert list(p.mask_begin)[:2] == [1, 2] and list(p.mask_end)[:2] == [3, 5]
    w = abi.view_pool(abi.view_contiguous([1, 1, 3, 3]), [2, 2], [1, 1])
    assert abi.view_dims(w) == [1, 1, 2, 2, 2, 2] and abi.view_strides(w) == [0, 0, 3, 1, 3, 1]
    s = abi.view_shrink(abi.view_contiguous([4, 5]), [1, 2], [3, 5])
    assert abi.view_dims(s) == [2, 3] and s.offset == 7


def test_dp_allreduce_refuses_bad_buffers_before_any_collective():
    """An argument error must come back before a collective is opened (a rank that issued a shorter group than its
    peers would leave them waiting): ids that are not live are refused with return code 1 on the spot."""
    lib = tinyhvm_b200.load()
    ids = (C.c_uint32 * 2)(123, 0)
    counts = (C.c_uint64 * 2)(16, 16)
    lib.thvm_cuda_clear_error()
    assert lib.thvm_cuda_dp_allreduce_sum(ids, counts, 2) == 1
    assert b"not live" in lib.thvm_cuda_last_error()
    lib.thvm_cuda_clear_error()
