"""ctypes mirrors of the C ABI in include/thvm_cuda.h, plus the small amount of
view algebra a host needs to describe a dispatch.

The structs are layout-identical to the reference's `Shape`, `View`,
`ShapeTracker`, `FusedOp`, `ReduceSpec`, `KOp` and `UOpKernel`
(reference: src/tinyhvm.h:531-717); the helpers produce views in the
reference's canonical form: size-1 dims carry stride 0
(src/tensor/view/create.c:5-8), PAD is a mask plus a negative offset
(src/tensor/view/pad.c:2-16), a pooling window is a strided alias
(src/nn/conv.c:26-80).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

MAX_DIM, MAX_VIEWS, MAX_OPS, MAX_LEAVES, KOP_MAX = 8, 4, 64, 64, 512

F32, F16, I32, U32 = 0, 1, 2, 3
NP_DTYPE = {F32: np.float32, F16: np.uint16, I32: np.int32, U32: np.uint32}  # f16 travels as raw bits
DTYPE_SIZE = {F32: 4, F16: 2, I32: 4, U32: 4}

NEG, EXP, LOG, RELU, CAST, SQRT, ADD, MUL, DIV, MAX, CMP, SUB, SUM, RMAX = range(3, 17)
UNARY = {NEG, EXP, LOG, RELU, CAST, SQRT}
BINARY = {ADD, MUL, DIV, MAX, CMP, SUB}


class Shape(C.Structure):
    _fields_ = [("dims", C.c_uint32 * MAX_DIM), ("rank", C.c_uint32)]


class CompoundMask(C.Structure):
    _fields_ = [("dim_a", C.c_uint8), ("dim_b", C.c_uint8), ("stride_a", C.c_int32),
                ("begin", C.c_uint32), ("end", C.c_uint32)]


class View(C.Structure):
    _fields_ = [("shape", Shape), ("strides", C.c_int32 * MAX_DIM), ("offset", C.c_int32),
                ("numel", C.c_uint32), ("contiguous", C.c_uint8), ("has_mask", C.c_uint8),
                ("mask_begin", C.c_uint32 * MAX_DIM), ("mask_end", C.c_uint32 * MAX_DIM),
                ("n_compound_masks", C.c_uint8), ("compound_masks", CompoundMask * 2),
                ("mod_size", C.c_uint32 * MAX_DIM)]


class Tracker(C.Structure):
    _fields_ = [("views", View * MAX_VIEWS), ("n_views", C.c_uint8)]


class FusedOp(C.Structure):
    _fields_ = [("uop", C.c_uint32), ("arg_a", C.c_uint32), ("arg_b", C.c_uint32), ("aux", C.c_uint32)]


class ReduceSpec(C.Structure):
    _fields_ = [("is_reduce", C.c_uint8 * MAX_DIM), ("reduce_type", C.c_uint32),
                ("post_reduce_start", C.c_uint32), ("n_post_leaves", C.c_uint32),
                ("reduce2_type", C.c_uint32), ("reduce2_start", C.c_uint32),
                ("is_reduce2", C.c_uint8 * MAX_DIM)]


class KImm(C.Union):
    _fields_ = [("f", C.c_float), ("u", C.c_uint32)]


class KOp(C.Structure):
    _fields_ = [("type", C.c_uint32), ("arg", C.c_uint32 * 3), ("imm", KImm)]


class UOpKernel(C.Structure):
    _fields_ = [("ops", KOp * KOP_MAX), ("n_ops", C.c_uint32), ("n_bufs", C.c_uint32), ("n_leaves", C.c_uint32),
                ("leaf_views", View * MAX_LEAVES), ("leaf_dtypes", C.c_uint32 * MAX_LEAVES),
                ("coord_uop", C.c_uint32 * MAX_DIM), ("rank", C.c_uint32), ("full_shape", Shape),
                ("grid", C.c_uint32 * 3), ("tg", C.c_uint32 * 3), ("local_size", C.c_uint32),
                ("reduce_numel", C.c_uint32), ("out_dtype", C.c_uint32)]


(KOP_NOOP, KOP_GID, KOP_CONST_F, KOP_CONST_U, KOP_RANGE, KOP_ENDRANGE, KOP_LOAD, KOP_STORE, KOP_ALU,
 KOP_ACC_INIT, KOP_ACC, KOP_IDX, KOP_MOD, KOP_DIV, KOP_MASK) = range(15)

assert C.sizeof(Shape) == 36 and C.sizeof(View) == 212 and C.sizeof(Tracker) == 852
assert C.sizeof(ReduceSpec) == 36 and C.sizeof(KOp) == 20


# ---------------------------------------------------------------- view algebra
def make_shape(dims: Sequence[int]) -> Shape:
    s = Shape()
    s.rank = len(dims)
    for i, d in enumerate(dims):
        s.dims[i] = int(d)
    return s


def _finish(v: View) -> View:
    n = 1
    for i in range(v.shape.rank):
        n *= v.shape.dims[i]
        if v.shape.dims[i] == 1:
            v.strides[i] = 0
    v.numel = n & 0xFFFFFFFF
    return v


def _copy(v: View) -> View:
    r = View()
    C.memmove(C.byref(r), C.byref(v), C.sizeof(View))
    return r


def view_contiguous(dims: Sequence[int]) -> View:
    v = View()
    v.shape = make_shape(dims)
    st = 1
    for i in range(len(dims) - 1, -1, -1):
        v.strides[i] = st
        st *= int(dims[i])
    v.contiguous = 1
    return _finish(v)


def view_dims(v: View) -> list[int]:
    return [v.shape.dims[i] for i in range(v.shape.rank)]


def view_strides(v: View) -> list[int]:
    return [v.strides[i] for i in range(v.shape.rank)]


def view_permute(v: View, axes: Sequence[int]) -> View:
    r = _copy(v)
    for i, a in enumerate(axes):
        r.shape.dims[i] = v.shape.dims[a]
        r.strides[i] = v.strides[a]
        r.mask_begin[i] = v.mask_begin[a]
        r.mask_end[i] = v.mask_end[a]
    r.contiguous = 0
    return _finish(r)


def view_expand(v: View, dims: Sequence[int]) -> View:
    """Broadcast size-1 dims (stride 0) up to `dims`."""
    assert len(dims) == v.shape.rank
    r = _copy(v)
    for i, d in enumerate(dims):
        if v.shape.dims[i] != d:
            assert v.shape.dims[i] == 1, "expand only grows size-1 dims"
            r.shape.dims[i] = d
            r.strides[i] = 0
            if r.has_mask:
                r.mask_begin[i], r.mask_end[i] = 0, d
    r.contiguous = 0
    return _finish(r)


def view_reshape(v: View, dims: Sequence[int]) -> View:
    """Reshape where no data movement is needed (merge/split of compatible dims,
    insertion/removal of size-1 dims).  Raises ValueError if a copy is needed."""
    assert not v.has_mask, "reshape of masked views is not modelled here"
    od = [v.shape.dims[i] for i in range(v.shape.rank) if v.shape.dims[i] != 1]
    os_ = [v.strides[i] for i in range(v.shape.rank) if v.shape.dims[i] != 1]
    nd = [int(d) for d in dims]
    if int(np.prod(nd, dtype=np.int64)) != int(np.prod(od, dtype=np.int64)):
        raise ValueError("reshape changes the element count")
    ns = [0] * len(nd)
    oi, oj, ni, nj = 0, 1, 0, 1
    while ni < len(nd) and oi < len(od):
        np_, op = nd[ni], od[oi]
        while np_ != op:
            if np_ < op:
                np_ *= nd[nj]; nj += 1
            else:
                op *= od[oj]; oj += 1
        for ok in range(oi, oj - 1):                      # the merged old dims must be laid out densely
            if os_[ok] != od[ok + 1] * os_[ok + 1]:
                raise ValueError("reshape needs a copy")
        ns[nj - 1] = os_[oj - 1]
        for nk in range(nj - 1, ni, -1):
            ns[nk - 1] = ns[nk] * nd[nk]
        ni, nj, oi, oj = nj, nj + 1, oj, oj + 1
    r = View()
    r.shape = make_shape(nd)
    for i, st in enumerate(ns):
        r.strides[i] = st
    r.offset = v.offset
    r = _finish(r)
    r.contiguous = 1 if (r.offset == 0 and view_strides(r) == view_strides(view_contiguous(nd))) else 0
    return r


def view_pad(v: View, before: Sequence[int], after: Sequence[int]) -> View:
    r = _copy(v)
    r.has_mask = 1
    for i in range(v.shape.rank):
        r.mask_begin[i] = before[i]
        r.mask_end[i] = before[i] + v.shape.dims[i]
        r.shape.dims[i] = v.shape.dims[i] + before[i] + after[i]
        r.offset -= before[i] * v.strides[i]
    r.contiguous = 0
    return _finish(r)


def view_shrink(v: View, begin: Sequence[int], end: Sequence[int]) -> View:
    r = _copy(v)
    for i in range(v.shape.rank):
        r.offset += begin[i] * v.strides[i]
        r.shape.dims[i] = end[i] - begin[i]
        if r.has_mask:
            mb = max(int(v.mask_begin[i]) - begin[i], 0)
            me = max(min(int(v.mask_end[i]), end[i]) - begin[i], 0)
            r.mask_begin[i], r.mask_end[i] = mb, me
    r.contiguous = 0
    return _finish(r)


def view_pool(v: View, kernel: Sequence[int], stride: Sequence[int]) -> View:
    """[..., H, W] -> [..., OH, OW, KH, KW] sliding-window alias of an unmasked view."""
    assert not v.has_mask
    nd = v.shape.rank
    bd = nd - 2
    r = View()
    dims = [v.shape.dims[i] for i in range(bd)]
    o = [(v.shape.dims[bd + j] - kernel[j]) // stride[j] + 1 for j in range(2)]
    dims += o + list(kernel)
    r.shape = make_shape(dims)
    for j in range(bd):
        r.strides[j] = v.strides[j]
    for j in range(2):
        r.strides[bd + j] = v.strides[bd + j] * stride[j]
        r.strides[bd + 2 + j] = v.strides[bd + j]
    r.offset = v.offset
    return _finish(r)


def tracker_of(views: Sequence[View]) -> Tracker:
    t = Tracker()
    t.n_views = len(views)
    for i, v in enumerate(views):
        t.views[i] = v
    return t


def make_reduce(rank: int, axes: Sequence[int], rtype: int, post_start: int = 0, n_post_leaves: int = 0) -> ReduceSpec:
    r = ReduceSpec()
    for a in axes:
        r.is_reduce[a] = 1
    r.reduce_type = rtype
    r.post_reduce_start = post_start
    r.n_post_leaves = n_post_leaves
    return r


# ---------------------------------------------------------------- a dispatch, host side
@dataclass
class Leaf:
    data: np.ndarray                 # 1-D buffer contents, dtype NP_DTYPE[dtype]
    view: View
    dtype: int = F32
    tracker: Optional[Tracker] = None


@dataclass
class Dispatch:
    """Everything `dispatch_kernel_rs` receives, with leaf buffers as host arrays."""
    leaves: list[Leaf]
    ops: list[tuple]                 # (uop, arg_a, arg_b[, aux])
    full: Sequence[int]
    reduce_axes: Sequence[int] = ()
    reduce_type: int = 0
    out_dtype: int = F32
    post_start: int = 0
    n_post_leaves: int = 0
    name: str = ""
    _keep: list = field(default_factory=list, repr=False)

    @property
    def out_numel(self) -> int:
        n = 1
        for d, dim in enumerate(self.full):
            if not (self.reduce_type and d in self.reduce_axes):
                n *= int(dim)
        return n

    def c_args(self):
        """ctypes pieces shared by every implementation of the boundary."""
        n = len(self.leaves)
        views = (C.POINTER(View) * n)(*[C.pointer(l.view) for l in self.leaves])
        any_st = any(l.tracker is not None for l in self.leaves)
        sts = None
        if any_st:
            sts = (C.POINTER(Tracker) * n)()
            for i, l in enumerate(self.leaves):
                if l.tracker is not None:
                    sts[i] = C.pointer(l.tracker)
        ops = (FusedOp * max(len(self.ops), 1))()
        for i, o in enumerate(self.ops):
            ops[i].uop, ops[i].arg_a, ops[i].arg_b = o[0], o[1], o[2]
            ops[i].aux = o[3] if len(o) > 3 else 0
        full = make_shape(self.full)
        red = make_reduce(len(self.full), self.reduce_axes, self.reduce_type, self.post_start,
                          self.n_post_leaves) if self.reduce_type else None
        dts = (C.c_uint32 * n)(*[l.dtype for l in self.leaves])
        self._keep = [views, sts, ops, full, red, dts]
        return views, sts, ops, full, red, dts
