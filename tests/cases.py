"""Dispatches used by the parity tests.

`named_cases()` are the patterns the reference's scheduler really hands to a
backend (captured at the vtable: matmul and its two backward forms, bias+relu,
conv fprop / wgrad as MUL+SUM over pooled views, 2x2 max-pool as RMAX, batch-norm
statistics, pad materialisation, bias gradient, soft-max pieces), at small sizes.
`fuzz_case(seed)` draws random-but-valid dispatches: rank 1..8, random op DAGs,
permuted / broadcast / padded / pooled leaves, stacked views, all dtypes,
reductions over any axis subset, post-reduce ops.
"""
from __future__ import annotations

import numpy as np

from tinyhvm_b200 import abi
from tinyhvm_b200.abi import (ADD, CAST, CMP, DIV, EXP, F16, F32, I32, LOG, MAX, MUL, NEG, RELU, RMAX, SQRT, SUB,
                              SUM, U32, Dispatch, Leaf)


def _f32(rng, n, lo=-2.0, hi=2.0):
    return rng.uniform(lo, hi, size=n).astype(np.float32)


def dense(rng, dims, **kw):
    return Leaf(_f32(rng, int(np.prod(dims)), **kw), abi.view_contiguous(dims))


def scalar_leaf(value, rank):
    """A 1-element tensor broadcast over a rank-`rank` iteration space."""
    v = abi.view_contiguous([1] * rank)
    return Leaf(np.array([value], dtype=np.float32), v)


# ------------------------------------------------------------------ named cases
def strided(full, strides, offset=0):
    """A view over the iteration shape `full` with explicit element strides."""
    v = abi.View()
    v.shape = abi.make_shape(full)
    for i, st in enumerate(strides):
        v.strides[i] = st
    v.offset = offset
    return abi._finish(v)


def mm_case(rng, M, K, N, ta=False, tb=False):
    """C = A@B as [M,K,N] MUL + SUM{1}; a transposed operand has swapped strides."""
    a = _f32(rng, M * K, -1, 1)
    b = _f32(rng, K * N, -1, 1)
    va = strided([M, K, N], [1, M, 0] if ta else [K, 1, 0])     # ta: A stored as [K,M]
    vb = strided([M, K, N], [0, 1, K] if tb else [0, N, 1])     # tb: B stored as [N,K]
    return Dispatch([Leaf(a, va), Leaf(b, vb)], [(MUL, 0, 1)], [M, K, N], [1], SUM,
                    name=f"mm_{M}x{K}x{N}{'_ta' if ta else ''}{'_tb' if tb else ''}")


def bias_relu_case(rng, M, N):
    y = dense(rng, [M, N])
    b = Leaf(_f32(rng, N), abi.view_expand(abi.view_contiguous([1, N]), [M, N]))
    return Dispatch([y, b], [(ADD, 0, 1), (RELU, 2, 0)], [M, N], name=f"bias_relu_{M}x{N}")


def chain_fwd_case(rng, R, Cc):
    """config-2 forward: sum over the last axis of relu(a*b+c)."""
    ls = [Leaf(rng.standard_normal(R * Cc).astype(np.float32), abi.view_contiguous([R, Cc])) for _ in range(3)]
    return Dispatch(ls, [(MUL, 0, 1), (ADD, 3, 2), (RELU, 4, 0)], [R, Cc], [1], SUM, name=f"chain_fwd_{R}x{Cc}")


def chain_bwd_case(rng, R, Cc):
    """config-2 VJP w.r.t. a with a ones seed: g = b * (a*b+c > 0)."""
    ls = [Leaf(rng.standard_normal(R * Cc).astype(np.float32), abi.view_contiguous([R, Cc])) for _ in range(3)]
    ls.append(scalar_leaf(0.0, 2))
    return Dispatch(ls, [(MUL, 0, 1), (ADD, 4, 2), (CMP, 5, 3), (MUL, 1, 6)], [R, Cc], name=f"chain_bwd_{R}x{Cc}")


def conv_fprop_case(rng, B, Ci, H, W, Co, K):
    OH, OW = H - K + 1, W - K + 1
    x = _f32(rng, B * Ci * H * W, -1, 1)
    w = _f32(rng, Co * Ci * K * K, -1, 1)
    full = [B, 1, Co, OH, OW, Ci, K, K]
    vx = abi.View()
    vx.shape = abi.make_shape(full)
    for i, s in enumerate([Ci * H * W, 0, 0, W, 1, H * W, W, 1]):
        vx.strides[i] = s
    vx = abi._finish(vx)
    vw = abi.View()
    vw.shape = abi.make_shape(full)
    for i, s in enumerate([0, 0, Ci * K * K, 0, 0, K * K, K, 1]):
        vw.strides[i] = s
    vw = abi._finish(vw)
    return Dispatch([Leaf(x, vx), Leaf(w, vw)], [(MUL, 0, 1)], full, [5, 6, 7], SUM,
                    name=f"conv_fprop_b{B}c{Ci}h{H}w{W}o{Co}k{K}")


def conv_wgrad_case(rng, B, Ci, H, W, Co, K):
    OH, OW = H - K + 1, W - K + 1
    x = _f32(rng, B * Ci * H * W, -1, 1)
    g = _f32(rng, B * Co * OH * OW, -1, 1)
    full = [B, Co, Ci, OH, OW, K, K]
    vx, vg = abi.View(), abi.View()
    vx.shape = abi.make_shape(full)
    vg.shape = abi.make_shape(full)
    for i, s in enumerate([Ci * H * W, 0, H * W, W, 1, W, 1]):
        vx.strides[i] = s
    for i, s in enumerate([Co * OH * OW, OH * OW, 0, OW, 1, 0, 0]):
        vg.strides[i] = s
    return Dispatch([Leaf(x, abi._finish(vx)), Leaf(g, abi._finish(vg))], [(MUL, 0, 1)], full, [0, 3, 4], SUM,
                    name=f"conv_wgrad_b{B}c{Ci}h{H}w{W}o{Co}k{K}")


def maxpool_case(rng, B, Cc, H, W, ties=False):
    OH, OW = H // 2, W // 2
    x = _f32(rng, B * Cc * H * W)
    if ties:
        x = np.round(x)                      # many equal values inside a window
    v = abi.View()
    full = [B, Cc, OH, OW, 2, 2]
    v.shape = abi.make_shape(full)
    for i, s in enumerate([Cc * H * W, H * W, 2 * W, 2, W, 1]):
        v.strides[i] = s
    return Dispatch([Leaf(x, abi._finish(v))], [], full, [4, 5], RMAX, name=f"maxpool_b{B}c{Cc}h{H}w{W}")


def maxpool_bwd_case(rng, B, Cc, H, W, ties=False):
    """Mask-form gradient of the 2x2 pool in window layout: g * (1 - (max > x)) over [B,C,OH,OW,2,2]."""
    from tinyhvm_b200.abi import CMP, SUB
    OH, OW = H // 2, W // 2
    x = _f32(rng, B * Cc * H * W)
    if ties:
        x = np.round(x)
    mx = x.reshape(B, Cc, OH, 2, OW, 2).max(axis=(3, 5)).ravel().astype(np.float32)
    g = _f32(rng, B * Cc * OH * OW)
    full = [B, Cc, OH, OW, 2, 2]
    vx = strided(full, [Cc * H * W, H * W, 2 * W, 2, W, 1])
    vp = strided(full, [Cc * OH * OW, OH * OW, OW, 1, 0, 0])
    return Dispatch([Leaf(g, vp), scalar_leaf(1.0, 6), Leaf(mx, vp), Leaf(x, vx)], [(CMP, 2, 3), (SUB, 1, 4), (MUL, 0, 5)], full,
                    name=f"maxpool_bwd_b{B}c{Cc}h{H}w{W}")


def bn_stats_case(rng, B, Cc, H, W):
    return Dispatch([dense(rng, [B, Cc, H, W])], [], [B, Cc, H, W], [0, 2, 3], SUM, name=f"bn_stats_b{B}c{Cc}h{H}w{W}")


def bn_var_case(rng, B, Cc, H, W):
    """sum((x-mean)^2) over axes 0,2,3 with a [1,C,1,1] mean leaf (rebuilt twice: tree-shaped)."""
    x = dense(rng, [B, Cc, H, W])
    mean = Leaf(_f32(rng, Cc, -0.1, 0.1), abi.view_expand(abi.view_contiguous([1, Cc, 1, 1]), [B, Cc, H, W]))
    return Dispatch([x, mean], [(SUB, 0, 1), (SUB, 0, 1), (MUL, 2, 3)], [B, Cc, H, W], [0, 2, 3], SUM,
                    name=f"bn_var_b{B}c{Cc}h{H}w{W}")


def bn_apply_case(rng, B, Cc, H, W):
    x = dense(rng, [B, Cc, H, W])
    per_c = lambda lo, hi: Leaf(_f32(rng, Cc, lo, hi), abi.view_expand(abi.view_contiguous([1, Cc, 1, 1]), [B, Cc, H, W]))
    mean, invstd, gamma, beta = per_c(-0.1, 0.1), per_c(0.5, 2), per_c(0.5, 1.5), per_c(-0.5, 0.5)
    ops = [(SUB, 0, 1), (MUL, 5, 2), (MUL, 6, 3), (ADD, 7, 4), (RELU, 8, 0)]
    return Dispatch([x, mean, invstd, gamma, beta], ops, [B, Cc, H, W], name=f"bn_apply_relu_b{B}c{Cc}h{H}w{W}")


def pad_case(rng, B, Cc, H, W, p):
    x = dense(rng, [B, Cc, H, W])
    x.view = abi.view_pad(x.view, [0, 0, p, p], [0, 0, p, p])
    full = [B, Cc, H + 2 * p, W + 2 * p]
    return Dispatch([x, scalar_leaf(0.0, 4)], [(ADD, 0, 1)], full, name=f"pad_b{B}c{Cc}h{H}w{W}p{p}")


def crop_case(rng, B, Cc, H, W, p, q=None):
    """ADD(shrink(x), 0): the H x W window at (p, q) of every (H + 2p) x (W + 2q) plane, as a convolution's input
    gradient is cut out of its padded form."""
    q = p if q is None else q
    x = dense(rng, [B, Cc, H + 2 * p, W + 2 * q])
    x.view = abi.view_shrink(x.view, [0, 0, p, q], [B, Cc, p + H, q + W])
    return Dispatch([x, scalar_leaf(0.0, 4)], [(ADD, 0, 1)], [B, Cc, H, W], name=f"crop_b{B}c{Cc}h{H}w{W}p{p}q{q}")


def bias_grad_case(rng, M, N):
    return Dispatch([dense(rng, [M, N])], [], [M, N], [0], SUM, name=f"bias_grad_{M}x{N}")


def rowmax_case(rng, M, N):
    return Dispatch([dense(rng, [M, N])], [], [M, N], [1], RMAX, name=f"rowmax_{M}x{N}")


def softmax_sum_case(rng, M, N):
    l = dense(rng, [M, N])
    m = Leaf(_f32(rng, M, 1.5, 2.5), abi.view_expand(abi.view_contiguous([M, 1]), [M, N]))
    return Dispatch([l, m], [(SUB, 0, 1), (EXP, 2, 0)], [M, N], [1], SUM, name=f"softmax_sum_{M}x{N}")


def total_sum_case(rng, M, N):
    return Dispatch([dense(rng, [M, N]), dense(rng, [M, N])], [(MUL, 0, 1)], [M, N], [0, 1], SUM, name=f"total_sum_{M}x{N}")


def permute_copy_case(rng, dims, axes):
    x = dense(rng, dims)
    x.view = abi.view_permute(x.view, axes)
    return Dispatch([x, scalar_leaf(0.0, len(dims))], [(ADD, 0, 1)], abi.view_dims(x.view), name=f"permute_copy_{dims}_{axes}")


def named_cases(rng):
    return [
        mm_case(rng, 4, 5, 6), mm_case(rng, 33, 70, 17), mm_case(rng, 8, 300, 8),
        mm_case(rng, 16, 12, 20, ta=True), mm_case(rng, 16, 12, 20, tb=True), mm_case(rng, 64, 128, 10),
        bias_relu_case(rng, 64, 128), bias_relu_case(rng, 7, 13),
        chain_fwd_case(rng, 16, 32), chain_fwd_case(rng, 5, 1000), chain_fwd_case(rng, 3, 4100),
        chain_bwd_case(rng, 16, 32), chain_bwd_case(rng, 9, 77),
        conv_fprop_case(rng, 2, 3, 8, 8, 4, 3), conv_fprop_case(rng, 3, 1, 12, 12, 6, 5),
        conv_wgrad_case(rng, 2, 3, 8, 8, 4, 3),
        maxpool_case(rng, 2, 4, 6, 6), maxpool_case(rng, 3, 6, 28, 28), maxpool_case(rng, 2, 3, 8, 8, ties=True),
        bn_stats_case(rng, 4, 8, 6, 6), bn_stats_case(rng, 16, 3, 20, 20), bn_var_case(rng, 4, 8, 6, 6),
        bn_apply_case(rng, 4, 8, 6, 6),
        pad_case(rng, 2, 3, 8, 8, 1), pad_case(rng, 2, 1, 28, 28, 2),
        bias_grad_case(rng, 64, 10), bias_grad_case(rng, 1000, 37),
        rowmax_case(rng, 64, 10), softmax_sum_case(rng, 64, 10), total_sum_case(rng, 37, 41),
        permute_copy_case(rng, [2, 3, 4, 2, 5, 2], [0, 1, 2, 4, 3, 5]), permute_copy_case(rng, [17, 33], [1, 0]),
    ]


# ------------------------------------------------------------------ fuzzer
_UN = [NEG, EXP, LOG, RELU, SQRT, CAST]
_BIN = [ADD, MUL, DIV, MAX, CMP, SUB]


def _random_leaf(rng, full, dtype):
    """A leaf whose view covers `full` through some mix of contiguous, permuted,
    broadcast, padded (masked, negative offset) or pooled addressing."""
    rank = len(full)
    kind = rng.choice(["dense", "dense", "perm", "bcast", "bcast", "pad", "scalar", "offset"])
    npdt = abi.NP_DTYPE[dtype]

    def data(n):
        if dtype == F32:
            return _f32(rng, n)
        if dtype == F16:
            return np.array([abi_f16(x) for x in _f32(rng, n)], dtype=np.uint16)
        if dtype == I32:
            return rng.integers(-50, 50, size=n).astype(np.int32)
        return rng.integers(0, 100, size=n).astype(np.uint32)

    if kind == "scalar":
        return Leaf(data(1), abi.view_contiguous([1] * rank), dtype)
    if kind == "perm" and rank >= 2:
        axes = list(rng.permutation(rank))
        src = [0] * rank
        for i, a in enumerate(axes):
            src[a] = full[i]
        v = abi.view_permute(abi.view_contiguous(src), axes)
        return Leaf(data(int(np.prod(full))), v, dtype)
    if kind == "bcast":
        keep = rng.random(rank) < 0.5
        small = [d if k else 1 for d, k in zip(full, keep)]
        v = abi.view_expand(abi.view_contiguous(small), full)
        return Leaf(data(int(np.prod(small))), v, dtype)
    if kind == "pad":
        before = [int(rng.integers(0, min(3, d))) for d in full]
        after = [int(rng.integers(0, min(3, d - b))) for d, b in zip(full, before)]
        inner = [d - b - a for d, b, a in zip(full, before, after)]
        if all(i >= 1 for i in inner):
            v = abi.view_pad(abi.view_contiguous(inner), before, after)
            return Leaf(data(int(np.prod(inner))), v, dtype)
    if kind == "offset":
        extra = int(rng.integers(1, 9))
        v = abi.view_contiguous(full)
        v.offset = extra
        v.contiguous = 0
        return Leaf(data(int(np.prod(full)) + extra), v, dtype)
    return Leaf(data(int(np.prod(full))), abi.view_contiguous(full), dtype)


def abi_f16(x: float) -> int:
    """IEEE half bits via numpy (inputs only; the conversion under test is the library's)."""
    return int(np.float16(x).view(np.uint16))


def fuzz_case(seed: int) -> Dispatch:
    rng = np.random.default_rng(seed)
    rank = int(rng.integers(1, 9))
    budget = int(rng.choice([64, 500, 4000, 20000]))
    full = []
    for _ in range(rank):
        hi = max(1, int(budget ** (1.0 / rank) * 1.8))
        full.append(int(rng.integers(1, hi + 1)))
    n_leaves = int(rng.integers(1, 5))
    dts = [F32 if rng.random() < 0.7 else int(rng.choice([F16, I32, U32])) for _ in range(n_leaves)]
    leaves = [_random_leaf(rng, full, dt) for dt in dts]
    n_ops = int(rng.integers(0, 7))
    ops = []
    for i in range(n_ops):
        avail = n_leaves + i
        if rng.random() < 0.4:
            u = int(rng.choice(_UN))
            a = int(rng.integers(0, avail))
            aux = int(rng.choice([F32, F16, I32, U32])) if u == CAST else 0
            ops.append((u, a, 0 if rng.random() < 0.5 else a, aux))
        else:
            ops.append((int(rng.choice(_BIN)), int(rng.integers(0, avail)), int(rng.integers(0, avail)), 0))
    if n_ops:                                   # make the last op depend on the previous value chain a bit
        u, a, b, aux = ops[-1]
        ops[-1] = (u, n_leaves + n_ops - 2 if n_ops > 1 else a, b, aux)
    red_type, axes = 0, []
    if rng.random() < 0.55:
        red_type = int(rng.choice([SUM, RMAX]))
        axes = [d for d in range(rank) if rng.random() < 0.5] or [rank - 1]
    out_dtype = F32 if rng.random() < 0.8 else int(rng.choice([F16, I32, U32]))
    return Dispatch(leaves, ops, full, axes, red_type, out_dtype, name=f"fuzz_{seed}")


def tracker_case(seed: int) -> Dispatch:
    """A leaf addressed through two stacked views: permute then a rank-changing reshape."""
    rng = np.random.default_rng(seed)
    a, b, c = (int(rng.integers(2, 6)) for _ in range(3))
    inner = abi.view_permute(abi.view_contiguous([a, b, c]), [2, 0, 1])          # shape [c,a,b]
    outer = abi.view_contiguous([c * a, b])
    x = Leaf(_f32(rng, a * b * c), outer, F32, abi.tracker_of([inner, outer]))
    y = dense(rng, [c * a, b])
    red = bool(rng.integers(0, 2))
    return Dispatch([x, y], [(ADD, 0, 1)], [c * a, b], [1] if red else [], SUM if red else 0, name=f"tracker_{seed}")


def post_reduce_case(seed: int) -> Dispatch:
    """Legacy form: pre-reduce ops, SUM, then ops on the reduced value with a post-reduce leaf."""
    rng = np.random.default_rng(seed)
    M, N = int(rng.integers(2, 9)), int(rng.integers(2, 40))
    x, y = dense(rng, [M, N]), dense(rng, [M, N])
    s = Leaf(_f32(rng, M, 0.5, 2.0), abi.view_contiguous([M, 1]))
    # ops: 0: MUL(x,y) | post: 1: MUL(reduced, s)  2: ADD(op1, s)
    ops = [(MUL, 0, 1), (MUL, 3, 2), (ADD, 4, 2)]
    return Dispatch([x, y, s], ops, [M, N], [1], SUM, post_start=1, n_post_leaves=1, name=f"post_reduce_{seed}")
