"""Pins for the oracle (CPU only).

1. Golden vectors the reference itself carries for this path, restated as the
   dispatches its scheduler emits for them:
     README.md:106-125      relu(linear(x,w,b))        -> [0, 2.6, 0, 5.0]
     README.md:127-146      d/dw sum(relu(x*w))        -> [5, 7, 9] (closed form)
     docs/step_graph_ic_goal.md:16-22  d/dt sum(t*t)   -> [2, 4, 6]
     test/archive/test_lower_multiview_kernel.m        -> multiview_total = 160.0
     test/archive/test_dtype_cast.m                    -> cast / i32 add / i32 sum / argmax outputs
2. The reference's own CPU backend, compiled from its sources into
   oracle/_ref/ (skipped where the reference checkout is absent): bit-exact on
   every named and fuzzed dispatch, on the signature hash and on f16 conversion.
3. The committed fixtures under tests/golden/, generated from (2) by
   tests/golden/make_golden.py.
"""
from pathlib import Path

import numpy as np
import pytest

import cases
from tinyhvm_b200 import abi
from tinyhvm_b200.abi import ADD, CAST, CMP, F16, F32, I32, MUL, RELU, SUM, U32, Dispatch, Leaf

GOLDEN = Path(__file__).parent / "golden"


def same(a, b):
    """bit-for-bit, treating NaN == NaN"""
    a, b = np.asarray(a), np.asarray(b)
    if a.dtype.kind == "f":
        return a.shape == b.shape and bool(np.all((a == b) | (np.isnan(a) & np.isnan(b))))
    return a.shape == b.shape and bool(np.all(a == b))


# ---- 1. reference golden vectors ------------------------------------------------
def golden_dispatches():
    f = lambda *v: np.array(v, dtype=np.float32)
    out = []
    # relu(linear): C = x@w as [2,3,2] MUL SUM{1}, then ADD bias, RELU
    x, w, b = f(1, 2, 3, 4, 5, 6), f(.1, -.2, .3, .4, -.5, .6), f(-.1, .2)
    mm = Dispatch([Leaf(x, cases.strided([2, 3, 2], [3, 1, 0])), Leaf(w, cases.strided([2, 3, 2], [0, 2, 1]))],
                  [(MUL, 0, 1)], [2, 3, 2], [1], SUM, name="readme_linear_mm")
    out.append(("readme_linear", [mm, lambda y: Dispatch(
        [Leaf(y, abi.view_contiguous([2, 2])), Leaf(b, cases.strided([2, 2], [0, 1]))],
        [(ADD, 0, 1), (RELU, 2, 0)], [2, 2])], f(0, 2.6, 0, 5.0), 1e-6))
    # d/dw sum(relu(x*w)) = sum_rows x * (x*w > 0)
    xw, ww = f(1, 2, 3, 4, 5, 6), f(.1, .2, .3)
    out.append(("readme_autograd", [Dispatch(
        [Leaf(xw, abi.view_contiguous([2, 3])), Leaf(ww, cases.strided([2, 3], [0, 1])), cases.scalar_leaf(0.0, 2)],
        [(MUL, 0, 1), (CMP, 3, 2), (MUL, 0, 4)], [2, 3], [0], SUM)], f(5, 7, 9), 0))
    # d/dt sum(t*t) = t + t
    t = f(1, 2, 3)
    out.append(("doc_grad_square", [Dispatch([Leaf(t, abi.view_contiguous([3]))], [(ADD, 0, 0)], [3])], f(2, 4, 6), 0))
    # pooled 3x3 -> 2x2 windows, doubled, summed over all 8 axes
    x9 = f(*range(1, 10))
    out.append(("multiview_total", [Dispatch([Leaf(x9, cases.strided([1, 1, 1, 1, 2, 2, 2, 2], [0, 0, 0, 0, 3, 1, 3, 1]))],
                                             [(ADD, 0, 0)], [1] * 4 + [2] * 4, list(range(8)), SUM)], f(160.0), 0))
    return out


def run_chain(impl, chain):
    y = None
    for d in chain:
        d = d(y) if callable(d) else d
        y = impl.run(d)
    return y


@pytest.mark.parametrize("name,chain,want,tol", golden_dispatches(), ids=[g[0] for g in golden_dispatches()])
def test_reference_golden_vectors(oracle, name, chain, want, tol):
    got = run_chain(oracle, chain)
    assert np.allclose(got, want, rtol=tol, atol=tol), (name, got, want)


def dtype_cast_dispatches():
    """test/archive/test_dtype_cast.m, as dispatches (expected values from its printed output)."""
    f = lambda *v: np.array(v, dtype=np.float32)
    i = lambda *v: np.array(v, dtype=np.int32)
    v3, v2 = abi.view_contiguous([3]), abi.view_contiguous([2])
    return [
        ("cast_i32", Dispatch([Leaf(f(1.9, -2.1, 3.0), v3)], [(CAST, 0, 0, I32)], [3], out_dtype=I32), i(1, -2, 3)),
        ("cast_f32", Dispatch([Leaf(i(3, -4), v2, I32)], [(CAST, 0, 0, F32)], [2]), f(3.0, -4.0)),
        ("sched_add_i32", Dispatch([Leaf(i(10, -20), v2, I32), Leaf(i(-3, 4), v2, I32)], [(ADD, 0, 1)], [2], out_dtype=I32), i(7, -16)),
        ("sched_sum_i32", Dispatch([Leaf(i(1, 2, 3), v3, I32)], [], [3], [0], SUM, out_dtype=I32), i(6)),
        ("sched_cast_add_i32", Dispatch([Leaf(f(1.9, -2.1, 3.0), v3), Leaf(i(1, 1, 1), v3, I32)],
                                        [(CAST, 0, 0, I32), (ADD, 2, 1)], [3], out_dtype=I32), i(2, -1, 4)),
    ]


@pytest.mark.parametrize("name,d,want", dtype_cast_dispatches(), ids=[c[0] for c in dtype_cast_dispatches()])
def test_reference_dtype_cast_vectors(oracle, name, d, want):
    assert same(oracle.run(d), want)


def test_reference_argmax_vector(oracle):
    import ctypes as C
    x = np.array([1, 9, 2, 8, 7, 3], dtype=np.float32)
    out = np.zeros(2, dtype=np.uint32)
    oracle.lib.oracle_argmax_rows(C.c_void_p(x.ctypes.data), C.c_uint32(2), C.c_uint32(3), C.c_void_p(out.ctypes.data))
    assert out.tolist() == [1, 0]
    assert oracle.lib.oracle_f16_to_f32(oracle.lib.oracle_f32_to_f16(1.0)) == 1.0


# ---- 2. the reference's CPU backend, compiled from source -------------------------
def all_cases():
    rng = np.random.default_rng(20261125)
    cs = cases.named_cases(rng)
    cs += [cases.fuzz_case(s) for s in range(400)]
    cs += [cases.tracker_case(s) for s in range(20)]
    cs += [cases.post_reduce_case(s) for s in range(20)]
    return cs


def test_oracle_matches_reference_cpu_backend(oracle, ref):
    bad = []
    for d in all_cases():
        a, b = oracle.run(d), ref.run(d)
        if not same(a, b):
            bad.append(d.name)
    assert not bad, f"{len(bad)} dispatches differ from the reference CPU backend: {bad[:10]}"


def test_signature_matches_reference(oracle, ref):
    import tinyhvm_b200
    lib = tinyhvm_b200.load()
    import ctypes as C
    for d in all_cases()[:200]:
        want = ref.signature(d)
        assert oracle.signature(d) == want, d.name
        views, sts, ops, full, red, _ = d.c_args()
        got = lib.thvm_cuda_signature(ops, len(d.ops), views, C.cast(sts, C.c_void_p) if sts is not None else None,
                                      len(d.leaves), C.byref(full), C.byref(red) if red is not None else None)
        assert got == want, d.name


def test_f16_conversion_matches_reference(oracle, ref):
    for h in range(0, 65536):
        a, b = oracle.lib.oracle_f16_to_f32(h), ref.lib.ref_f16_to_f32(h)
        assert a == b or (a != a and b != b), hex(h)
    rng = np.random.default_rng(7)
    xs = np.concatenate([rng.standard_normal(20000) * 10 ** rng.uniform(-9, 6, 20000),
                         [0.0, -0.0, 65504.0, 65520.0, 1e10, -1e10, 6e-8, 5.96e-8, 2.98e-8, np.inf, -np.inf, np.nan]]).astype(np.float32)
    for x in xs:
        assert oracle.lib.oracle_f32_to_f16(float(x)) == ref.lib.ref_f32_to_f16(float(x)), float(x)


# ---- 3. committed fixtures ---------------------------------------------------------
def golden_case_list():
    """(key, dispatch) pairs in the order make_golden.py stores them."""
    rng = np.random.default_rng(4242)
    cs = cases.named_cases(rng) + [cases.fuzz_case(s) for s in range(1000, 1120)]
    cs += [cases.tracker_case(s) for s in range(100, 108)] + [cases.post_reduce_case(s) for s in range(100, 108)]
    return [(f"{i:03d}_{d.name}", d) for i, d in enumerate(cs)]


def test_oracle_matches_committed_fixtures(oracle):
    z = np.load(GOLDEN / "boundary_cases.npz")
    pairs = golden_case_list()
    assert len(pairs) == len(z.files)
    for key, d in pairs:
        assert same(oracle.run(d), z[key]), key
