"""Parity on the shapes that are benchmarked (all through the C ABI, on a B200).

The small-shape parity tests establish that every kernel family agrees with the
oracle; the cases here run the very dispatches `bench.py` times, at their full
sizes, where the scalar CPU interpreter would need hours:

  * config 2 at 8192 x 8192: every row of the forward chain against float64 row
    sums (1e-5), every element of the VJP bit for bit against numpy;
  * config 3: the three 4096^3 GEMMs, 64 sampled rows and 64 sampled columns of
    each result against float64 (1e-4 of |exact sum| + rms of the result);
  * configs 4 and 5: every MUL+SUM contraction of the committed LeNet / VGG step
    programs (tinyhvm_b200/traces: the dispatches the reference's scheduler emits
    for those steps, at per-GPU batches 1024 / 128 and 512 / 64) on seeded random
    operands, a few hundred sampled outputs each against a float64 evaluation of
    exactly those outputs through the dispatch's own views;
  * whole steps of the committed programs, replayed call by call and as a captured
    CUDA graph, against torch-CPU autograd on the same synthetic batches: loss and
    every updated parameter against the f32 run (1e-4 LeNet, 2e-3 for the
    batch-normalised net, the tolerances of the same-program tests), every gradient
    against a float64 run (see the comment at the check: at these sizes gradients are
    limited by relu / max-pool decisions that flip under last-bit differences).  The
    staged programs themselves are proven equal to torch autograd at small sizes by
    tests/test_host_dropin.py.
"""
import zlib

import numpy as np
import pytest

from tinyhvm_b200 import abi, configs, replay, synth
from tinyhvm_b200.abi import ADD, CMP, MUL, RELU, SUM, Dispatch, Leaf

pytestmark = pytest.mark.gpu


def close(a, b, rtol):
    """|a-b| <= rtol * (|b| + rms(b)) elementwise (the measure of the same-program tests)"""
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    if a.shape != b.shape:
        return False
    rms = np.sqrt(np.mean(b ** 2)) if b.size else 0.0
    return bool(np.all(np.abs(a - b) <= rtol * (np.abs(b) + rms) + 1e-30))


# ------------------------------------------------------------------ config 2 at full size
def test_chain_config_full_size_every_row(cuda):
    R = Cc = 8192
    seed = synth.SEED_BASE + 2
    a, b, c = (synth.normal(seed, t, R * Cc) for t in range(3))
    v = abi.view_contiguous([R, Cc])
    la, lb, lc = Leaf(a, v), Leaf(b, v), Leaf(c, v)
    zero = Leaf(np.zeros(1, np.float32), abi.view_contiguous([1, 1]))
    fwd = Dispatch([la, lb, lc], [(MUL, 0, 1), (ADD, 3, 2), (RELU, 4, 0)], [R, Cc], [1], SUM, name="chain_fwd_full")
    bwd = Dispatch([la, lb, lc, zero], [(MUL, 0, 1), (ADD, 4, 2), (CMP, 5, 3), (MUL, 1, 6)], [R, Cc], name="chain_bwd_full")
    cuda.reset(0)
    ids = [cuda.upload(x) for x in (a, b, c)]
    zid = cuda.upload(zero.data)
    y_id, g_id = cuda.alloc(R * 4), cuda.alloc(R * Cc * 4)
    cuda.dispatch_ids(y_id, ids, fwd)
    assert cuda.last_plan() == "reduce_rows_cta", cuda.last_plan()      # the kernel the headline number times
    cuda.dispatch_ids(g_id, ids + [zid], bwd)
    assert cuda.last_plan() == "ew_flat_static", cuda.last_plan()
    y = cuda.read(y_id, np.float32, R)
    g = cuda.read(g_id, np.float32, R * Cc)
    cuda.reset(0)
    u = a * b + c                                                       # f32, one rounding per op as on the device
    assert np.array_equal(g, np.where(u > 0, b, np.float32(0))), "VJP is not bit-exact"
    exact = np.maximum(u, 0).reshape(R, Cc).sum(axis=1, dtype=np.float64)
    err = np.abs(y.astype(np.float64) - exact)
    assert np.all(err <= 1e-5 * np.abs(exact)), f"forward: {np.max(err / np.abs(exact)):.2e} relative"
    assert cuda.last_error() == ""


# ------------------------------------------------------------------ config 3 at full size
def test_gemm_config_full_size_sampled_rows_and_columns(cuda):
    import bench
    n = 4096
    seed = synth.SEED_BASE + 3
    A, B, dC = (synth.normal(seed, t, n * n) / np.float32(np.sqrt(n)) for t in range(3))
    ds = bench.gemm_dispatches(n, A, B, dC)
    cuda.reset(0)
    ids = {k: cuda.upload(v) for k, v in (("A", A), ("B", B), ("dC", dC))}
    out = cuda.alloc(n * n * 4)
    leaf_ids = {"C=A@B": [ids["A"], ids["B"]], "dA=dC@B^T": [ids["dC"], ids["B"]], "dB=A^T@dC": [ids["A"], ids["dC"]]}
    A64, B64, dC64 = (x.reshape(n, n).astype(np.float64) for x in (A, B, dC))
    forms = {"C=A@B": (A64, B64), "dA=dC@B^T": (dC64, B64.T), "dB=A^T@dC": (A64.T, dC64)}
    rng = np.random.default_rng(3)
    for name, d in ds.items():
        cuda.dispatch_ids(out, leaf_ids[name], d)
        assert cuda.last_plan().startswith("gemm"), cuda.last_plan()
        got = cuda.read(out, np.float32, n * n).reshape(n, n).astype(np.float64)
        L, Rm = forms[name]
        rows, cols = rng.choice(n, 64, replace=False), rng.choice(n, 64, replace=False)
        want_rows, want_cols = L[rows] @ Rm, L @ Rm[:, cols]
        rms = float(np.sqrt(np.mean(want_rows ** 2)))
        for g_, w in ((got[rows], want_rows), (got[:, cols], want_cols)):
            err = np.abs(g_ - w)
            # 1e-4 of the exact sum; sums that cancel towards zero are measured against the rms of the result instead
            # (the measure of the same-program tests: |err| <= rtol * (|exact| + rms))
            bound = 1e-4 * (np.abs(w) + rms)
            assert np.all(err <= bound), f"{name}: {np.max(err / bound):.2f}x over 1e-4 of the exact sum"
            assert np.max(err) <= 6e-5 * rms, f"{name}: worst error {np.max(err) / rms:.2e} of the output rms"
    cuda.reset(0)
    assert cuda.last_error() == ""


# ------------------------------------------------------------------ configs 4 / 5: the contractions of the committed step programs
def view_extent(v):
    """(lowest, highest) element offset the view can address"""
    lo = hi = int(v.offset)
    for d in range(v.shape.rank):
        e = int(v.strides[d]) * (int(v.shape.dims[d]) - 1)
        if e < 0:
            lo += e
        else:
            hi += e
    return lo, hi


def trace_contractions(trace):
    """The distinct MUL+SUM dispatches over two unmasked single-view f32 leaves of a step program's steady-state cycle."""
    recs = replay.load_trace(replay.TRACE_DIR / f"{trace}.thtr.gz")
    _, cycles = replay.split_steps(recs)
    seen, out = set(), []
    for r in cycles[1]:
        if r.op != replay.DISPATCH:
            continue
        a = replay.DispatchArgs(r.blob)
        if not (a.n == 2 and a.n_ops == 1 and a.ops[0].uop == MUL and a.has_red and a.red.reduce_type == SUM and a.sts is None):
            continue
        if any(a.views[i].has_mask or a.dts[i] != abi.F32 for i in range(2)) or a.out_dt != abi.F32:
            continue
        key = (bytes(a.full), bytes(a.red), bytes(a.views))
        if key in seen:
            continue
        seen.add(key)
        out.append(a)
    return out


def sampled_exact(a, leaves, picks):
    """float64 value of the sampled outputs of a MUL+SUM dispatch, addressed through its own views"""
    rank = a.full.rank
    dims = [int(a.full.dims[d]) for d in range(rank)]
    kept = [d for d in range(rank) if not a.red.is_reduce[d]]
    red = [d for d in range(rank) if a.red.is_reduce[d]]
    rdims = [dims[d] for d in red]
    ridx = np.indices(rdims, dtype=np.int64).reshape(len(red), -1) if red else np.zeros((0, 1), np.int64)
    roff = []
    for i in range(2):
        v = a.views[i]
        o = np.zeros(ridx.shape[1], np.int64)
        for k, d in enumerate(red):
            if int(v.shape.dims[d]) != 1:
                o += ridx[k] * int(v.strides[d])
        roff.append(o)
    kdims = [dims[d] for d in kept]
    out = np.empty(len(picks), np.float64)
    for j, flat in enumerate(picks):
        coords = np.unravel_index(int(flat), kdims) if kdims else ()
        base = []
        for i in range(2):
            v = a.views[i]
            o = int(v.offset)
            for cval, d in zip(coords, kept):
                if int(v.shape.dims[d]) != 1:
                    o += int(cval) * int(v.strides[d])
            base.append(o)
        out[j] = np.dot(leaves[0][base[0] + roff[0]].astype(np.float64), leaves[1][base[1] + roff[1]].astype(np.float64))
    return out


@pytest.mark.parametrize("trace", ["vgg_b512", "vgg_b64", "lenet_b1024", "lenet_b128"])
def test_contractions_of_the_committed_step_programs(cuda, trace):
    rng = np.random.default_rng(zlib.crc32(trace.encode()))
    todo = trace_contractions(trace)
    assert len(todo) >= (8 if trace.startswith("vgg") else 5), len(todo)
    plans = {}
    t = replay.CudaTarget(cuda)
    for a in todo:
        cuda.reset(0)
        leaves, ids = [], []
        for i in range(2):
            lo, hi = view_extent(a.views[i])
            assert lo >= 0
            x = rng.standard_normal(hi + 1, dtype=np.float32)
            leaves.append(x)
            ids.append(cuda.upload(x))
        dims = [int(a.full.dims[d]) for d in range(a.full.rank)]
        n_out = int(np.prod([dims[d] for d in range(a.full.rank) if not a.red.is_reduce[d]]))
        K = int(np.prod([dims[d] for d in range(a.full.rank) if a.red.is_reduce[d]]))
        out = cuda.alloc(n_out * 4)
        a.out = out
        for i in range(2):
            a.ids[i] = ids[i]
        t.dispatch(a)
        plan = cuda.last_plan()
        plans[plan] = plans.get(plan, 0) + 1
        got = cuda.read(out, np.float32, n_out).astype(np.float64)
        assert cuda.last_error() == "", (dims, cuda.last_error())
        picks = rng.choice(n_out, min(n_out, 256 if K <= (1 << 18) else 96), replace=False)
        want = sampled_exact(a, leaves, picks)
        scale = np.sqrt(K)                                               # rms of a sum of K products of N(0,1) operands
        err = np.abs(got[picks] - want)
        bound = 1e-4 * (np.abs(want) + scale)                             # |err| <= rtol * (|exact| + rms), as above
        assert np.all(err <= bound), f"{trace} full={dims} plan={plan}: {np.max(err / bound):.2f}x over 1e-4 of the exact sum"
    cuda.reset(0)
    print(trace, "plans:", plans)
    assert all(p.startswith("gemm") or p.startswith("contract") or p.startswith("reduce") for p in plans), plans


# ------------------------------------------------------------------ configs 4 / 5: whole steps against torch autograd
class GradTap(replay.CudaTarget):
    """The CUDA library with one addition: right after the step's gradient sum the gradient buffers are read back."""

    def __init__(self, backend):
        super().__init__(backend)
        self.grads, self.enabled = None, True

    def allreduce(self, ids, counts):
        super().allreduce(ids, counts)
        if self.enabled:                                   # (a read while a step is being captured would become a graph result)
            self.grads = [self.be.read(i, np.float32, int(n)) for i, n in zip(ids, counts)]


def noisy(c, noise, gen):
    """c + noise * rms(c) * N(0,1): a convolution that is off by `noise` of its output scale"""
    import torch
    if not noise:
        return c
    return c + noise * c.detach().pow(2).mean().sqrt() * torch.randn(c.shape, generator=gen, dtype=c.dtype)


def torch_lenet(tp, x, lab, noise=0.0, gen=None):
    import torch
    F = torch.nn.functional
    B = lab.size
    tx = torch.from_numpy(x.reshape(B, 1, 28, 28)).to(tp[0].dtype)
    h = F.max_pool2d(torch.relu(noisy(F.conv2d(tx, tp[0], tp[1], padding=2), noise, gen)), 2)
    h = F.max_pool2d(torch.relu(noisy(F.conv2d(h, tp[2], tp[3]), noise, gen)), 2).reshape(B, 400)
    h = torch.relu(torch.relu(h @ tp[4] + tp[5]) @ tp[6] + tp[7])
    return F.cross_entropy(h @ tp[8] + tp[9], torch.from_numpy(lab.astype(np.int64)))


def torch_vgg(tp, x, lab, noise=0.0, gen=None):
    import torch
    F = torch.nn.functional
    B = lab.size
    a = torch.from_numpy(x.reshape(B, 3, 64, 64)).to(tp[0].dtype)
    for l in range(6):
        a = torch.relu(F.batch_norm(noisy(F.conv2d(a, tp[3 * l], padding=1), noise, gen), None, None, tp[3 * l + 1], tp[3 * l + 2],
                                    training=True, eps=1e-5))
        if l & 1:
            a = F.max_pool2d(a, 2)
    return F.cross_entropy(a.reshape(B, -1) @ tp[18] + tp[19], torch.from_numpy(lab.astype(np.int64)))


STEP_CASES = {
    "lenet_b1024": ("lenet", 1024, 1e-4), "lenet_b128": ("lenet", 128, 1e-4),
    "vgg_b512": ("vgg", 512, 2e-3), "vgg_b64": ("vgg", 64, 2e-3),
}


@pytest.mark.parametrize("trace", list(STEP_CASES))
def test_committed_step_programs_match_torch_autograd(cuda, trace):
    """Steps 0 and 1 call by call (gradients tapped at step 1), step 2 as a launch of the captured graph."""
    import torch
    model, B, rtol = STEP_CASES[trace]
    lr = 0.01
    if model == "lenet":
        names, shapes, ps, E, classes, fwd = configs.LENET_NAMES, configs.LENET_SHAPES, configs.lenet_params(), 784, 10, torch_lenet
        gen, seed = synth.uniform, synth.SEED_BASE + 4
    else:
        (shapes, names), ps, E, classes, fwd = configs.vgg_shapes(), configs.vgg_params(), 3 * 64 * 64, 100, torch_vgg
        gen, seed = synth.normal, synth.SEED_BASE + 5
    xs = [gen(seed, 300 + k, B * E) for k in range(3)]
    labs = [synth.labels(seed, 400 + k, B, classes) for k in range(3)]
    lrv = np.array([lr], dtype=np.float32)
    ext = lambda k: {"x": xs[k], "onehot": configs.onehot(labs[k], classes), "lr": lrv}

    recs = replay.load_trace(replay.TRACE_DIR / f"{trace}.thtr.gz")
    cuda.reset(0)
    tap = GradTap(cuda)
    rp = replay.Replayer(tap, recs)
    rp.run_prefix(dict(zip(names, ps)))
    read_params = lambda: [cuda.read(k + 1, np.float32, int(np.prod(s))) for k, s in enumerate(shapes)]
    got = {"loss": [], "params": []}
    got["loss"].append(float(rp.run(rp.cycles[0], ext(0))["loss"][0]))
    got["params"].append(read_params())
    got["loss"].append(float(rp.run(rp.cycles[1], ext(1))["loss"][0]))
    grads1 = tap.grads
    got["params"].append(read_params())
    tap.enabled = False
    step = rp.capture(rp.cycles[1], ext(2))
    step.launch(ext(2))
    got["loss"].append(float(step.results()["loss"][0]))
    got["params"].append(read_params())
    step.destroy()
    cuda.reset(0)
    assert cuda.last_error() == ""

    tp = [torch.tensor(p.reshape(s), requires_grad=True) for p, s in zip(ps, shapes)]
    for k in range(3):
        loss = fwd(tp, xs[k], labs[k])
        for q in tp:
            q.grad = None
        loss.backward()
        assert abs(got["loss"][k] - loss.item()) <= rtol * max(1.0, abs(loss.item())), (k, got["loss"][k], loss.item())
        if k == 1:
            # Gradients that pass back through a max-pool or a relu depend on which element won / which side of zero a
            # value fell.  A perturbation of relative size d flips a fraction ~d of those choices, and each flip changes
            # the gradient by a whole contribution, so two evaluations of the same net whose convolutions differ by d are
            # ~sqrt(d) apart in their early-layer gradients: torch's own f32 run is 2e-3 from its f64 run on this net, and
            # an f32 run with 1e-4 (the tolerance convolutions are held to) of noise on its convolution outputs is 4e-2
            # away.  The gradients are therefore measured against a float64 evaluation and must be within the step
            # tolerance of it, or within twice the distance of that calibration run with the allowed convolution error (both
            # distances are sums over a random handful of flips, hence the factor).
            g64, gcal = [], []
            del loss
            tp64 = [q.detach().double().requires_grad_(True) for q in tp]
            fwd(tp64, xs[k].astype(np.float64), labs[k]).backward()
            g64 = [q.grad.numpy().ravel() for q in tp64]
            del tp64
            tpc = [q.detach().clone().requires_grad_(True) for q in tp]
            fwd(tpc, xs[k], labs[k], noise=1e-4, gen=torch.Generator().manual_seed(7)).backward()
            gcal = [q.grad.numpy().astype(np.float64).ravel() for q in tpc]
            del tpc
            for n, ref, cal, gg in zip(names, g64, gcal, grads1):
                norm = np.linalg.norm(ref) + 1e-30
                e_ours = np.linalg.norm(gg.astype(np.float64) - ref) / norm
                e_cal = np.linalg.norm(cal - ref) / norm
                assert e_ours <= max(rtol, 2.0 * e_cal), f"step 1: gradient of {n}: {e_ours:.2e} from float64 (calibration run: {e_cal:.2e})"
        with torch.no_grad():
            for q in tp:
                q -= lr * q.grad
        # parameters: relative distance in the 2-norm per tensor (the flipped decisions above move single elements of a
        # gradient by whole contributions; over a tensor they average out, element by element they do not)
        for n, q, pp in zip(names, tp, got["params"][k]):
            want = q.detach().numpy().ravel().astype(np.float64)
            dist = np.linalg.norm(pp.astype(np.float64) - want) / (np.linalg.norm(want) + 1e-30)
            assert dist <= rtol, f"step {k}: parameter {n} is {dist:.2e} from the autograd run (tolerance {rtol})"
