"""Trace record / replay.

The reference's host runtime runs the staged LeNet driver on a recording backend
(oracle/ref_trace.c); the trace is then replayed call by call
  * through the reference's own CPU backend at the vtable boundary (CPU test):
    losses and parameters must equal the recorded run bit for bit, which shows the
    trace and the replayer are faithful;
  * through libthvm_cuda.so (GPU test): same numbers within the training tolerance.
Also checked: the steady-state step cycle is identical from step to step (that is
what makes replaying one recorded cycle for every later step legitimate), and the
committed full-size trace used by the benchmark parses and has the expected shape.
"""
import ctypes as C

import numpy as np
import pytest

import hostref
from test_host_dropin import LENET_NAMES, LENET_SHAPES, lenet_inputs, needs_ref
from tinyhvm_b200 import replay
from tinyhvm_b200.configs import onehot

_u32, _u64, _vp = C.c_uint32, C.c_uint64, C.c_void_p


class RefTarget:
    """The reference's CPU backend behind its vtable (oracle/_ref/libthvm_cpu_ref.so)."""

    def __init__(self, ref):
        self.lib = ref.lib
        self.lib.ref_pool_reset(_u32(0))

    def alloc(self, nbytes): return self.lib.ref_buf_alloc(nbytes)
    def write(self, i, ptr, nbytes): self.lib.ref_buf_write(i, ptr, nbytes)
    def read(self, i, ptr, nbytes): self.lib.ref_buf_read(i, ptr, nbytes)
    def free(self, i): pass
    def incref(self, i): pass
    def decref(self, i): pass
    def set_persistent(self, m): pass
    def allreduce(self, ids, counts): pass
    def pool_reset(self, keep): self.lib.ref_pool_reset(_u32(keep))

    def copy(self, d, s, nbytes):
        tmp = np.empty(nbytes, dtype=np.uint8)
        self.lib.ref_buf_read(s, tmp.ctypes.data, nbytes)
        self.lib.ref_buf_write(d, tmp.ctypes.data, nbytes)

    def sgd_step(self, params, grads, counts, lr_buf):
        """What thvm_cuda_dp_sgd_step computes at world size 1, on the reference backend's buffers: p <- p - g * lr
        (one rounding per operation, like the dispatch it replaces)."""
        lr = np.empty(1, dtype=np.float32)
        self.lib.ref_buf_read(lr_buf, lr.ctypes.data, 4)
        for pid, gid, n in zip(params, grads, counts):
            pv, gv = np.empty(n, dtype=np.float32), np.empty(n, dtype=np.float32)
            self.lib.ref_buf_read(pid, pv.ctypes.data, 4 * n)
            self.lib.ref_buf_read(gid, gv.ctypes.data, 4 * n)
            pv = (pv - (gv * lr[0]).astype(np.float32)).astype(np.float32)
            self.lib.ref_buf_write(pid, pv.ctypes.data, 4 * n)

    def dispatch(self, a):
        self.lib.ref_dispatch_kernel_rs(_u32(a.out), a.ids, a.view_ptrs, a.st_ptrs, _u32(a.n), a.ops, _u32(a.n_ops), C.byref(a.full),
                                        C.byref(a.red) if a.has_red else None, a.dts, _u32(a.out_dt))


def record(tmp_path, B, steps, dry=0):
    x, lab, ps = lenet_inputs(B, steps)
    path = tmp_path / f"lenet_b{B}.thtr"
    res = hostref.run("drv_record_lenet", str(path), dry, B, steps, 0.01, x, lab, np.concatenate(ps))
    return path, res, (x, lab, ps)


def replay_lenet(target, recs, B, steps, data, lr=0.01, fused=False):
    x, lab, ps = data
    rp = replay.Replayer(target, recs, fused_optimizer=fused)
    rp.run_prefix(dict(zip(LENET_NAMES, ps)))
    losses = []
    for s in range(steps):
        ext = {"x": x[s * B * 784:(s + 1) * B * 784], "onehot": onehot(lab[s * B:(s + 1) * B], 10),
               "lr": np.array([lr], dtype=np.float32)}
        cyc = rp.cycles[min(s, 1)]                        # cycle 0 = first step, cycle 1 = every later step
        out = rp.run(cyc, ext)
        losses.append(float(out["loss"][0]))
    params = {}
    for k, (name, shape) in enumerate(zip(LENET_NAMES, LENET_SHAPES)):
        buf = np.empty(int(np.prod(shape)), dtype=np.float32)
        target.read(k + 1, buf.ctypes.data, buf.nbytes)   # parameters are the first ten buffers of the prefix
        params[name] = buf
    return losses, params


@needs_ref
def test_replay_through_reference_cpu_backend_is_bit_exact(tmp_path, ref):
    B, steps = 8, 4
    path, res, data = record(tmp_path, B, steps)
    recs = replay.load_trace(path)
    prefix, cycles = replay.split_steps(recs)
    assert len(cycles) == steps
    key = lambda c: [(r.op, r.f, r.blob) for r in c if r.op != replay.MARK]
    assert key(cycles[1]) == key(cycles[2]), "the steady-state step cycle changes from step to step"
    losses, params = replay_lenet(RefTarget(ref), recs, B, steps, data)
    for s in range(steps):
        assert losses[s] == float(res[f"loss{s}"][0]), s
    for n in LENET_NAMES:
        assert np.array_equal(params[n], res[n]), n
    ref.lib.ref_pool_reset(_u32(0))


@needs_ref
def test_fused_optimizer_rewrite_is_equivalent_on_the_reference_backend(tmp_path, ref):
    """The replayer's rewrite of a step's optimizer tail (all-reduce + per-tensor `p - g*lr` dispatch + copy -> one fused
    record) changes nothing: replayed through the reference's CPU backend, losses and parameters are bit-identical."""
    B, steps = 8, 3
    path, res, data = record(tmp_path, B, steps)
    recs = replay.load_trace(path)
    _, cycles = replay.split_steps(recs)
    fused = replay.fuse_optimizer(cycles[1])
    assert sum(r.op == replay.SGD_FUSED for r in fused) == 1
    assert sum(r.op == replay.DISPATCH for r in cycles[1]) - sum(r.op == replay.DISPATCH for r in fused) == len(LENET_NAMES)
    assert not any(r.op == replay.ALLREDUCE for r in fused)
    losses, params = replay_lenet(RefTarget(ref), recs, B, steps, data, fused=True)
    for s in range(steps):
        assert losses[s] == float(res[f"loss{s}"][0]), s
    for n in LENET_NAMES:
        assert np.array_equal(params[n], res[n]), n
    ref.lib.ref_pool_reset(_u32(0))


def test_committed_traces_have_a_fusable_optimizer_tail():
    for name, n_params in (("lenet_b128", 10), ("lenet_b1024", 10), ("vgg_b64", 20), ("vgg_b512", 20)):
        recs = replay.load_trace(replay.TRACE_DIR / f"{name}.thtr.gz")
        _, cycles = replay.split_steps(recs)
        for cyc in cycles[:2]:
            fused = [r for r in replay.fuse_optimizer(cyc) if r.op == replay.SGD_FUSED]
            assert len(fused) == 1 and len(fused[0].f[0]) == n_params, name
            assert fused[0].f[0] == tuple(range(1, n_params + 1)), name        # the parameters are the first buffers of the prefix


def test_committed_lenet_trace_parses():
    path = replay.TRACE_DIR / "lenet_b1024.thtr.gz"
    recs = replay.load_trace(path)
    prefix, cycles = replay.split_steps(recs)
    assert len(cycles) >= 2
    n_disp = sum(1 for r in cycles[1] if r.op == replay.DISPATCH)
    assert 50 <= n_disp <= 80
    ext = {r.f[3] for r in cycles[1] if r.op == replay.WRITE and r.f[1]}
    assert ext == {"x", "onehot", "lr"}, ext
    x_bytes = [r.f[2] for r in cycles[1] if r.op == replay.WRITE and r.f[3] == "x"]
    assert x_bytes == [1024 * 784 * 4]


@needs_ref
@pytest.mark.gpu
def test_replay_on_gpu_matches_recorded_run(tmp_path, cuda):
    B, steps = 8, 3
    path, res, data = record(tmp_path, B, steps)
    recs = replay.load_trace(path)
    cuda.reset(0)
    losses, params = replay_lenet(replay.CudaTarget(cuda), recs, B, steps, data)
    for s in range(steps):
        assert abs(losses[s] - float(res[f"loss{s}"][0])) < 2e-5, s
    for n in LENET_NAMES:
        assert np.allclose(params[n], res[n], rtol=1e-4, atol=1e-6), n
    cuda.reset(0)
    assert cuda.last_error() == ""


# ------------------------------------------------------------------ the VGG-style step (conv3x3 + batchnorm + relu blocks)
VGG_SMALL = dict(B=8, H=8, classes=10, chan=(3, 4, 4, 8, 8, 8, 8))


def record_vgg(tmp_path, steps, dry=0):
    from tinyhvm_b200.configs import vgg_inputs
    c = VGG_SMALL
    x, lab, ps = vgg_inputs(c["B"], steps, c["H"], c["classes"], c["chan"])
    path = tmp_path / "vgg_small.thtr"
    res = hostref.run("drv_record_vgg", str(path), dry, c["B"], c["H"], c["classes"], np.array(c["chan"], np.uint32), steps, 0.05,
                      x, lab, np.concatenate(ps))
    return path, res, (x, lab, ps)


def replay_vgg(target, recs, steps, data, lr=0.05):
    from tinyhvm_b200.configs import vgg_shapes
    c = VGG_SMALL
    x, lab, ps = data
    shapes, names = vgg_shapes(c["chan"], c["H"], c["classes"])
    rp = replay.Replayer(target, recs)
    rp.run_prefix(dict(zip(names, ps)))
    losses, n = [], c["B"] * 3 * c["H"] * c["H"]
    for s in range(steps):
        ext = {"x": x[s * n:(s + 1) * n], "onehot": onehot(lab[s * c["B"]:(s + 1) * c["B"]], c["classes"]),
               "lr": np.array([lr], dtype=np.float32)}
        losses.append(float(rp.run(rp.cycles[min(s, 1)], ext)["loss"][0]))
    params = {}
    for k, (name, shape) in enumerate(zip(names, shapes)):
        buf = np.empty(int(np.prod(shape)), dtype=np.float32)
        target.read(k + 1, buf.ctypes.data, buf.nbytes)
        params[name] = buf
    return losses, params


@needs_ref
def test_vgg_replay_through_reference_cpu_backend_is_bit_exact(tmp_path, ref):
    steps = 4
    path, res, data = record_vgg(tmp_path, steps)
    recs = replay.load_trace(path)
    prefix, cycles = replay.split_steps(recs)
    key = lambda c: [(r.op, r.f, r.blob) for r in c if r.op != replay.MARK]
    assert key(cycles[1]) == key(cycles[2]), "the steady-state step cycle changes from step to step"
    losses, params = replay_vgg(RefTarget(ref), recs, steps, data)
    for s in range(steps):
        assert losses[s] == float(res[f"loss{s}"][0]), s
    for n in params:
        assert np.array_equal(params[n], res[n]), n
    ref.lib.ref_pool_reset(_u32(0))


def test_committed_vgg_trace_parses():
    recs = replay.load_trace(replay.TRACE_DIR / "vgg_b512.thtr.gz")
    prefix, cycles = replay.split_steps(recs)
    assert len(cycles) >= 2
    assert 120 <= sum(1 for r in cycles[1] if r.op == replay.DISPATCH) <= 200
    ext = {(r.f[3], r.f[2]) for r in cycles[1] if r.op == replay.WRITE and r.f[1]}
    assert ext == {("x", 512 * 3 * 64 * 64 * 4), ("onehot", 512 * 100 * 4), ("lr", 4)}, ext


@needs_ref
@pytest.mark.gpu
def test_vgg_replay_on_gpu_matches_recorded_run(tmp_path, cuda):
    steps = 3
    path, res, data = record_vgg(tmp_path, steps)
    recs = replay.load_trace(path)
    cuda.reset(0)
    losses, params = replay_vgg(replay.CudaTarget(cuda), recs, steps, data)
    for s in range(steps):
        assert abs(losses[s] - float(res[f"loss{s}"][0])) < 1e-4, s
    for n in params:
        assert np.allclose(params[n], res[n], rtol=2e-3, atol=2e-5), n
    cuda.reset(0)
    assert cuda.last_error() == ""


@needs_ref
@pytest.mark.gpu
def test_captured_step_graph_matches_recorded_run(tmp_path, cuda):
    """Steps 0 and 1 run eagerly; the steady-state cycle is then recorded as a CUDA graph and launched for
    steps 2..5 with fresh inputs each time: losses and final parameters as in the recorded CPU run."""
    B, steps = 8, 6
    path, res, (x, lab, ps) = record(tmp_path, B, steps)
    recs = replay.load_trace(path)
    cuda.reset(0)
    rp = replay.Replayer(replay.CudaTarget(cuda), recs)
    rp.run_prefix(dict(zip(LENET_NAMES, ps)))
    lr = np.array([0.01], dtype=np.float32)
    ext = lambda s: {"x": x[s * B * 784:(s + 1) * B * 784].copy(), "onehot": onehot(lab[s * B:(s + 1) * B], 10), "lr": lr}
    losses = [float(rp.run(rp.cycles[min(s, 1)], ext(s))["loss"][0]) for s in range(2)]
    launches_eager = cuda.launches()
    step = rp.capture(rp.cycles[1], ext(2))
    assert cuda.launches() - launches_eager == step.n_kernels > 0
    # the step's memory plan: every buffer the step allocates sits at a fixed offset of one arena made when the capture
    # began (sized from the eager step before it), so the recorded graph holds no allocation or free nodes
    ab, au, bt = C.c_uint64(), C.c_uint64(), C.c_uint64()
    na, npool = C.c_uint32(), C.c_uint32()
    assert cuda.lib.thvm_cuda_graph_memory(step.handle, C.byref(ab), C.byref(au), C.byref(na), C.byref(npool), C.byref(bt)) == 0
    assert na.value > 20 and npool.value == 0, (na.value, npool.value)
    assert 0 < au.value <= ab.value and au.value <= bt.value + 1024 * na.value, (au.value, ab.value, bt.value)
    nk, ncp, nms, no = (C.c_uint32() for _ in range(4))
    assert cuda.lib.thvm_cuda_graph_nodes(step.handle, C.byref(nk), C.byref(ncp), C.byref(nms), C.byref(no)) == 0
    assert nk.value == step.n_kernels and ncp.value >= 3 and no.value == 0, (nk.value, ncp.value, nms.value, no.value)
    # steps 2 and 3: inputs uploaded on the main stream before the launch; steps 4 and 5: uploaded ahead on the copy
    # stream while the step before them is still running, into another staging slot
    keep = [ext(s) for s in range(steps)]                 # the host arrays stay alive until their step has run
    for s in (2, 3):
        step.launch(keep[s])
        if s == 3:
            step.prefetch(keep[4])
        losses.append(float(step.results()["loss"][0]))
    for s in (4, 5):
        step.launch_prefetched()
        if s == 4:
            step.prefetch(keep[5])
        losses.append(float(step.results()["loss"][0]))
    for s in range(steps):
        assert abs(losses[s] - float(res[f"loss{s}"][0])) < 2e-5, s
    for k, (name, shape) in enumerate(zip(LENET_NAMES, LENET_SHAPES)):
        got = cuda.read(k + 1, np.float32, int(np.prod(shape)))
        assert np.allclose(got, res[name], rtol=1e-4, atol=1e-6), name
    step.destroy()
    cuda.reset(0)
    assert cuda.last_error() == ""


@pytest.mark.gpu
def test_capture_refuses_a_step_that_leaks_a_buffer(cuda):
    cuda.reset(0)
    assert cuda.lib.thvm_cuda_capture_begin() == 0
    leaked = cuda.alloc(4096)                       # allocated inside the capture and never freed
    assert cuda.lib.thvm_cuda_capture_end() == 0
    assert "still live" in cuda.last_error()
    cuda.lib.thvm_cuda_clear_error()
    cuda.reset(0)
    a = cuda.upload(np.arange(1024, dtype=np.float32))
    assert np.array_equal(cuda.read(a, np.float32, 1024), np.arange(1024, dtype=np.float32))    # the backend is still usable
    cuda.reset(0)


@pytest.mark.gpu
def test_capture_refuses_a_dispatch_it_has_not_seen_and_caches_no_plan(cuda):
    """A dispatch whose plan does not exist yet cannot be built while the stream records (its tables would live in
    memory the recorded graph owns).  The capture is refused before anything is allocated, the plan cache is left as
    it was, and the same dispatch then runs eagerly with the right result."""
    import cases
    from tinyhvm_b200 import abi
    cuda.reset(0)
    rng = np.random.default_rng(11)
    # shapes no other test uses, so the plans cannot exist yet: a tracker leaf (device tables), a contraction
    # (offset tables) and a non-f32 output (descriptor-driven kernel)
    fresh = [cases.tracker_case(987654), cases.mm_case(rng, 77, 131, 59)]
    for d in fresh:
        ids = [cuda.upload(l.data) for l in d.leaves]
        out = cuda.alloc(d.out_numel * 4)
        cuda.sync()
        plans = cuda.lib.thvm_cuda_plan_count()
        assert cuda.lib.thvm_cuda_capture_begin() == 0
        cuda.dispatch_ids(out, ids, d)
        assert cuda.lib.thvm_cuda_capture_end() == 0
        assert "inside the captured step" in cuda.last_error()
        cuda.clear_error()
        assert cuda.lib.thvm_cuda_plan_count() == plans, "a plan built inside the refused capture stayed in the cache"
        cuda.dispatch_ids(out, ids, d)                      # eager: builds the plan now
        got = cuda.read(out, np.float32, d.out_numel)
        want = cases_oracle().run(d)
        assert np.allclose(got, want, rtol=1e-4, atol=1e-5), d.name
        assert cuda.lib.thvm_cuda_plan_count() == plans + 1
        cuda.reset(0)
    assert cuda.last_error() == ""


def cases_oracle():
    import checkers
    return checkers.Oracle()


@pytest.mark.gpu
def test_refused_capture_leaves_older_buffers_as_they_were(cuda):
    """Buffers that existed before a refused capture keep their contents: a small host-written constant that the
    captured step was the first to touch on the device still feeds later kernels correctly, a fresh buffer still reads
    as zero, and a host write made inside the refused step is gone."""
    from tinyhvm_b200 import abi
    from tinyhvm_b200.abi import ADD, Dispatch, Leaf
    cuda.reset(0)
    n = 4096
    x = np.arange(n, dtype=np.float32)
    d = Dispatch([Leaf(x, abi.view_contiguous([n])), Leaf(np.array([2.5], np.float32), abi.view_contiguous([1]))], [(ADD, 0, 1)], [n])
    bx, bs = cuda.upload(x), cuda.upload(np.array([2.5], np.float32))   # bs: host shadow only so far
    fresh = cuda.alloc(n * 4)                                            # owes its zero-fill
    out = cuda.alloc(n * 4)
    cuda.dispatch_ids(out, [bx, cuda.upload(np.array([1.0], np.float32))], d)   # plan exists now; its scalar buffer is a third one
    cuda.sync()
    assert cuda.lib.thvm_cuda_capture_begin() == 0
    cuda.dispatch_ids(out, [bx, bs], d)                                  # first device use of bs happens inside the capture
    cuda.dispatch_ids(fresh, [bx, bs], d)                                # would overwrite the fresh buffer
    cuda.write(bs, np.array([7.0], np.float32))                          # host write inside the step
    leaked = cuda.alloc(1 << 16)                                         # makes the capture fail
    assert cuda.lib.thvm_cuda_capture_end() == 0
    cuda.clear_error()
    assert cuda.read(bs, np.float32, 1)[0] == 2.5
    assert not cuda.read(fresh, np.float32, n).any()
    out2 = cuda.alloc(n * 4)
    cuda.dispatch_ids(out2, [bx, bs], d)
    assert np.array_equal(cuda.read(out2, np.float32, n), x + np.float32(2.5))
    cuda.reset(0)
    assert cuda.last_error() == ""


@pytest.mark.gpu
def test_step_constants_are_uploaded_once_and_survive_a_step_that_overwrites_them(cuda):
    """What the host writes inside a recorded step is a constant of the step: it gets no copy node (it is placed in the
    never-recycled part of the step arena and uploaded while the step is recorded).  A step that overwrites such a
    constant with a kernel still sees the original bytes at every replay, because a put-back copy ends the graph."""
    from tinyhvm_b200 import abi
    from tinyhvm_b200.abi import ADD, Dispatch, Leaf
    cuda.reset(0)
    n = 4096
    v = abi.view_contiguous([n])
    table = np.linspace(-1, 1, n).astype(np.float32)
    add_scalar = Dispatch([Leaf(table, v), Leaf(np.array([2.5], np.float32), abi.view_contiguous([1]))], [(ADD, 0, 1)], [n])
    add_table = Dispatch([Leaf(table, v), Leaf(table, v)], [(ADD, 0, 1)], [n])
    add_s = Dispatch([Leaf(np.zeros(1, np.float32), abi.view_contiguous([1])), Leaf(np.zeros(1, np.float32), abi.view_contiguous([1]))], [(ADD, 0, 1)], [1])
    bx, out = cuda.alloc(n * 4), cuda.alloc(n * 4)              # older than the step: the input and the result
    keep = out

    def step(overwrite: bool):
        cs = cuda.upload(np.array([2.5], np.float32))           # 4 bytes: host shadow until a kernel needs it
        cl = cuda.upload(table)                                 # 16 KB: device memory at once, then the host write
        t = cuda.alloc(n * 4)
        cuda.dispatch_ids(t, [bx, cs], add_scalar)              # t = x + 2.5
        cuda.dispatch_ids(out, [t, cl], add_table)              # out = t + table
        if overwrite:
            cuda.dispatch_ids(cl, [cl, cs], add_scalar)         # the step clobbers both constants afterwards
            cuda.dispatch_ids(cs, [cs, cs], add_s)
        res = cuda.read(out, np.float32, n)
        cuda.reset(keep)
        return res

    for overwrite in (False, True):
        x0 = np.arange(n, dtype=np.float32)
        cuda.write(bx, x0)
        assert np.array_equal(step(overwrite), x0 + np.float32(2.5) + table)      # eager: plans built
        cuda.sync()
        cuda.reset(keep)
        step(overwrite)                                                          # a finished step sizes the arena
        assert cuda.lib.thvm_cuda_capture_begin() == 0
        xin = np.ascontiguousarray(x0)
        assert cuda.lib.thvm_cuda_capture_input(bx, xin.ctypes.data, xin.nbytes) == 0
        step(overwrite)
        gr = cuda.lib.thvm_cuda_capture_end()
        assert gr > 0, cuda.last_error()
        nk, ncp, nms, no = (C.c_uint32() for _ in range(4))
        assert cuda.lib.thvm_cuda_graph_nodes(gr, C.byref(nk), C.byref(ncp), C.byref(nms), C.byref(no)) == 0
        # copies: the input's second hop and the result read-back; plus one put-back per clobbered constant
        assert ncp.value == (4 if overwrite else 2), (overwrite, nk.value, ncp.value, nms.value, no.value)
        for k in range(3):
            xk = (x0 * (k + 1)).astype(np.float32)
            assert cuda.lib.thvm_cuda_graph_set_input(gr, 0, xk.ctypes.data) == 0
            assert cuda.lib.thvm_cuda_graph_launch(gr) == 0
            got = np.empty(n, np.float32)
            assert cuda.lib.thvm_cuda_graph_result(gr, 0, got.ctypes.data, got.nbytes) == 0
            assert np.array_equal(got, xk + np.float32(2.5) + table), (overwrite, k)
        cuda.lib.thvm_cuda_graph_destroy(gr)
    cuda.reset(0)
    assert cuda.last_error() == ""
