"""End-to-end drop-in tests: the reference's own host runtime (reducer, fuser,
scheduler, nn library; compiled from its sources into oracle/_ref/) runs the
same staged driver program once with thvm_init("cpu") and once with
thvm_init("cuda"), where the scheduler reaches libthvm_cuda.so through the
vtable hub (tinyhvm_b200/backend_cuda/_.c).  Every realised tensor is compared.

CPU-only part: the drivers themselves are checked against closed forms (numpy /
torch autograd), so the same-program comparison on the GPU box rests on a
verified program.  Skipped where oracle/_ref/ was not built.
"""
import numpy as np
import pytest

import hostref
from tinyhvm_b200 import synth
from tinyhvm_b200.configs import (LENET_NAMES, LENET_SHAPES, VGG_CHAN, lenet_inputs, vgg_inputs,  # noqa: F401
                                   vgg_shapes)

needs_ref = pytest.mark.skipif(not hostref.available(), reason="oracle/_ref/libthvm_host_ref.so not built")

def mlp_inputs(B=64, I=784, H=128, O=10, seed=synth.SEED_BASE + 1):
    x = synth.uniform(seed, 0, B * I)
    W1, b1 = synth.kaiming_uniform(seed, 1, I * H, I), synth.kaiming_uniform(seed, 2, H, I)
    W2, b2 = synth.kaiming_uniform(seed, 3, H * O, H), synth.kaiming_uniform(seed, 4, O, H)
    lab = synth.labels(seed, 5, B, O)
    return (B, I, H, O, x, W1, b1, W2, b2, lab)


def close(a, b, rtol):
    """|a-b| <= rtol * (|b| + rms(b)) elementwise"""
    a, b = a.astype(np.float64), b.astype(np.float64)
    if a.shape != b.shape:
        return False
    rms = np.sqrt(np.mean(b ** 2)) if b.size else 0.0
    return bool(np.all(np.abs(a - b) <= rtol * (np.abs(b) + rms) + 1e-30))


# ------------------------------------------------------------------ CPU: the programs are right
@needs_ref
def test_chain_and_gemm_drivers_match_numpy():
    rng = np.random.default_rng(0)
    R, C = 16, 32
    a, b, c = (rng.standard_normal(R * C).astype(np.float32) for _ in range(3))
    r = hostref.run("drv_chain", "cpu", R, C, a, b, c)
    u = a * b + c
    assert np.allclose(r["y"], np.maximum(u, 0).reshape(R, C).astype(np.float64).sum(1), rtol=1e-5)
    assert np.array_equal(r["g"], np.where(u > 0, b, np.float32(0)))
    n = 24
    A, B = (rng.standard_normal(n * n).astype(np.float32) / 5 for _ in range(2))
    r = hostref.run("drv_gemm", "cpu", n, A, B)
    Cm = A.reshape(n, n).astype(np.float64) @ B.reshape(n, n)
    assert np.allclose(r["C"], Cm.ravel(), atol=1e-5)
    assert np.allclose(r["dA"], (2 * Cm @ B.reshape(n, n).T).ravel(), atol=1e-5)
    assert np.allclose(r["dB"], (A.reshape(n, n).T @ (2 * Cm)).ravel(), atol=1e-5)
    assert np.allclose(r["L"], (Cm * Cm).sum(), rtol=1e-5)


@needs_ref
def test_mlp_driver_matches_torch_autograd():
    import torch
    B, I, H, O, x, W1, b1, W2, b2, lab = mlp_inputs(B=8, I=20, H=16)
    r = hostref.run("drv_mlp", "cpu", B, I, H, O, x, W1, b1, W2, b2, lab)
    t = lambda a, *s: torch.tensor(a.reshape(*s), requires_grad=True)
    tW1, tb1, tW2, tb2 = t(W1, I, H), t(b1, H), t(W2, H, O), t(b2, O)
    loss = torch.nn.functional.cross_entropy(torch.relu(torch.tensor(x.reshape(B, I)) @ tW1 + tb1) @ tW2 + tb2,
                                             torch.tensor(lab.astype(np.int64)))
    loss.backward()
    assert abs(r["loss"][0] - loss.item()) < 1e-5
    for k, q in (("dW1", tW1), ("db1", tb1), ("dW2", tW2), ("db2", tb2)):
        assert np.allclose(r[k], q.grad.numpy().ravel(), atol=1e-6), k


@needs_ref
def test_lenet_driver_matches_torch_autograd():
    import torch
    F = torch.nn.functional
    B, steps, lr = 4, 2, 0.01
    x, lab, ps = lenet_inputs(B, steps)
    r = hostref.run("drv_lenet", "cpu", B, steps, lr, x, lab, np.concatenate(ps), 1)
    tp = [torch.tensor(p.reshape(s), requires_grad=True) for p, s in zip(ps, LENET_SHAPES)]
    for s in range(steps):
        tx = torch.tensor(x[s * B * 784:(s + 1) * B * 784].reshape(B, 1, 28, 28))
        h = F.max_pool2d(torch.relu(F.conv2d(tx, tp[0], tp[1], padding=2)), 2)
        h = F.max_pool2d(torch.relu(F.conv2d(h, tp[2], tp[3])), 2).reshape(B, 400)
        h = torch.relu(torch.relu(h @ tp[4] + tp[5]) @ tp[6] + tp[7])
        loss = F.cross_entropy(h @ tp[8] + tp[9], torch.tensor(lab[s * B:(s + 1) * B].astype(np.int64)))
        for q in tp:
            q.grad = None
        loss.backward()
        assert abs(r[f"loss{s}"][0] - loss.item()) < 2e-5
        if s == 0:
            for n, q in zip(LENET_NAMES, tp):
                assert np.allclose(r["d" + n], q.grad.numpy().ravel(), atol=2e-6), n
        with torch.no_grad():
            for q in tp:
                q -= lr * q.grad
    for n, q in zip(LENET_NAMES, tp):
        assert np.allclose(r[n], q.detach().numpy().ravel(), atol=1e-6), n


@needs_ref
def test_vgg_driver_matches_torch_autograd():
    import torch
    F = torch.nn.functional
    B, steps, lr, H, classes, chan = 4, 2, 0.05, 8, 10, (3, 4, 4, 8, 8, 8, 8)
    x, lab, ps = vgg_inputs(B, steps, H, classes, chan)
    shapes, names = vgg_shapes(chan, H, classes)
    r = hostref.run("drv_vgg", "cpu", B, H, classes, np.array(chan, np.uint32), steps, lr, x, lab, np.concatenate(ps), 1)
    tp = [torch.tensor(p.reshape(s), requires_grad=True) for p, s in zip(ps, shapes)]
    for s in range(steps):
        a = torch.tensor(x[s * B * 3 * H * H:(s + 1) * B * 3 * H * H].reshape(B, 3, H, H))
        for l in range(6):
            a = torch.relu(F.batch_norm(F.conv2d(a, tp[3 * l], padding=1), None, None, tp[3 * l + 1], tp[3 * l + 2], training=True, eps=1e-5))
            if l & 1:
                a = F.max_pool2d(a, 2)
        loss = F.cross_entropy(a.reshape(B, -1) @ tp[18] + tp[19], torch.tensor(lab[s * B:(s + 1) * B].astype(np.int64)))
        for q in tp:
            q.grad = None
        loss.backward()
        assert abs(r[f"loss{s}"][0] - loss.item()) < 2e-5
        if s == 0:
            for n, q in zip(names, tp):
                assert np.allclose(r["d" + n], q.grad.numpy().ravel(), atol=1e-5), n
        with torch.no_grad():
            for q in tp:
                q -= lr * q.grad
    for n, q in zip(names, tp):
        assert np.allclose(r[n], q.detach().numpy().ravel(), atol=2e-6), n


# ------------------------------------------------------------------ GPU: cuda == cpu through the reference's scheduler
def compare_runs(driver, args, rtol, exact=()):
    cpu = hostref.run(driver, "cpu", *args)
    gpu = hostref.run(driver, "cuda", *args)
    assert set(cpu) == set(gpu)
    for k in cpu:
        if k.startswith("_"):
            continue
        assert cpu[k].size > 0, f"{k}: the CPU run kept nothing"
        if k in exact:
            assert np.array_equal(cpu[k], gpu[k]), f"{k}: not bit-exact"
        else:
            assert close(gpu[k], cpu[k], rtol), f"{k}: cuda differs from cpu beyond {rtol}"
    return cpu, gpu


@needs_ref
@pytest.mark.gpu
def test_chain_config_cuda_vs_cpu():
    R, C = 64, 1024
    a, b, c = (synth.normal(synth.SEED_BASE + 2, t, R * C) for t in range(3))
    compare_runs("drv_chain", (R, C, a, b, c), 1e-5, exact=("g",))


@needs_ref
@pytest.mark.gpu
def test_gemm_config_cuda_vs_cpu():
    n = 96
    A, B = (synth.normal(synth.SEED_BASE + 3, t, n * n) / np.float32(np.sqrt(n)) for t in range(2))
    compare_runs("drv_gemm", (n, A, B), 1e-4)


@needs_ref
@pytest.mark.gpu
def test_mlp_config_cuda_vs_cpu():
    compare_runs("drv_mlp", mlp_inputs(), 1e-4)          # the full config-1 sizes: [64,784] x [784,128] x [128,10]


@needs_ref
@pytest.mark.gpu
def test_lenet_training_steps_cuda_vs_cpu():
    B, steps = 8, 2
    x, lab, ps = lenet_inputs(B, steps)
    compare_runs("drv_lenet", (B, steps, 0.01, x, lab, np.concatenate(ps), 1), 1e-4)


@needs_ref
@pytest.mark.gpu
def test_vgg_training_steps_cuda_vs_cpu():
    B, steps, H, classes, chan = 8, 2, 16, 10, (3, 8, 8, 16, 16, 16, 16)
    x, lab, ps = vgg_inputs(B, steps, H, classes, chan)
    compare_runs("drv_vgg", (B, H, classes, np.array(chan, np.uint32), steps, 0.05, x, lab, np.concatenate(ps), 1), 2e-3)


@needs_ref
@pytest.mark.gpu
def test_lowered_kop_programs_cuda_vs_cpu(monkeypatch):
    """With THVM_CUDA_UOP set the hub fills the dispatch_uop_kernel slot, so the reference's scheduler hands
    over the lowered KOP programs of its own lowerer (src/lower/_.c:765-973, src/schedule/_.c:2370) and the
    device-side KOP interpreter runs them: same tensors as the CPU run of the same programs."""
    import tinyhvm_b200
    monkeypatch.setenv("THVM_CUDA_UOP", "1")
    R, C = 64, 1024
    a, b, c = (synth.normal(synth.SEED_BASE + 2, t, R * C) for t in range(3))
    compare_runs("drv_chain", (R, C, a, b, c), 1e-5, exact=("g",))
    last = tinyhvm_b200.load().thvm_cuda_last_plan()
    assert last == b"uop_program", f"the KOP interpreter did not run (last kernel family: {last})"
    n = 48
    A, B = (synth.normal(synth.SEED_BASE + 3, t, n * n) / np.float32(np.sqrt(n)) for t in range(2))
    compare_runs("drv_gemm", (n, A, B), 1e-4)
    compare_runs("drv_mlp", mlp_inputs(B=16, I=64, H=32), 1e-4)


@needs_ref
@pytest.mark.gpu
def test_lenet_step_captured_by_the_live_host_and_replayed():
    """The reference's own capture / replay entry points (jit_begin_capture / jit_end_capture / jit_replay,
    src/tinyhvm.h:1294-1300), bound by the CUDA hub: the live reference host issues step 2 between begin and end, and
    steps 2..5 are replays of the recorded step on fresh batches.  Losses and final parameters as in the eager run."""
    B, steps = 8, 6
    x, lab, ps = lenet_inputs(B, steps)
    eager = hostref.run("drv_lenet", "cuda", B, steps, 0.01, x, lab, np.concatenate(ps), 0)
    cap = hostref.run("drv_lenet_captured", "cuda", B, steps, 0.01, x, lab, np.concatenate(ps), 2)
    for s in range(steps):
        assert abs(cap[f"loss{s}"][0] - eager[f"loss{s}"][0]) < 2e-5, (s, cap[f"loss{s}"][0], eager[f"loss{s}"][0])
    for n in LENET_NAMES:
        assert np.allclose(cap[n], eager[n], rtol=1e-5, atol=1e-6), n
