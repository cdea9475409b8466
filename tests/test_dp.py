"""Data-parallel training: world_size-2 runs of the staged LeNet driver must
reproduce the single-process full-batch run (same losses, same parameters after
the SGD steps).  On CPU the ranks exchange gradients through gloo; on the GPU box
(2 GPUs needed) through NCCL inside libthvm_cuda.so (thvm_cuda_dp_allreduce_sum).
"""
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import hostref
from test_host_dropin import LENET_NAMES, lenet_inputs, needs_ref

ROOT = Path(__file__).resolve().parent.parent


def free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def run_world(device, world, out, B, steps, tmp_path):
    port = free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(ROOT / "tests" / "dp_worker.py"), "--device", device, "--out", str(out),
                                       "--B", str(B), "--steps", str(steps)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o[-3000:]
    return np.load(out)


def check_against_single_process(z, device, B, steps):
    x, lab, ps = lenet_inputs(B, steps)
    ref = hostref.run("drv_lenet", device, B, steps, 0.01, x, lab, np.concatenate(ps), 0)
    for s in range(steps):
        assert abs(z["losses"][s] - ref[f"loss{s}"][0]) < 2e-5, (s, z["losses"][s], ref[f"loss{s}"][0])
    for n in LENET_NAMES:
        assert np.allclose(z[n], ref[n], atol=2e-6, rtol=1e-5), n


@needs_ref
def test_two_rank_lenet_on_cpu_matches_single_process(tmp_path):
    B, steps = 8, 2
    z = run_world("cpu", 2, tmp_path / "dp_cpu.npz", B, steps, tmp_path)
    check_against_single_process(z, "cpu", B, steps)


@needs_ref
@pytest.mark.gpu
def test_two_rank_lenet_on_gpus_matches_single_process(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    B, steps = 16, 2
    z = run_world("cuda", 2, tmp_path / "dp_gpu.npz", B, steps, tmp_path)
    check_against_single_process(z, "cpu", B, steps)


# ------------------------------------------------------------------ the fused optimizer tail (thvm_cuda_dp_sgd_step)
def replay_steps(cuda, trace, steps, fused, rank=0, world=1, lr=0.01):
    """`steps` steps of a committed LeNet step program on the CUDA library; returns (losses, parameters)."""
    from tinyhvm_b200 import configs, replay, synth
    B = int(trace.split("_b")[1])
    recs = replay.load_trace(replay.TRACE_DIR / f"{trace}.thtr.gz")
    cuda.reset(0)
    rp = replay.Replayer(replay.CudaTarget(cuda), recs, fused_optimizer=fused)
    ps = configs.lenet_params()
    rp.run_prefix(dict(zip(configs.LENET_NAMES, ps)))
    seed = synth.SEED_BASE + 4
    G = B * world
    losses = []
    for s in range(steps):
        x = synth.uniform(seed, 500 + s, G * 784).reshape(G, 784)[rank * B:(rank + 1) * B].ravel().copy()
        lab = synth.labels(seed, 600 + s, G, 10)[rank * B:(rank + 1) * B]
        ext = {"x": x, "onehot": configs.onehot(lab, 10), "lr": np.array([lr / world], dtype=np.float32)}
        losses.append(float(rp.run(rp.cycles[min(s, 1)], ext)["loss"][0]))
    params = [cuda.read(k + 1, np.float32, int(np.prod(sh))) for k, sh in enumerate(configs.LENET_SHAPES)]
    cuda.reset(0)
    return losses, params


@pytest.mark.gpu
def test_fused_sgd_step_equals_the_recorded_optimizer_tail(cuda):
    """World size 1: one fused kernel instead of ten dispatches and ten copies, same bits."""
    l0, p0 = replay_steps(cuda, "lenet_b128", 3, fused=False)
    l1, p1 = replay_steps(cuda, "lenet_b128", 3, fused=True)
    assert cuda.last_plan() != "" and cuda.last_error() == ""
    assert l0 == l1
    for a, b, n in zip(p0, p1, LENET_NAMES):
        assert np.array_equal(a, b), n


@pytest.mark.gpu
def test_wait_for_a_peer_that_never_arrives_runs_out_and_reports(cuda):
    """The one-shot gradient exchange waits for every peer's flag with a bounded spin.  Here the local arena stands in for
    a second rank that never publishes a step: the wait runs out after its poll limit, the kernel returns, the status
    word says so, the parameters are untouched and the backend stays usable."""
    import ctypes as C
    lib = cuda.lib
    cuda.reset(0)
    n = 1000
    p = np.arange(n, dtype=np.float32)
    pid, gid, lrb = cuda.upload(p), cuda.upload(np.ones(n, np.float32)), cuda.upload(np.array([0.5], np.float32))
    try:
        assert lib.thvm_cuda_dp_arena_create(1 << 16, None) == 0, cuda.last_error()
        assert lib.thvm_cuda_dp_arena_attach_silent(1) == 0
        lib.thvm_cuda_dp_set_poll_limit(2000)                       # 0.2 ms
        args = ((C.c_uint32 * 1)(pid), (C.c_uint32 * 1)(gid), (C.c_uint64 * 1)(n), 1, lrb)
        assert lib.thvm_cuda_dp_sgd_step(*args) == 0, cuda.last_error()
        cuda.sync()
        assert "peer never arrived" in cuda.last_error()
        cuda.clear_error()
        assert np.array_equal(cuda.read(pid, np.float32, n), p)     # not updated
    finally:
        lib.thvm_cuda_dp_set_poll_limit(0)
        lib.thvm_cuda_dp_shutdown()                                 # back to world size 1, arena released
    assert lib.thvm_cuda_dp_sgd_step(*args) == 0                    # world 1: plain update, no exchange
    assert np.array_equal(cuda.read(pid, np.float32, n), p - np.float32(0.5))
    cuda.reset(0)
    assert cuda.last_error() == ""


@pytest.mark.gpu
def test_two_ranks_with_the_fused_exchange_match_one_process_on_the_whole_batch(tmp_path, cuda):
    """2 GPUs, one process each: the committed 128-sample step program per rank, gradients exchanged through the peer-mapped
    arenas and summed by the fused kernel, against one process running the 256-sample program on the concatenated batch."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    steps = 3
    want_l, want_p = replay_steps(cuda, "lenet_b256", steps, fused=True)
    cuda.lib.thvm_cuda_shutdown()                                   # the workers take the GPUs
    port = free_port()
    out = tmp_path / "fused2.npz"
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(ROOT / "tests" / "dp_replay_worker.py"), "--out", str(out), "--steps", str(steps)],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o[-3000:]
    z = np.load(out)
    for s in range(steps):
        assert abs(z["losses"][s] - want_l[s]) < 2e-5, (s, z["losses"][s], want_l[s])
    for k, n in enumerate(LENET_NAMES):
        assert np.array_equal(z[f"r0_{n}"], z[f"r1_{n}"]), f"{n}: the two ranks hold different parameters"
        assert np.allclose(z[f"r0_{n}"], want_p[k], atol=2e-6, rtol=1e-5), n
