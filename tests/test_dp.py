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
