"""One rank of a 2-GPU run of the committed LeNet step program (launched by tests/test_dp.py): replay of the 128-sample
program on this rank's half of each batch, optimizer tail through thvm_cuda_dp_sgd_step with the gradients exchanged
over the peer-mapped arenas.  The NCCL token and the arena handles travel over a gloo group.  Rank 0 stores the
mean losses and both ranks' final parameters in --out."""
import argparse
import ctypes as C
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path[:0] = [str(ROOT), str(ROOT / "tests")]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--steps", type=int, default=3)
    args = ap.parse_args()
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    os.environ["THVM_CUDA_DEVICE"] = os.environ.get("LOCAL_RANK", str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import tinyhvm_b200
    from tinyhvm_b200.configs import LENET_NAMES
    from test_dp import replay_steps
    be = tinyhvm_b200.CudaBackend()
    lib = be.lib
    token = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        raw = (C.c_uint8 * 128)()
        assert lib.thvm_cuda_dp_unique_id(raw) == 0, be.last_error()
        token = torch.tensor(list(raw), dtype=torch.uint8)
    dist.broadcast(token, 0)
    assert lib.thvm_cuda_dp_init(rank, world, (C.c_uint8 * 128)(*token.tolist())) == 0, be.last_error()
    h = (C.c_uint8 * 64)()
    assert lib.thvm_cuda_dp_arena_create(1 << 20, h) == 0, be.last_error()
    every = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(every, torch.tensor(list(h), dtype=torch.uint8))
    for r in range(world):
        if r != rank:
            assert lib.thvm_cuda_dp_arena_attach(r, (C.c_uint8 * 64)(*every[r].tolist())) == 0, be.last_error()
    dist.barrier()
    losses, params = replay_steps(be, "lenet_b128", args.steps, fused=True, rank=rank, world=world)
    assert be.last_error() == "", be.last_error()
    t = torch.tensor(losses, dtype=torch.float64)
    dist.all_reduce(t)
    flat = torch.from_numpy(np.concatenate(params))
    both = [torch.zeros_like(flat) for _ in range(world)]
    dist.all_gather(both, flat)
    if rank == 0:
        out = {"losses": (t / world).numpy()}
        for r in range(world):
            pos = 0
            for n, p in zip(LENET_NAMES, params):
                out[f"r{r}_{n}"] = both[r][pos:pos + p.size].numpy()
                pos += p.size
        np.savez(args.out, **out)
    dist.barrier()
    be.shutdown()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
