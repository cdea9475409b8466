"""One rank of a data-parallel LeNet run (launched by tests/test_dp.py or torchrun).

Every rank runs the staged LeNet driver of oracle/ref_host.c on its shard of each
batch through the reference's own host runtime; after the backward pass the driver
hands the gradient buffers to a hook that sums them over the ranks:
  --device cpu   the hook reads each buffer from the reference CPU backend, all-reduces
                 it with torch.distributed (gloo) and writes it back;
  --device cuda  the hook is thvm_cuda_dp_allreduce_sum of libthvm_cuda.so (NCCL on the
                 backend's stream); the NCCL token travels over a gloo broadcast.
Rank 0 stores the losses and the final parameters in --out.
"""
import argparse
import ctypes as C
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path[:0] = [str(ROOT), str(ROOT / "tests")]

import hostref  # noqa: E402
from test_host_dropin import lenet_inputs  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--out", required=True)
    ap.add_argument("--B", type=int, default=8)          # global batch
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--lr", type=float, default=0.01)
    args = ap.parse_args()
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    os.environ.setdefault("THVM_CUDA_DEVICE", os.environ.get("LOCAL_RANK", str(rank)))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    L = hostref.lib()
    L.drv_current_ctx.restype = C.c_void_p

    x, lab, ps = lenet_inputs(args.B, args.steps)
    Bl = args.B // world
    xs = np.concatenate([x[s * args.B * 784:(s + 1) * args.B * 784].reshape(args.B, 784)[rank * Bl:(rank + 1) * Bl].ravel()
                         for s in range(args.steps)])
    labs = np.concatenate([lab[s * args.B:(s + 1) * args.B][rank * Bl:(rank + 1) * Bl] for s in range(args.steps)])

    HOOK = C.CFUNCTYPE(C.c_int, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64), C.c_uint32)
    AFTER = C.CFUNCTYPE(None)
    keep = []
    if args.device == "cpu":
        def hook(ids, counts, n):
            ctx = C.c_void_p(L.drv_current_ctx())
            for i in range(n):
                buf = np.empty(counts[i], dtype=np.float32)
                L.drv_buf_read(ctx, C.c_uint32(ids[i]), C.c_void_p(buf.ctypes.data), C.c_uint64(buf.nbytes))
                t = torch.from_numpy(buf)
                dist.all_reduce(t)
                L.drv_buf_write(ctx, C.c_uint32(ids[i]), C.c_void_p(buf.ctypes.data), C.c_uint64(buf.nbytes))
            return 0
        hook_c, after_c = HOOK(hook), AFTER(lambda: None)
        hook_ptr = hook_c
    else:
        import tinyhvm_b200
        lib = tinyhvm_b200.load()

        def after_init():
            token = torch.zeros(128, dtype=torch.uint8)
            if rank == 0:
                raw = (C.c_uint8 * 128)()
                assert lib.thvm_cuda_dp_unique_id(raw) == 0
                token = torch.tensor(list(raw), dtype=torch.uint8)
            dist.broadcast(token, 0)
            raw = (C.c_uint8 * 128)(*token.tolist())
            assert lib.thvm_cuda_dp_init(rank, world, raw) == 0, lib.thvm_cuda_last_error()
        after_c = AFTER(after_init)
        hook_ptr = C.cast(lib.thvm_cuda_dp_allreduce_sum, HOOK)
        hook_c = hook_ptr
    keep += [hook_c, after_c]
    L.drv_set_dp.argtypes = [C.c_uint32, HOOK, AFTER]
    L.drv_set_dp(world, hook_ptr, after_c)
    r = hostref.run("drv_lenet", args.device, Bl, args.steps, float(args.lr), xs, labs, np.concatenate(ps), 0)
    losses = np.array([r[f"loss{s}"][0] for s in range(args.steps)], dtype=np.float32)
    t = torch.from_numpy(losses.copy())
    dist.all_reduce(t)                                    # mean of the shard losses = the global-batch loss
    if rank == 0:
        out = {k: v for k, v in r.items() if not k.startswith("_") and not k.startswith("loss")}
        out["losses"] = t.numpy() / world
        out["seconds"] = np.array([r["_seconds"]])
        np.savez(args.out, **out)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
