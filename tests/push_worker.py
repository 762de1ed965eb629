"""Worker of tests/test_gpu_multi.py: one rank of an N-sharded W4A16 dispatch whose epilogue stores its
column block into every rank's result (run under torchrun)."""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import iree_b200 as ib  # noqa: E402
import oracle  # noqa: E402
from iree_b200 import workloads  # noqa: E402
from iree_b200.sharding import PushGather, shard_weights  # noqa: E402


def main() -> int:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group(backend="gloo", rank=rank, world_size=world)
    ctx = ib.Context(local)
    M, N, K = 512, 128 * 3 * world, 512
    n_local = N // world
    rng = np.random.default_rng(5)
    ok = True
    push = PushGather(ctx, None, rank, world, M, N, buffers=2)
    p = ib.W4A16Params(M, n_local, K, 128, N, rank * n_local, ib.W4A16_GEMM_WT, 0)
    layers = []
    for layer in range(3):                      # every rank draws the same full problem, keeps its rows
        a = rng.integers(-2, 3, (M, K)).astype(np.float16)
        wq = workloads.pack_int4(rng.integers(-8, 8, (N, K), dtype=np.int8))
        s = (2.0 ** rng.integers(-3, 1, (N, K // 128))).astype(np.float16)
        wq_r, s_r = shard_weights(wq, s, world, rank)
        want = oracle.w4a16(a, wq, s, threads=os.cpu_count() or 1)
        layers.append((ctx.to_device(a), ctx.to_device(wq_r), ctx.to_device(s_r), want))
    workspaces = {}
    # Rounds without a host barrier in between: what keeps a fast rank from overwriting a result a
    # slow rank still holds is the arrival protocol itself (two buffers in rotation).
    steps = 9
    for i in range(steps):
        da, dw, ds, want = layers[i % 3]
        key = (i % 2, i % 3)
        if key not in workspaces:
            workspaces[key] = ctx.w4a16_workspace(n_local)
            push.prepare(i % 2, p, da, dw, ds, workspaces[key])
        push.run(i, p, ds, workspaces[key])
        got = push.result(i % 2).download(np.float16, (M, N))   # stream-ordered after this rank's wait
        ok = ok and bool((got == want).all())
        ctx.workspace_status(workspaces[key])
    push.close()
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("PUSH_OK" if int(flag[0]) else "PUSH_MISMATCH", flush=True)
    ctx.close()
    return 0 if int(flag[0]) else 1


if __name__ == "__main__":
    sys.exit(main())
