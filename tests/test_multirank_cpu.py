"""world_size-2 checks of the N > 1 path on CPU ranks (gloo): rank-dependent sharding, the
channel-id broadcast and max-over-ranks helpers of bench.py, and the assembly of all-gathered
slices. The per-rank arithmetic is done by the CPU oracle here (a test may use it); on GPUs the
same slices come from the kernels (tests/test_gpu_w4a16.py::test_sharded_slices_...)."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from iree_b200 import sharding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

RANK_SCRIPT = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, %r)
    import numpy as np
    import torch, torch.distributed as dist
    import bench, oracle
    from iree_b200 import sharding, workloads
    rank, world, local = bench.dist_setup(2)
    assert world == 2 and rank == int(os.environ["RANK"])
    # channel id: created on rank 0, identical everywhere afterwards
    ident = bytes(range(128)) if rank == 0 else bytes(128)
    got = bench.dist_broadcast_bytes(world, rank, ident, 128)
    assert got == bytes(range(128)), "channel id broadcast"
    assert bench.dist_max(world, 1.0 + rank) == 2.0
    # N-sharded W4A16: every rank computes its slice, slices are all-gathered and assembled
    M, N, K = 4, 64, 256
    a, wq, s = workloads.c4_w4a16(M, N=N, K=K, seed=4)
    wq_r, s_r = sharding.shard_weights(wq, s, world, rank)
    mine = oracle.w4a16(a, wq_r, s_r)
    parts = [torch.zeros(M, N // world, dtype=torch.float16) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(mine.copy()))
    full = sharding.assemble(np.stack([p.numpy() for p in parts]))
    want = oracle.w4a16(a, wq, s)
    assert (full == want).all(), "assembled result differs from the unsharded one"
    bench.dist_barrier(world)
    print("rank", rank, "ok")
""") % ROOT


def test_two_gloo_ranks_shard_gather_and_assemble(built, tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29541", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o
        assert "rank %d ok" % r in o


def test_column_ranges_and_assembly():
    assert sharding.column_range(28672, 8, 3) == (10752, 14336)
    with pytest.raises(ValueError):
        sharding.column_range(10, 3, 0)
    with pytest.raises(ValueError):
        sharding.column_range(16, 2, 2)
    g = np.arange(2 * 3 * 4).reshape(2, 3, 4)
    full = sharding.assemble(g)
    assert full.shape == (3, 8) and (full[:, :4] == g[0]).all() and (full[:, 4:] == g[1]).all()


def test_reference_arm_runs_on_rank_zero_only(built):
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--workload", "c1_i8_1024"], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.strip() == ""       # other ranks exit 0 without work
    env["RANK"] = "0"
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--workload", "c1_i8_1024"], env=env, capture_output=True, text=True, timeout=300)
    import json
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["cpu_baseline"]["kind"] in ("reference", "port") and line["value"] > 0
