#!/usr/bin/env python
"""Benchmark of the contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One JSON line on stdout (rank 0). A "step" is one pass of the hot path over one batch of
seeded synthetic input: one contraction dispatch (plus, with N > 1 ranks, the all-gather of the
N-sharded output through the collective channel).

* ``value``    device-timed throughput with operands resident in HBM (CUDA events on the
               dispatch stream, max over ranks). Operand sets rotate so consecutive steps never
               find their inputs in L2.
* ``e2e``      the same metric through the host-buffer C-ABI call (``iree_b200_matmul_host`` /
               ``iree_b200_w4a16_host``): pinned host operands copied in, result copied out,
               every step, inside the timed region.
* ``roofline`` achieved vs the measured peak of MEASURED_PEAKS.json (fallback constants if the
               file is absent) for the dominant kernel.
* ``cpu_baseline`` the reference's own CPU arithmetic (oracle/_ref when built, else the C
               restatement) timed on this box's host cores on a bounded sample.

``--impl reference`` times only that CPU arm and prints the same line shape with
``"impl": "reference"``.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "GEMM TOP/s & TFLOP/s vs tcgen05 peak; W4A16 decode GB/s vs HBM peak"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
L2_BYTES = 126 * 1024 * 1024


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------------------------------
# Workloads. ops = 2*M*N*K; bytes = every operand and the output touched once at storage width.
# ------------------------------------------------------------------------------------------
class Workload:
    def __init__(self, name, family, desc, unit, bound, dtype, **kw):
        self.name, self.family, self.desc, self.unit, self.bound, self.dtype = name, family, desc, unit, bound, dtype
        self.__dict__.update(kw)


def workloads():
    w = {}
    w["c2_f16_4096"] = Workload("c2_f16_4096", "matmul", "C2: f16 x f16 -> f32 acc -> f16 linalg.matmul M=N=K=4096, seed 1",
                                "TFLOP/s", "tensor", "f16", kind=0, epi=0, M=4096, N=4096, K=4096, B=1)
    w["c2_f16_bmm"] = Workload("c2_f16_bmm", "matmul", "C2: f16 batch_matmul B=32 M=N=512 K=128, seed 1",
                               "TFLOP/s", "hbm", "f16", kind=0, epi=0, M=512, N=512, K=128, B=32)
    w["c1_i8_1024"] = Workload("c1_i8_1024", "matmul", "C1: i8 x i8 -> i32 linalg.matmul M=N=K=1024, seed 0",
                               "TOP/s", "tensor", "i8", kind=2, epi=1, M=1024, N=1024, K=1024, B=1)
    for m in (1, 16, 512, 4096):
        w["c3_w8a8_m%d" % m] = Workload("c3_w8a8_m%d" % m, "matmul",
                                        "C3: W8A8 M=%d N=11008 K=4096, requant to f16, seed 2" % m, "TOP/s",
                                        "hbm" if m <= 16 else "tensor", "i8", kind=2, epi=2, M=m, N=11008, K=4096, B=1)
    for m in (1, 8, 16, 128, 2048):
        w["c4_w4a16_m%d" % m] = Workload("c4_w4a16_m%d" % m, "w4a16",
                                         "C4: W4A16 group-128 M=%d N=11008 K=4096, seed 3" % m,
                                         "GB/s" if m <= 16 else "TFLOP/s", "hbm" if m <= 16 else "tensor", "f16",
                                         M=m, N=11008, K=4096)
    for m in (16, 4096):
        w["c5_w4a16_m%d" % m] = Workload("c5_w4a16_m%d" % m, "w4a16",
                                         "C5: Llama-70B-shaped W4A16 M=%d N=28672 K=8192 sharded along N, seed 4" % m,
                                         "GB/s" if m <= 16 else "TFLOP/s", "hbm" if m <= 16 else "tensor", "f16",
                                         M=m, N=28672, K=8192, sharded=True)
    # Data-tiled entry points (the micro kernels llvm-cpu's matmul is made of), on operands of the configurations above.
    w["f2_pack_rhs_c3"] = Workload("f2_pack_rhs_c3", "tiling", "pack of the C3 int8 weight matrix [4096, 11008] into RHS "
                                   "tiles [688, 2048, 16, 2] (transpose inner + outer)", "GB/s", "hbm", "u8", op="pack",
                                   M=0, N=11008, K=4096)
    w["f2_unpack_acc_c2"] = Workload("f2_unpack_acc_c2", "tiling", "unpack of a C2-sized f32 accumulator [256, 256, 16, 16] "
                                     "to row-major [4096, 4096]", "GB/s", "hbm", "u32", op="unpack", M=4096, N=4096, K=0)
    w["f2_mmt4d_c1"] = Workload("f2_mmt4d_c1", "tiling", "mmt4d s8s8s32 on C1-sized tiled operands [64, 512, 16, 2] x "
                                "[64, 512, 16, 2] -> [64, 64, 16, 16]", "TOP/s", "tensor", "i8", op="mmt4d",
                                M=1024, N=1024, K=1024)
    w["f2_mmt4d_c3_m512"] = Workload("f2_mmt4d_c3_m512", "tiling", "mmt4d s8s8s32 on C3-sized tiled operands, M=512 "
                                     "N=11008 K=4096 in 16x16x2 tiles", "TOP/s", "tensor", "i8", op="mmt4d",
                                     M=512, N=11008, K=4096)
    return w


def algorithmic(wl, n_local=None):
    """(ops, bytes) of one dispatch; n_local overrides N for an N-sharded rank."""
    N = n_local if n_local is not None else wl.N
    if wl.family == "matmul":
        es = 1 if wl.kind == 2 else 2
        osz = 4 if wl.epi == 1 else 2
        B = wl.B
        ops = 2.0 * B * wl.M * N * wl.K
        byts = B * (wl.M * wl.K + wl.K * N) * es + B * wl.M * N * osz
        if wl.epi == 2:
            byts += 4 * (wl.M + N)
        return ops, float(byts)
    ops = 2.0 * wl.M * N * wl.K
    byts = N * wl.K / 2 + N * (wl.K // 128) * 2 + wl.M * wl.K * 2 + wl.M * N * 2
    return ops, float(byts)


def metric_value(wl, ops, byts, seconds):
    if wl.unit == "GB/s":
        return byts / seconds / 1e9
    return ops / seconds / 1e12


# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0, t1):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [l for (t, l) in self.lines if t0 <= t <= t1 + 0.06] or [l for (_, l) in self.lines[-2:]]
        for l in rows:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = max(mx, float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# CPU arm: the reference's own arithmetic on the host cores.
# ------------------------------------------------------------------------------------------
def cpu_arm(wl, steps=1, warmup=0):
    import oracle
    from iree_b200 import workloads as gen
    cores = os.cpu_count() or 1
    kind = "reference" if oracle.have_ref() else "port"
    if wl.family == "tiling":
        from iree_b200 import data_tiling
        arrays = data_tiling.operands(wl)
        use_ref = oracle.have_ref()
        kind, cores = ("reference" if use_ref else "port"), 1
        sample = "the whole operation through %s, 1 thread" % (
            "the reference's iree_uk_%s" % wl.op if use_ref else "the plain-C restatement")
        if wl.op == "pack":
            K, N = arrays[0].shape
            fn = oracle.pack_ref if use_ref else oracle.pack_port

            def once():
                fn(arrays[0], (N // 16, K // 2, 16, 2), True, True)
            ops_per, byts_per = 0.0, 2.0 * arrays[0].nbytes
        elif wl.op == "unpack":
            fn = oracle.unpack_ref if use_ref else oracle.unpack_port

            def once():
                fn(arrays[0], (wl.M, wl.N))
            ops_per, byts_per = 0.0, 2.0 * arrays[0].nbytes
        else:
            fn = oracle.mmt4d_ref if use_ref else oracle.mmt4d_port

            def once():
                fn(oracle.TYPE_S8S8S32, arrays[0], arrays[1])
            ops_per = 2.0 * wl.M * wl.N * wl.K
            byts_per = float(arrays[0].nbytes + arrays[1].nbytes + wl.M * wl.N * 4)
    elif wl.family == "matmul":
        t = oracle.TYPE_S8S8S32 if wl.kind == 2 else oracle.TYPE_F16F16F32
        rng = np.random.default_rng(1)
        M, N, K = wl.M, wl.N, wl.K
        if wl.kind == 2:
            a = rng.integers(-128, 128, (M, K), dtype=np.int8)
            b = rng.integers(-127, 128, (K, N), dtype=np.int8)
        else:
            a = (rng.standard_normal((M, K), dtype=np.float32) * K ** -0.5).astype(np.float16)
            b = (rng.standard_normal((K, N), dtype=np.float32) * K ** -0.5).astype(np.float16)
        sample = "one batch element: pack(LHS)+pack(RHS)+iree_uk_mmt4d+unpack+epilogue, M=%d N=%d K=%d, %d threads" % (
            M, N, K, cores)

        def once():
            if kind == "reference":
                acc = oracle.matmul_ref(t, a, b, threads=cores)
            else:
                acc = oracle.matmul_port(t, a[:64], b)  # the scalar restatement: a 64-row slab
            if wl.epi == 0:
                oracle.truncf(acc)
            return acc.shape[0]
        rows_done = M if kind == "reference" else min(64, M)
        if kind != "reference":
            sample = "64-row slab of the same matmul through the scalar C restatement, 1 thread"
            cores = 1
        ops_per = 2.0 * rows_done * N * K
        byts_per = (rows_done * K + K * N) * (1 if wl.kind == 2 else 2) + rows_done * N * (4 if wl.epi == 1 else 2)
    else:
        n = min(wl.N, 2048)
        a, wq, s = gen.c4_w4a16(wl.M, N=n, K=wl.K, seed=3)
        sample = "W4A16 restatement (plain C, -O3) on the first %d of %d output columns, M=%d K=%d, %d threads" % (
            n, wl.N, wl.M, wl.K, cores)
        kind = "port"

        def once():
            oracle.w4a16(a, wq, s, threads=cores)
        ops_per = 2.0 * wl.M * n * wl.K
        byts_per = n * wl.K / 2 + n * (wl.K // 128) * 2 + wl.M * wl.K * 2 + wl.M * n * 2
    for _ in range(warmup):
        once()
    t0 = time.perf_counter()
    for _ in range(steps):
        once()
    dt = (time.perf_counter() - t0) / steps
    return {"value": metric_value(wl, ops_per, byts_per, dt), "unit": wl.unit, "cores": cores, "kind": kind,
            "sample": sample, "seconds_per_step": dt}


# ------------------------------------------------------------------------------------------
def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend="gloo", rank=rank, world_size=world)
    return rank, world, local


def dist_barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def dist_max(world, x):
    if world > 1:
        import torch
        import torch.distributed as dist
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])
    return x


def dist_broadcast_bytes(world, rank, data, size):
    if world == 1:
        return data
    import torch
    import torch.distributed as dist
    t = torch.zeros(size, dtype=torch.uint8)
    if rank == 0:
        t[:] = torch.frombuffer(bytearray(data), dtype=torch.uint8)
    dist.broadcast(t, src=0)
    return bytes(t.numpy().tobytes())


def allgather_mode(block_bytes):
    """IREE_B200_ALLGATHER=peer|nccl; by default peer copies (copy engines, no SMs) for blocks of a
    megabyte or more and the NCCL collective below that, where its lower latency wins."""
    mode = os.environ.get("IREE_B200_ALLGATHER", "auto")
    if mode == "auto":
        mode = "peer" if block_bytes >= (1 << 20) else "nccl"
    return mode


def make_peer_gather(ctx, channel, rank, world, gathers):
    if channel is None or allgather_mode(gathers[0].nbytes // world) == "nccl":
        return None
    from iree_b200.sharding import PeerGather
    return PeerGather(ctx, channel, rank, world, gathers)


def verify_gather(ctx, world, rank, send_buffers, gather_buffers, slot_bytes):
    """Every slot of every receive buffer must hold the block the owning rank computed (checksums
    travel over the control plane). Run after the timed region, with all streams idle."""
    import torch
    import torch.distributed as dist
    mine = torch.zeros(len(send_buffers), dtype=torch.int64)
    for k, b in enumerate(send_buffers):
        mine[k] = int(b.download(np.uint16, (slot_bytes // 2,)).astype(np.uint64).sum() & np.uint64(0x7fffffffffffffff))
    everyone = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    bad = 0
    for k, g in enumerate(gather_buffers):
        host = g.download(np.uint16, (world, slot_bytes // 2))
        for p in range(world):
            got = int(host[p].astype(np.uint64).sum() & np.uint64(0x7fffffffffffffff))
            bad += got != int(everyone[p][k])
    return bad


def run_b200(args, wl):
    import ctypes as C
    import iree_b200 as ib
    from iree_b200 import runtime as rt
    from iree_b200 import workloads as gen
    rank, world, local = dist_setup(args.gpus)
    ctx = ib.Context(local)
    lib = ib.library()
    peaks, peak_src = load_peaks()
    # Exports that order themselves on the device (the decode kernels) may start, and prefetch their
    # first weight tiles, before the dispatch ahead of them has finished; stream order of every
    # read of an earlier result is kept by the kernels themselves.
    ctx.set_dispatch_overlap(True)
    if world > 1 and int(os.environ.get("IREE_B200_RESERVED_SMS", "0")):
        # optional: leave SMs free for the collective's blocks (measured at 2 GPUs: no gain, off by default)
        ctx.set_reserved_sms(int(os.environ["IREE_B200_RESERVED_SMS"]))

    channel = None
    if world > 1:
        ident = C.create_string_buffer(128)
        if rank == 0:
            rt.check(lib.iree_hal_b200_channel_create_id(ident, C.c_size_t(128)))
        raw = dist_broadcast_bytes(world, rank, ident.raw, 128)
        channel = C.c_void_p()
        rt.check(lib.iree_hal_b200_channel_create(ctx.device, raw, C.c_size_t(128), C.c_int32(rank),
                                                  C.c_int32(world), C.byref(channel)))

    # ---- operands --------------------------------------------------------------------
    if wl.family == "matmul":
        if wl.name.startswith("c1"):
            a, b = gen.c1_i8_matmul()
            scales = None
        elif wl.name == "c2_f16_4096":
            a, b = gen.c2_f16_matmul()
            scales = None
        elif wl.name == "c2_f16_bmm":
            a, b = gen.c2_f16_batch_matmul()
            scales = None
        else:
            a, b, sa, sw = gen.c3_w8a8(wl.M)
            scales = (sa, sw)
        n_local = wl.N
        ops, byts = algorithmic(wl)
        out_dtype = rt.out_dtype(wl.kind, wl.epi)
        out_shape = (wl.B, wl.M, wl.N) if wl.B > 1 else (wl.M, wl.N)
        set_bytes = a.nbytes + b.nbytes + int(np.prod(out_shape)) * np.dtype(out_dtype).itemsize
        n_sets = max(2, int(np.ceil(2.2 * L2_BYTES / set_bytes))) if set_bytes < 2 * L2_BYTES else 1
        n_sets = min(n_sets, 64)
        sets = []
        for _ in range(n_sets):
            da, db = ctx.to_device(a), ctx.to_device(b)
            dc = ctx.alloc(int(np.prod(out_shape)) * np.dtype(out_dtype).itemsize)
            ws = ctx.workspace()
            p = rt.MatmulParams(wl.kind, wl.epi, wl.M, wl.N, wl.K, wl.B, ib.RHS_KN, 0, 0)
            bn = ctx.matmul_prepare(p, da, db, ws)
            rs = ctx.to_device(scales[0]) if scales else None
            cs = ctx.to_device(scales[1]) if scales else None
            sets.append((p, da, db, dc, ws, bn, rs, cs))
        etype = {np.dtype(np.float16): 1, np.dtype(np.int32): 2, np.dtype(np.float32): 3, np.dtype(np.uint16): 4}[
            np.dtype(out_dtype)]

        gathers = [ctx.alloc(world * int(np.prod(out_shape)) * np.dtype(out_dtype).itemsize) for _ in sets] \
            if channel is not None else None
        peer = make_peer_gather(ctx, channel, rank, world, gathers)
        out_bytes = int(np.prod(out_shape)) * np.dtype(out_dtype).itemsize

        def step(i):
            p, da, db, dc, ws, bn, rs, cs = sets[i % n_sets]
            if channel is not None and i % n_sets == 0:
                # the operand set about to be overwritten was read by a gather n_sets steps ago
                rt.check(lib.iree_hal_b200_command_buffer_join_collectives(ctx.command_buffer))
            ctx.matmul_run(p, da, db, dc, ws, bn, rs, cs)
            if peer is not None:
                peer.gather(i % n_sets, dc, out_bytes)   # copy engines, beside the next steps' dispatches
            elif channel is not None:
                # the gather of this step overlaps the next steps' dispatches (second stream)
                rt.check(lib.iree_hal_b200_command_buffer_all_gather_overlapped(
                    ctx.command_buffer, channel, C.c_int32(etype), C.c_void_p(dc.ptr),
                    C.c_void_p(gathers[i % n_sets].ptr), C.c_size_t(int(np.prod(out_shape)))))

        def check():
            for s in sets:
                ctx.workspace_status(s[4])

        host_out = ctx.pinned_empty(out_shape, out_dtype)
        pa, pb = ctx.pinned_copy(a), ctx.pinned_copy(b)
        ps = (ctx.pinned_copy(scales[0]), ctx.pinned_copy(scales[1])) if scales else None

        def e2e_step():
            p = rt.MatmulParams(wl.kind, wl.epi, wl.M, wl.N, wl.K, wl.B, ib.RHS_KN, 0, 0)
            ctx.matmul_host(p, pa, pb, host_out, ps[0] if ps else None, ps[1] if ps else None)
        h2d = a.nbytes + b.nbytes + (scales[0].nbytes + scales[1].nbytes if scales else 0)
        d2h = host_out.nbytes
        workload_desc = wl.desc + ("; weak scaling: every rank runs its own N-slice of an N=%d*%d problem and the f16 "
                                   "outputs are all-gathered through the channel" % (wl.N, world) if world > 1 else "")
        l2_note = "operands rotate over %d sets (%.0f MB > 126 MB L2)" % (n_sets, n_sets * set_bytes / 1e6)
    elif wl.family == "tiling":
        from iree_b200 import data_tiling
        if world > 1:
            raise SystemExit("the data-tiling workloads are single-GPU (replicas only)")
        state = data_tiling.bench_state(ctx, wl)
        step, check, e2e_step = state.step, state.check, state.e2e_step
        ops, byts, h2d, d2h = state.ops, state.bytes, state.h2d, state.d2h
        workload_desc, l2_note = state.desc, state.l2_note
    else:
        from iree_b200 import w4a16 as w4
        state = w4.bench_state(ctx, wl, rank, world, channel, make_peer_gather)
        step, check, e2e_step = state.step, state.check, state.e2e_step
        ops, byts, h2d, d2h = state.ops, state.bytes, state.h2d, state.d2h
        workload_desc, l2_note = state.desc, state.l2_note

    # ---- timed region -------------------------------------------------------------------
    # One rank: the K steps are recorded once as a CUDA graph (the reference's graph command
    # buffer mode) and replayed by a single launch, so host launch overhead does not sit between
    # the dispatches. Several ranks: stream mode, each step is dispatch + all-gather.
    for i in range(max(args.warmup, 3)):
        step(i)
    ctx.synchronize()
    check()
    graph = None
    if world == 1:
        ctx.begin_graph()
        for i in range(args.steps):
            step(i)
        graph = ctx.end_graph()
        graph.execute()          # untimed: first replay uploads the graph
        ctx.synchronize()
    dist_barrier(world)
    launches0 = ctx.launch_count
    with ClockSampler(local) as clocks:
        time.sleep(0.06)
        t_begin = time.time()
        e0 = ctx.event().record()
        if graph is not None:
            graph.execute()
        else:
            for i in range(args.steps):
                step(i)
        if channel is not None:
            rt.check(lib.iree_hal_b200_command_buffer_join_collectives(ctx.command_buffer))
        e1 = ctx.event().record()
        ms = e0.elapsed_ms(e1)
        ctx.synchronize()
        t_end = time.time()
        time.sleep(0.06)
    launches = ctx.launch_count - launches0
    dist_barrier(world)
    check()
    ms = dist_max(world, ms)
    sec_per_step = ms / 1e3 / args.steps
    clock_summary = clocks.summary(t_begin, t_end)

    gather_mismatches = None
    if world > 1 and args.verify:
        ctx.synchronize()
        dist_barrier(world)
        if wl.family == "matmul":
            gather_mismatches = verify_gather(ctx, world, rank, [x[3] for x in sets], gathers, out_bytes)
        else:
            gather_mismatches = verify_gather(ctx, world, rank, [x[4] for x in state.sets], state.gathers,
                                              wl.M * (wl.N // world if getattr(wl, "sharded", False) else wl.N) * 2)
        gather_mismatches = int(dist_max(world, float(gather_mismatches)))
        dist_barrier(world)

    # ---- end to end through host buffers ----------------------------------------------------
    e2e_steps = max(1, min(args.steps, int(os.environ.get("IREE_B200_E2E_STEPS", "10"))))
    e2e_step()
    dist_barrier(world)
    e0 = ctx.event().record()
    for _ in range(e2e_steps):
        e2e_step()
    e1 = ctx.event().record()
    e2e_sec = dist_max(world, e0.elapsed_ms(e1)) / 1e3 / e2e_steps

    if rank == 0:
        timed_seconds = ms / 1e3
        if wl.bound == "tensor":
            # Denominator: the sustained cuBLAS figure when the timed region itself ran in that regime
            # (longer than a second, or the sampled clocks show the 1 kW power cap holding the SM clock
            # down, which sets in within tens of milliseconds of back-to-back GEMMs), else the burst one.
            capped = "sw_power_cap" in (clock_summary.get("reasons") or [])
            peak_key = "bf16_tflops_sustained" if (timed_seconds > 1.0 or (capped and timed_seconds > 0.05)) else "bf16_tflops"
            achieved = ops / sec_per_step / 1e12
            scale = 2.0 if wl.dtype == "i8" else 1.0   # the i8 tensor rate is twice the 16-bit rate
            peak = float(peaks[peak_key]) * scale
            r_unit = "TOP/s" if wl.dtype == "i8" else "TFLOP/s"
            peak_note = "%s %s%s" % (peak_src, peak_key, " x2 (i8 rate = 2 x measured bf16)" if scale == 2.0 else "")
        else:
            achieved = byts / sec_per_step / 1e9
            peak, r_unit, peak_note = float(peaks["hbm_gbs"]), "GB/s", "%s hbm_gbs" % peak_src
        traffic = None
        prof = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(prof):
            with open(prof) as f:
                traffic = json.load(f).get(wl.name)
        line = {
            "metric": METRIC, "value": metric_value(wl, ops, byts, sec_per_step) * world, "unit": wl.unit,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": sec_per_step * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": {"workload": workload_desc, "name": wl.name, "l2": l2_note,
                       "submission": ("CUDA graph of %d dispatches" % args.steps if world == 1 else "stream") +
                                     ", programmatic dependent launch for the decode exports",
                       "parallelism": "1 rank" if world == 1 else "N-sharded x%d + all-gather (%s)" % (
                           world, "NCCL" if allgather_mode(d2h) == "nccl"
                           else "peer copies over NVLink by the copy engines + channel barrier")},
            "roofline": {"bound": wl.bound, "achieved": achieved, "peak": peak, "unit": r_unit,
                         "frac": achieved / peak, "traffic": traffic, "peak_source": peak_note,
                         "frac_of_burst_peak": (achieved / (float(peaks["bf16_tflops"]) * scale)) if wl.bound == "tensor" else None,
                         "algorithmic_bytes": byts, "algorithmic_ops": ops},
            "e2e": {"value": metric_value(wl, ops, byts, e2e_sec) * world, "unit": wl.unit,
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_sec * 1e3},
            "gpu_launches": int(launches), "clocks": clock_summary,
        }
        if gather_mismatches is not None:
            line["config"]["gather_mismatches"] = gather_mismatches
        if world == 1:
            line["cpu_baseline"] = cpu_arm(wl)
        print(json.dumps(line), flush=True)
    dist_barrier(world)
    ctx.close()


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 5))
    base = cpu_arm(wl, steps=steps, warmup=min(args.warmup, 1))
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": wl.unit,
            "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps, "warmup": min(args.warmup, 1),
            "ms_per_step": base["seconds_per_step"] * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": {"workload": wl.desc, "name": wl.name},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2_f16_4096")
    ap.add_argument("--verify", action="store_true",
                    help="N > 1: after the timed region, check every rank's gathered buffers against the owners' checksums")
    args = ap.parse_args()
    table = workloads()
    if args.workload not in table:
        raise SystemExit("unknown workload %s; choose from %s" % (args.workload, ", ".join(sorted(table))))
    wl = table[args.workload]
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_b200(args, wl)


if __name__ == "__main__":
    main()
