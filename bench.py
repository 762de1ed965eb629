#!/usr/bin/env python
"""Benchmark of the contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--rows all|none] [--impl reference]

One JSON line on stdout (rank 0). A "step" is one pass of the hot path over one batch of
seeded synthetic input: one contraction dispatch (plus, with N > 1 ranks, the exchange that
leaves the N-sharded output complete on every rank). The default workload is the largest
single-GPU configuration and the one the benchmark list shards: the Llama-70B-shaped W4A16
product at M = 4096; with N ranks its weight rows are split N ways (fixed total work).
With one rank the line also carries `rows`: every workload of the table, each with its own
value, roofline, clocks and end-to-end figure.

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


from bench_workloads import (DEFAULT_WORKLOAD, algorithmic, describe, local_n, make_state, metric_value,
                             tiling_operands, workloads)


# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: through NVML in this process
    (one sample taken by the timing code itself right after the last launch, while the steps run, plus - with
    one rank, where the steps are one graph launch - a thread polling every 25 ms; several ranks launch step
    by step and NVML queries take driver locks that launches need too, so they are not polled),
    or, where NVML cannot be loaded, with an nvidia-smi child at 50 ms. Read-only queries."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    # bits of nvmlDeviceGetCurrentClocksEventReasons, in the order of the four names of summary()
    REASON_BITS = (0x8, 0x40, 0x20, 0x4)

    def __init__(self, index, poll=True):
        self.index, self.lines, self.proc, self.nvml, self.handle, self.poll = index, [], None, None, None, poll
        self.stop = threading.Event()
        self.period = float(os.environ.get("IREE_B200_CLOCK_POLL_MS", "25")) / 1e3

    def _nvml_line(self):
        n, h = self.nvml, self.handle
        sm = n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)
        mx = n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)
        get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        bits = int(get(h))
        flags = ["Active" if bits & b else "Not Active" for b in self.REASON_BITS]
        return ",".join([str(self.index), str(sm), str(mx), "", hex(bits)] + flags)

    def sample_now(self):
        """One sample taken by the caller's thread (so that even a region of a few milliseconds has one)."""
        if self.nvml is not None:
            try:
                self.lines.append((time.time(), self._nvml_line()))
            except Exception:
                pass

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.nvml = pynvml
            self._nvml_line()
            self.thread = None
            if self.poll:
                self.thread = threading.Thread(target=self._poll, daemon=True)
                self.thread.start()
            return self
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _poll(self):
        while not self.stop.is_set():
            try:
                self.lines.append((time.time(), self._nvml_line()))
            except Exception:
                return
            self.stop.wait(self.period)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def __exit__(self, *exc):
        self.stop.set()
        if self.nvml is not None and self.thread is not None:
            self.thread.join(timeout=1)
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
def cpu_arm(wl, steps=1, warmup=0, world=1, budget_s=1.5):
    """Times the reference's CPU implementation of the workload on this box's host cores, on a
    bounded sample: whole problems where a step takes about `budget_s` seconds or less, else the
    leading rows / columns that do (the sample is stated). N-sharded workloads use one rank's slice,
    like the GPU arm."""
    import oracle
    from iree_b200 import workloads as gen
    cores = os.cpu_count() or 1
    kind = "reference" if oracle.have_ref() else "port"
    if wl.family == "tiling":
        arrays = tiling_operands(wl)
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
        elif wl.op == "pack_lhs":
            fn = oracle.pack_ref if use_ref else oracle.pack_port
            sample = sample.replace("iree_uk_pack_lhs", "iree_uk_pack")

            def once():
                fn(arrays[0], (wl.M // 16, wl.K // 2, 16, 2), False, False)
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
        # Grouped int4 dequant + contraction: the reference has no ukernel for it (llvm-cpu generates
        # that loop nest), so the timed code is the plain-C restatement of the dispatch. The sample is
        # the leading n columns of one rank's slice, n sized from a probe so that a step stays near
        # the budget.
        kind = "port"
        n_full = local_n(wl, world)
        probe_n = min(n_full, 64)
        a, wq, s = gen.c4_w4a16(wl.M, N=probe_n, K=wl.K, seed=3)
        t0 = time.perf_counter()
        oracle.w4a16(a, wq, s, threads=cores)
        per_col = max((time.perf_counter() - t0) / probe_n, 1e-7)
        n = int(min(n_full, max(64, budget_s / per_col))) // 16 * 16
        a, wq, s = gen.c4_w4a16(wl.M, N=n, K=wl.K, seed=3)
        sample = "W4A16 restatement (plain C, -O3) on the first %d of %d output columns, M=%d K=%d, %d threads" % (
            n, n_full, wl.M, wl.K, cores)

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


def checksum(host_u16):
    return int(host_u16.astype(np.uint64).sum() & np.uint64(0x7fffffffffffffff))


def verify_gather(ctx, world, rank, st, wl):
    """Every rank must hold the block every other rank computed (checksums travel over the control
    plane). Run after the timed region, with all streams idle. Returns the number of wrong blocks."""
    import torch
    import torch.distributed as dist
    push = getattr(st, "push", None)
    n_sets = len(st.sets)
    mine = torch.zeros(n_sets, dtype=torch.int64)
    n_loc = local_n(wl, world)
    for k in range(n_sets):
        if push is not None:
            full = push.result(k).download(np.uint16, (wl.M, wl.N))
            mine[k] = checksum(full[:, rank * n_loc:(rank + 1) * n_loc])
        else:
            mine[k] = checksum(st.send_buffers[k].download(np.uint16, (st.slot_bytes // 2,)))
    everyone = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    bad = 0
    for k in range(n_sets):
        if push is not None:
            full = push.result(k).download(np.uint16, (wl.M, wl.N))
            for p in range(world):
                bad += checksum(full[:, p * n_loc:(p + 1) * n_loc]) != int(everyone[p][k])
        else:
            host = st.gathers[k].download(np.uint16, (world, st.slot_bytes // 2))
            for p in range(world):
                bad += checksum(host[p]) != int(everyone[p][k])
    return bad


def roofline_of(wl, ops, byts, sec_per_step, timed_seconds, clock_summary, peaks, peak_src):
    burst, sustained = float(peaks["bf16_tflops"]), float(peaks["bf16_tflops_sustained"])
    if wl.bound == "tensor":
        # Denominator: the sustained cuBLAS figure when the timed region itself ran in that regime
        # (longer than a second, or the sampled clocks show the 1 kW power cap holding the SM clock
        # down, which sets in within tens of milliseconds of back-to-back GEMMs), else the burst one.
        # Both fractions are always reported next to it.
        capped = "sw_power_cap" in (clock_summary.get("reasons") or [])
        peak_key = "bf16_tflops_sustained" if (timed_seconds > 1.0 or (capped and timed_seconds > 0.05)) else "bf16_tflops"
        achieved = ops / sec_per_step / 1e12
        scale = 2.0 if wl.dtype == "i8" else 1.0   # the i8 tensor rate is twice the 16-bit rate
        peak = float(peaks[peak_key]) * scale
        r_unit = "TOP/s" if wl.dtype == "i8" else "TFLOP/s"
        peak_note = "%s %s%s" % (peak_src, peak_key, " x2 (i8 rate = 2 x measured bf16)" if scale == 2.0 else "")
        extra = {"frac_of_burst_peak": achieved / (burst * scale), "frac_of_sustained_peak": achieved / (sustained * scale)}
    else:
        achieved = byts / sec_per_step / 1e9
        peak, r_unit, peak_note = float(peaks["hbm_gbs"]), "GB/s", "%s hbm_gbs" % peak_src
        extra = {"frac_of_burst_peak": None, "frac_of_sustained_peak": None}
    traffic = None
    prof = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(prof):
        with open(prof) as f:
            traffic = json.load(f).get(wl.name)
    r = {"bound": wl.bound, "achieved": achieved, "peak": peak, "unit": r_unit, "frac": achieved / peak,
         "traffic": traffic, "peak_source": peak_note, "algorithmic_bytes": byts, "algorithmic_ops": ops}
    r.update(extra)
    return r


def measure(ctx, wl, rank, world, local, channel, steps, warmup, verify, peaks, peak_src, e2e_steps):
    """One workload: device-timed steps, then the end-to-end steps. Returns the JSON fields."""
    import ctypes as C
    from iree_b200 import runtime as rt
    lib = rt.library()
    st = make_state(ctx, wl, rank, world, channel)
    step, check = st.step, st.check
    # One rank: the K steps are recorded once as a CUDA graph (the reference's graph command
    # buffer mode) and replayed by a single launch, so host launch overhead does not sit between
    # the dispatches. Several ranks: stream mode, each step is dispatch + output exchange.
    for i in range(max(warmup, 3)):
        step(i)
    ctx.synchronize()
    check()
    graph = None
    if world == 1:
        ctx.begin_graph()
        for i in range(steps):
            step(i)
        graph = ctx.end_graph()
        graph.execute()          # untimed: first replay uploads the graph
        ctx.synchronize()
    dist_barrier(world)
    launches0 = ctx.launch_count
    with ClockSampler(local, poll=world == 1) as clocks:
        time.sleep(0.06)
        t_begin = time.time()
        e0 = ctx.event().record()
        if graph is not None:
            graph.execute()
        else:
            for i in range(steps):
                step(i)
        if channel is not None:
            rt.check(lib.iree_hal_b200_command_buffer_join_collectives(ctx.command_buffer))
        e1 = ctx.event().record()
        clocks.sample_now()      # the steps are in flight: submission returns before they finish
        ms = e0.elapsed_ms(e1)
        ctx.synchronize()
        t_end = time.time()
        time.sleep(0.06)
    launches = ctx.launch_count - launches0
    if graph is not None:
        graph.release()
    dist_barrier(world)
    check()
    ms = dist_max(world, ms)
    sec_per_step = ms / 1e3 / steps
    clock_summary = clocks.summary(t_begin, t_end)

    gather_mismatches = None
    if world > 1 and verify and wl.family != "tiling":
        ctx.synchronize()
        dist_barrier(world)
        gather_mismatches = int(dist_max(world, float(verify_gather(ctx, world, rank, st, wl))))
        dist_barrier(world)

    # ---- end to end through host buffers ----------------------------------------------------
    e2e_steps = max(1, min(steps, e2e_steps))
    st.e2e_step()
    dist_barrier(world)
    e0 = ctx.event().record()
    for _ in range(e2e_steps):
        st.e2e_step()
    e1 = ctx.event().record()
    e2e_sec = dist_max(world, e0.elapsed_ms(e1)) / 1e3 / e2e_steps

    ops, byts = st.ops, st.bytes
    out = {
        "name": wl.name, "value": metric_value(wl, ops, byts, sec_per_step) * world, "unit": wl.unit,
        "ms_per_step": sec_per_step * 1e3, "steps": steps, "dtype": wl.dtype,
        "roofline": roofline_of(wl, ops, byts, sec_per_step, ms / 1e3, clock_summary, peaks, peak_src),
        "e2e": {"value": metric_value(wl, ops, byts, e2e_sec) * world, "unit": wl.unit,
                "h2d_bytes_per_step": int(st.h2d), "d2h_bytes_per_step": int(st.d2h), "ms_per_step": e2e_sec * 1e3},
        "gpu_launches": int(launches), "clocks": clock_summary,
    }
    if gather_mismatches is not None:
        out["gather_mismatches"] = gather_mismatches
    st.release()
    return out


def run_b200(args, wl, table):
    import ctypes as C
    import iree_b200 as ib
    from iree_b200 import runtime as rt
    rank, world, local = dist_setup(args.gpus)
    ctx = ib.Context(local)
    lib = ib.library()
    peaks, peak_src = load_peaks()
    # Exports that order themselves on the device (the decode kernels, the tensor-core GEMMs) may be
    # launched, set up and -- the decode kernels -- prefetch their first weight tiles before the dispatch
    # ahead of them has finished; stream order of every read of an earlier result is kept by the
    # kernels themselves.
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

    e2e_steps = int(os.environ.get("IREE_B200_E2E_STEPS", "10"))
    verify = world > 1 and not args.no_verify
    main_row = measure(ctx, wl, rank, world, local, channel, args.steps, args.warmup, verify, peaks, peak_src, e2e_steps)

    # Every workload of the measurement table as a row of the same line (one rank only): a short
    # graph-replayed run each, with its own clock record and end-to-end figure.
    rows = []
    if world == 1 and args.rows == "all":
        for name, w in table.items():
            if name == wl.name:
                rows.append(dict(main_row))
                continue
            rows.append(measure(ctx, w, rank, world, local, None, min(args.steps, args.row_steps), 3, False, peaks,
                                peak_src, min(e2e_steps, 3)))

    if rank == 0:
        sharded = wl.sharded and world > 1
        line = {
            "metric": METRIC, "value": main_row["value"], "unit": wl.unit,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": main_row["ms_per_step"],
            "higher_is_better": True, "scaling": "strong" if sharded or world == 1 else "weak", "vs_baseline": None,
            "dtype": wl.dtype, "data": "synthetic", "config": describe(wl, world, args.steps),
            "roofline": main_row["roofline"], "e2e": main_row["e2e"],
            "gpu_launches": main_row["gpu_launches"], "clocks": main_row["clocks"],
        }
        if "gather_mismatches" in main_row:
            line["gather_mismatches"] = main_row["gather_mismatches"]
        if world == 1:
            line["cpu_baseline"] = cpu_arm(wl)
            if rows:
                line["rows"] = rows
        print(json.dumps(line), flush=True)
    dist_barrier(world)
    ctx.close()


def run_reference(args, wl):
    """The reference's CPU implementation of the path on this box's host cores, all of them, on
    the GPU arm's config / metric / unit. Under torchrun rank 0 alone works and prints."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    warm = max(1, min(args.warmup, 2))
    budget = min(1.5, 90.0 / max(1, args.steps + warm))   # the whole run stays within a couple of minutes
    base = cpu_arm(wl, steps=args.steps, warmup=warm, world=world, budget_s=budget)
    sharded = wl.sharded and world > 1
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": wl.unit,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": base["seconds_per_step"] * 1e3, "higher_is_better": True,
            "scaling": "strong" if sharded or world == 1 else "weak",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": describe(wl, world, args.steps),
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--rows", default="all", choices=["all", "none"],
                    help="one rank: also measure every workload of the table and report them as `rows`")
    ap.add_argument("--row-steps", type=int, default=20, help="steps per row (at most --steps)")
    ap.add_argument("--no-verify", action="store_true",
                    help="N > 1: skip the check of every rank's gathered output against the owners' checksums")
    args = ap.parse_args()
    table = workloads()
    if args.workload not in table:
        raise SystemExit("unknown workload %s; choose from %s" % (args.workload, ", ".join(sorted(table))))
    wl = table[args.workload]
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_b200(args, wl, table)


if __name__ == "__main__":
    main()
