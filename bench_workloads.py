"""Workload table of bench.py and the buffers / step functions behind every row.

Not part of the library: this is measurement scaffolding that sits next to bench.py. Every
workload is one configuration of the benchmark list (C1 .. C5, in that order) or one of the
data-tiled entry points on operands of those configurations. A "state" owns the device buffers of
a workload on one rank and offers

    step(i)      one pass of the hot path over operand set i (device resident)
    check()      raises if a kernel left a non-zero status word
    e2e_step()   the same through the host-buffer C-ABI call (pinned host operands in, result out)
    release()    frees what the state allocated

ops = 2*M*N*K; bytes = every operand and the output touched once at storage width.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

import iree_b200 as ib
from iree_b200 import runtime as rt
from iree_b200 import workloads as gen

L2_BYTES = 126 * 1024 * 1024


class Workload:
    def __init__(self, name, family, desc, unit, bound, dtype, **kw):
        self.name, self.family, self.desc, self.unit, self.bound, self.dtype = name, family, desc, unit, bound, dtype
        self.sharded = False
        self.__dict__.update(kw)


def workloads():
    w = {}
    w["c1_i8_1024"] = Workload("c1_i8_1024", "matmul", "C1: i8 x i8 -> i32 linalg.matmul M=N=K=1024, seed 0",
                               "TOP/s", "tensor", "i8", kind=2, epi=1, M=1024, N=1024, K=1024, B=1)
    w["c2_f16_4096"] = Workload("c2_f16_4096", "matmul", "C2: f16 x f16 -> f32 acc -> f16 linalg.matmul M=N=K=4096, seed 1",
                                "TFLOP/s", "tensor", "f16", kind=0, epi=0, M=4096, N=4096, K=4096, B=1)
    w["c2_f16_bmm"] = Workload("c2_f16_bmm", "matmul", "C2: f16 batch_matmul B=32 M=N=512 K=128, seed 1",
                               "TFLOP/s", "hbm", "f16", kind=0, epi=0, M=512, N=512, K=128, B=32)
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
    # The same few-row products through the tensor-core decode variant (not what AUTO picks: it is
    # the slower of the two decode kernels today; the rows keep its numbers beside the other's).
    w["c4_w4a16_m16_tc"] = Workload("c4_w4a16_m16_tc", "w4a16", "C4: W4A16 group-128 M=16 N=11008 K=4096, seed 3, "
                                    "tensor-core decode variant", "GB/s", "hbm", "f16", M=16, N=11008, K=4096,
                                    variant="decode_tc")
    w["c5_w4a16_m16_tc"] = Workload("c5_w4a16_m16_tc", "w4a16", "C5: Llama-70B-shaped W4A16 M=16 N=28672 K=8192, seed 4, "
                                    "tensor-core decode variant", "GB/s", "hbm", "f16", M=16, N=28672, K=8192,
                                    sharded=True, variant="decode_tc")
    # Data-tiled entry points (the micro kernels llvm-cpu's matmul is made of), on operands of the configurations above.
    w["f2_pack_rhs_c3"] = Workload("f2_pack_rhs_c3", "tiling", "pack of the C3 int8 weight matrix [4096, 11008] into RHS "
                                   "tiles [688, 2048, 16, 2] (transpose inner + outer)", "GB/s", "hbm", "u8", op="pack",
                                   M=0, N=11008, K=4096)
    w["f2_pack_lhs_c3"] = Workload("f2_pack_lhs_c3", "tiling", "pack of C3 M=4096 int8 activations [4096, 4096] into LHS tiles "
                                   "[256, 2048, 16, 2] (no transposes)", "GB/s", "hbm", "u8", op="pack_lhs",
                                   M=4096, N=0, K=4096)
    w["f2_unpack_acc_c2"] = Workload("f2_unpack_acc_c2", "tiling", "unpack of a C2-sized f32 accumulator [256, 256, 16, 16] "
                                     "to row-major [4096, 4096]", "GB/s", "hbm", "u32", op="unpack", M=4096, N=4096, K=0)
    w["f2_mmt4d_c1"] = Workload("f2_mmt4d_c1", "tiling", "mmt4d s8s8s32 on C1-sized tiled operands [64, 512, 16, 2] x "
                                "[64, 512, 16, 2] -> [64, 64, 16, 16]", "TOP/s", "tensor", "i8", op="mmt4d",
                                M=1024, N=1024, K=1024)
    w["f2_mmt4d_c3_m512"] = Workload("f2_mmt4d_c3_m512", "tiling", "mmt4d s8s8s32 on C3-sized tiled operands, M=512 "
                                     "N=11008 K=4096 in 16x16x2 tiles", "TOP/s", "tensor", "i8", op="mmt4d",
                                     M=512, N=11008, K=4096)
    return w


DEFAULT_WORKLOAD = "c5_w4a16_m4096"


def local_n(wl, world):
    """Output columns one rank computes: N-sharded workloads split N over the ranks."""
    return wl.N // world if (wl.sharded and world > 1) else wl.N


def algorithmic(wl, n_local=None):
    """(ops, bytes) of one dispatch; n_local overrides N for an N-sharded rank."""
    N = n_local if n_local is not None else wl.N
    if wl.family == "tiling":
        if wl.op == "pack":
            return 0.0, 2.0 * wl.K * wl.N
        if wl.op == "pack_lhs":
            return 0.0, 2.0 * wl.M * wl.K
        if wl.op == "unpack":
            return 0.0, 2.0 * wl.M * wl.N * 4
        return 2.0 * wl.M * wl.N * wl.K, float(wl.M * wl.K + wl.N * wl.K + wl.M * wl.N * 4)
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


def set_count(set_bytes, cap):
    """Operand sets to rotate over so that consecutive steps never find their inputs in L2."""
    n = int(np.ceil(2.2 * L2_BYTES / set_bytes)) if set_bytes < 2 * L2_BYTES else 1
    return max(2, min(n, cap))


def describe(wl, world, steps):
    """The `config` object of the JSON line: the same for both arms of a run."""
    n_loc = local_n(wl, world)
    desc = wl.desc
    if world > 1 and wl.sharded:
        desc += "; N-sharded over %d ranks (N/world = %d columns each), f16 outputs gathered on every rank" % (world, n_loc)
    elif world > 1:
        desc += "; %d independent replicas (this workload does not shard)" % world
    return {"workload": desc, "name": wl.name,
            "l2": "operand sets rotate so that every step's operands exceed the 126 MB L2 (2.2 x L2 in rotation)",
            "submission": ("CUDA graph of %d dispatches" % steps if world == 1 else "stream") +
                          ", programmatic dependent launch for the exports that order themselves on the device (decode, tensor-core GEMMs)",
            "parallelism": "1 rank" if world == 1 else (
                "N-sharded x%d, output all-gather (%s)" % (world, gather_mode_name(wl, world)) if wl.sharded
                else "replicas x%d" % world)}


def allgather_mode(block_bytes, push_ok=False):
    """IREE_B200_ALLGATHER=push|peer|nccl. Default: the W4A16 tensor-core kernel pushes its output
    tiles into every rank's result buffer from its epilogue (push); dispatches that cannot do that
    use peer copies (copy engines) for blocks of a megabyte or more and the NCCL collective below."""
    mode = os.environ.get("IREE_B200_ALLGATHER", "auto")
    if mode == "auto":
        mode = "push" if push_ok else ("peer" if block_bytes >= (1 << 20) else "nccl")
    if mode == "push" and not push_ok:
        mode = "peer" if block_bytes >= (1 << 20) else "nccl"
    return mode


def gather_mode_name(wl, world):
    block = wl.M * local_n(wl, world) * 2
    mode = allgather_mode(block, push_ok=wl.family == "w4a16" and wl.M >= 256 and local_n(wl, world) % 8 == 0)
    return {"nccl": "NCCL all-gather through the channel",
            "peer": "peer copies over NVLink by the copy engines + channel barrier",
            "push": "epilogue stores into every rank's result buffer over NVLink + arrival flags"}[mode]


class _State:
    def __init__(self, ctx):
        self.ctx, self.buffers, self.pinned = ctx, [], []
        self.gathers, self.sets, self.peer = None, [], None

    def alloc(self, nbytes):
        b = self.ctx.alloc(nbytes)
        self.buffers.append(b)
        return b

    def to_device(self, host):
        b = self.ctx.to_device(host)
        self.buffers.append(b)
        return b

    def track(self, b):
        self.buffers.append(b)
        return b

    def pinned_copy(self, host):
        p = self.ctx.pinned_copy(host)
        self.pinned.append(p)
        return p

    def pinned_empty(self, shape, dtype):
        p = self.ctx.pinned_empty(shape, dtype)
        self.pinned.append(p)
        return p

    def release(self):
        self.ctx.synchronize()
        if self.peer is not None:
            self.peer.close()
        for b in self.buffers:
            b.free()
        lib = rt.library()
        for p in self.pinned:
            lib.iree_hal_b200_host_free(self.ctx.device, C.c_void_p(p.ctypes.data))
        self.buffers, self.pinned = [], []


def make_peer_gather(ctx, channel, rank, world, gathers):
    if channel is None or allgather_mode(gathers[0].nbytes // world) != "peer":
        return None
    from iree_b200.sharding import PeerGather
    return PeerGather(ctx, channel, rank, world, gathers)


def _gather_step(st, lib, channel, etype, i, send, count, nbytes):
    """All-gather of one step's output through the channel, overlapping the next dispatches."""
    n_sets = len(st.sets)
    if st.peer is not None:
        st.peer.gather(i % n_sets, send, nbytes)       # copy engines, beside the following dispatches
    elif channel is not None:
        rt.check(lib.iree_hal_b200_command_buffer_all_gather_overlapped(
            st.ctx.command_buffer, channel, C.c_int32(etype), C.c_void_p(send.ptr),
            C.c_void_p(st.gathers[i % n_sets].ptr), C.c_size_t(count)))


def matmul_state(ctx, wl, rank, world, channel):
    lib = rt.library()
    st = _State(ctx)
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
    st.ops, st.bytes = algorithmic(wl)
    out_dtype = rt.out_dtype(wl.kind, wl.epi)
    out_shape = (wl.B, wl.M, wl.N) if wl.B > 1 else (wl.M, wl.N)
    out_bytes = int(np.prod(out_shape)) * np.dtype(out_dtype).itemsize
    n_sets = set_count(a.nbytes + b.nbytes + out_bytes, 64)
    for _ in range(n_sets):
        da, db = st.to_device(a), st.to_device(b)
        dc = st.alloc(out_bytes)
        p = rt.MatmulParams(wl.kind, wl.epi, wl.M, wl.N, wl.K, wl.B, ib.RHS_KN, 0, 0)
        ws = st.track(ctx.matmul_workspace(p))
        bn = ctx.matmul_prepare(p, da, db, ws)
        rs = st.to_device(scales[0]) if scales else None
        cs = st.to_device(scales[1]) if scales else None
        st.sets.append((p, da, db, dc, ws, bn, rs, cs))
    etype = {np.dtype(np.float16): 1, np.dtype(np.int32): 2, np.dtype(np.float32): 3, np.dtype(np.uint16): 4}[
        np.dtype(out_dtype)]
    if channel is not None:
        st.gathers = [st.alloc(world * out_bytes) for _ in st.sets]
        st.peer = make_peer_gather(ctx, channel, rank, world, st.gathers)
    st.send_buffers = [x[3] for x in st.sets]
    st.slot_bytes = out_bytes

    def step(i):
        p, da, db, dc, ws, bn, rs, cs = st.sets[i % n_sets]
        if channel is not None and i % n_sets == 0:
            # the operand set about to be overwritten was read by a gather n_sets steps ago
            rt.check(lib.iree_hal_b200_command_buffer_join_collectives(ctx.command_buffer))
        ctx.matmul_run(p, da, db, dc, ws, bn, rs, cs)
        _gather_step(st, lib, channel, etype, i, dc, int(np.prod(out_shape)), out_bytes)

    def check():
        for s in st.sets:
            ctx.workspace_status(s[4])

    host_out = st.pinned_empty(out_shape, out_dtype)
    pa, pb = st.pinned_copy(a), st.pinned_copy(b)
    ps = (st.pinned_copy(scales[0]), st.pinned_copy(scales[1])) if scales else None

    def e2e_step():
        p = rt.MatmulParams(wl.kind, wl.epi, wl.M, wl.N, wl.K, wl.B, ib.RHS_KN, 0, 0)
        ctx.matmul_host(p, pa, pb, host_out, ps[0] if ps else None, ps[1] if ps else None)

    st.step, st.check, st.e2e_step = step, check, e2e_step
    st.h2d = a.nbytes + b.nbytes + (scales[0].nbytes + scales[1].nbytes if scales else 0)
    st.d2h = host_out.nbytes
    return st


def w4a16_state(ctx, wl, rank, world, channel):
    """With more than one rank the weight rows are sharded along N; every rank computes its
    [M, N/world] slice and every rank ends up with all slices. Three ways to get them there:
    the kernel's epilogue stores its tiles straight into every rank's [M, N] result (push), or
    the slice is all-gathered afterwards through the channel (NCCL, or copy-engine peer copies;
    the gathered buffer then holds the slices rank after rank)."""
    lib = rt.library()
    st = _State(ctx)
    M, K = wl.M, wl.K
    sharded = wl.sharded and world > 1
    n_local = local_n(wl, world)
    if wl.name.startswith("c5"):
        a, wq, s = gen.c5_w4a16_sharded(M, world if sharded else 1, rank if sharded else 0, N=wl.N, K=K)
    else:
        a, wq, s = gen.c4_w4a16(M, N=wl.N, K=K)
    st.ops, st.bytes = algorithmic(wl, n_local)
    n_sets = set_count(wq.nbytes + s.nbytes + a.nbytes + M * n_local * 2, 24)
    mode = allgather_mode(M * n_local * 2, push_ok=M >= 256 and (rank * n_local) % 8 == 0) if channel is not None else None
    push = None
    if mode == "push":
        from iree_b200.sharding import PushGather
        push = PushGather(ctx, channel, rank, world, M, wl.N, n_sets)
        st.peer = push
    for k in range(n_sets):
        da, dw, ds = st.to_device(a), st.to_device(wq), st.to_device(s)
        ws = st.track(ctx.w4a16_workspace(n_local))
        if push is not None:
            dc = push.result(k)
            p = rt.W4A16Params(M, n_local, K, 128, wl.N, rank * n_local, rt.W4A16_GEMM_WT, 0)
            push.prepare(k, p, da, dw, ds, ws)
            variant, tile_n = rt.W4A16_GEMM_WT, 128
        else:
            dc = st.alloc(M * n_local * 2)
            wanted = rt.W4A16_DECODE_TC if getattr(wl, "variant", "") == "decode_tc" else rt.W4A16_AUTO
            p = rt.W4A16Params(M, n_local, K, 128, n_local, 0, wanted, 0)
            variant, tile_n = ctx.w4a16_prepare(p, da, dw, ds, dc, ws)
        st.sets.append((p, da, dw, ds, dc, ws, variant, tile_n))
    if channel is not None and push is None:
        st.gathers = [st.alloc(world * M * n_local * 2) for _ in st.sets]
        st.peer = make_peer_gather(ctx, channel, rank, world, st.gathers)
    st.send_buffers = [x[4] for x in st.sets]
    st.slot_bytes = M * n_local * 2
    st.push = push

    def step(i):
        p, da, dw, ds, dc, ws, variant, tile_n = st.sets[i % n_sets]
        if push is not None:
            push.run(i, p, ds, ws)
            return
        if channel is not None and i % n_sets == 0:
            rt.check(lib.iree_hal_b200_command_buffer_join_collectives(ctx.command_buffer))
        ctx.w4a16_run(p, da, dw, ds, dc, ws, variant, tile_n)
        _gather_step(st, lib, channel, 1, i, dc, M * n_local, M * n_local * 2)

    def check():
        for x in st.sets:
            ctx.workspace_status(x[5])
        if push is not None:
            push.check()

    pa, pw, ps = st.pinned_copy(a), st.pinned_copy(wq), st.pinned_copy(s)
    host_out = st.pinned_empty((M, n_local), np.float16)

    def e2e_step():
        p = rt.W4A16Params(M, n_local, K, 128, n_local, 0, rt.W4A16_AUTO, 0)
        ctx.w4a16_host(p, pa, pw, ps, host_out)

    st.step, st.check, st.e2e_step = step, check, e2e_step
    st.h2d = a.nbytes + wq.nbytes + s.nbytes
    st.d2h = host_out.nbytes
    st.variant = st.sets[0][6]
    return st


def tiling_operands(wl):
    """Seeded host operands of a data-tiling workload."""
    if wl.op == "pack":
        _, w, _, _ = gen.c3_w8a8(1)            # the [K, N] int8 weight matrix of the W8A8 configuration
        return (w,)
    if wl.op == "pack_lhs":
        rng = np.random.default_rng(2)
        return (rng.integers(-128, 128, (wl.M, wl.K), dtype=np.int8),)
    if wl.op == "unpack":
        rng = np.random.default_rng(1)
        return (rng.standard_normal((wl.M // 16, wl.N // 16, 16, 16), dtype=np.float32),)
    # mmt4d on already-tiled int8 operands (16x16x2, the x86-64 VNNI tile)
    rng = np.random.default_rng(0)
    lhs = rng.integers(-128, 128, (wl.M // 16, wl.K // 2, 16, 2), dtype=np.int8)
    rhs = rng.integers(-127, 128, (wl.N // 16, wl.K // 2, 16, 2), dtype=np.int8)
    return lhs, rhs


def tiling_state(ctx, wl):
    lib = rt.library()
    st = _State(ctx)
    arrays = tiling_operands(wl)
    in_bytes = sum(x.nbytes for x in arrays)
    st.ops, st.bytes = algorithmic(wl)
    if wl.op == "pack":
        K, N = arrays[0].shape
        out_shape, out_dtype = (N // 16, K // 2, 16, 2), np.int8
    elif wl.op == "pack_lhs":
        out_shape, out_dtype = (wl.M // 16, wl.K // 2, 16, 2), np.int8
    elif wl.op == "unpack":
        out_shape, out_dtype = (wl.M, wl.N), np.float32
    else:
        out_shape, out_dtype = (wl.M // 16, wl.N // 16, 16, 16), np.int32
    out_bytes = int(np.prod(out_shape)) * np.dtype(out_dtype).itemsize
    n_sets = set_count(in_bytes + out_bytes, 24)
    for _ in range(n_sets):
        ins = [st.to_device(x) for x in arrays]
        out = st.alloc(out_bytes)
        ws = st.track(ctx.uk_mmt4d_workspace(wl.M // 16, wl.N // 16, wl.K // 2, 16, 16, 2, rt.UK_MMT4D_S8S8S32)) \
            if wl.op == "mmt4d" else None
        st.sets.append((ins, out, ws))

    def run(ins, out, ws):
        if wl.op == "pack":
            K, N = arrays[0].shape
            ctx.uk_pack(ins[0], 0, N, 1, out, 0, (K // 2) * 32, 32, K, N, N // 16, K // 2, 16, 2, 0,
                        rt.UK_PACK_TYPE[1] | rt.UK_TRANSPOSE_INNER | rt.UK_TRANSPOSE_OUTER)
        elif wl.op == "pack_lhs":
            ctx.uk_pack(ins[0], 0, wl.K, 1, out, 0, (wl.K // 2) * 32, 32, wl.M, wl.K, wl.M // 16, wl.K // 2, 16, 2, 0,
                        rt.UK_PACK_TYPE[1])
        elif wl.op == "unpack":
            ctx.uk_unpack(ins[0], 0, (wl.N // 16) * 256, 256, out, 0, wl.N, 1, wl.M // 16, wl.N // 16, 16, 16, wl.M, wl.N,
                          rt.UK_PACK_TYPE[4])
        else:
            k1 = wl.K // 2
            ctx.uk_mmt4d(ins[0], 0, k1 * 32, ins[1], 0, k1 * 32, out, 0, (wl.N // 16) * 256, wl.M // 16, wl.N // 16, k1,
                         16, 16, 2, rt.UK_MMT4D_S8S8S32, ws)

    def step(i):
        run(*st.sets[i % n_sets])

    def check():
        for (_, _, ws) in st.sets:
            if ws is not None:
                ctx.workspace_status(ws)

    pinned = [st.pinned_copy(x) for x in arrays]
    host_out = st.pinned_empty(out_shape, out_dtype)

    def e2e_step():
        ins, out, ws = st.sets[0]
        for d, h in zip(ins, pinned):
            rt.check(lib.iree_hal_b200_transfer_h2d(ctx.device, rt._vp(h), C.c_void_p(d.ptr), C.c_size_t(h.nbytes)))
        run(ins, out, ws)
        rt.check(lib.iree_hal_b200_transfer_d2h(ctx.device, C.c_void_p(out.ptr), rt._vp(host_out), C.c_size_t(host_out.nbytes)))
        ctx.synchronize()

    st.step, st.check, st.e2e_step = step, check, e2e_step
    st.h2d, st.d2h = in_bytes, host_out.nbytes
    return st


def make_state(ctx, wl, rank, world, channel):
    if wl.family == "matmul":
        return matmul_state(ctx, wl, rank, world, channel)
    if wl.family == "tiling":
        if world > 1:
            raise SystemExit("the data-tiling workloads are single-GPU (replicas only)")
        return tiling_state(ctx, wl)
    return w4a16_state(ctx, wl, rank, world, channel)
