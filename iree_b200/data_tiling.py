"""Host-side helpers for the data-tiled entry points (``iree_b200_uk_pack / _unpack / _mmt4d``):
the buffers and step functions bench.py uses for them."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import runtime as rt


class _BenchState:
    pass


def operands(wl):
    """Seeded host operands of a data-tiling workload: (op, arrays...)."""
    from . import workloads as gen
    if wl.op == "pack":
        _, w, _, _ = gen.c3_w8a8(1)            # the [K, N] int8 weight matrix of the W8A8 configuration
        return (w,)
    if wl.op == "unpack":
        rng = np.random.default_rng(1)
        return (rng.standard_normal((wl.M // 16, wl.N // 16, 16, 16), dtype=np.float32),)
    # mmt4d on already-tiled int8 operands (16x16x2, the x86-64 VNNI tile)
    rng = np.random.default_rng(0)
    lhs = rng.integers(-128, 128, (wl.M // 16, wl.K // 2, 16, 2), dtype=np.int8)
    rhs = rng.integers(-127, 128, (wl.N // 16, wl.K // 2, 16, 2), dtype=np.int8)
    return lhs, rhs


def bench_state(ctx: rt.Context, wl):
    lib = rt.library()
    st = _BenchState()
    arrays = operands(wl)
    in_bytes = sum(x.nbytes for x in arrays)
    if wl.op == "pack":
        K, N = arrays[0].shape
        out_shape, out_dtype = (N // 16, K // 2, 16, 2), np.int8
        st.ops, st.bytes = 0.0, 2.0 * arrays[0].nbytes
    elif wl.op == "unpack":
        out_shape, out_dtype = (wl.M, wl.N), np.float32
        st.ops, st.bytes = 0.0, 2.0 * arrays[0].nbytes
    else:
        out_shape, out_dtype = (wl.M // 16, wl.N // 16, 16, 16), np.int32
        st.ops = 2.0 * wl.M * wl.N * wl.K
        st.bytes = float(in_bytes + wl.M * wl.N * 4)
    out_bytes = int(np.prod(out_shape)) * np.dtype(out_dtype).itemsize
    set_bytes = in_bytes + out_bytes
    n_sets = max(2, min(24, int(np.ceil(2.2 * 126 * 2 ** 20 / set_bytes))))
    sets = []
    for _ in range(n_sets):
        ins = [ctx.to_device(x) for x in arrays]
        out = ctx.alloc(out_bytes)
        ws = ctx.uk_mmt4d_workspace(wl.M // 16, wl.N // 16, wl.K // 2, 16, 16, 2, rt.UK_MMT4D_S8S8S32) \
            if wl.op == "mmt4d" else None
        sets.append((ins, out, ws))

    def run(ins, out, ws):
        if wl.op == "pack":
            K, N = arrays[0].shape
            ctx.uk_pack(ins[0], 0, N, 1, out, 0, (K // 2) * 32, 32, K, N, N // 16, K // 2, 16, 2, 0,
                        rt.UK_PACK_TYPE[1] | rt.UK_TRANSPOSE_INNER | rt.UK_TRANSPOSE_OUTER)
        elif wl.op == "unpack":
            ctx.uk_unpack(ins[0], 0, (wl.N // 16) * 256, 256, out, 0, wl.N, 1, wl.M // 16, wl.N // 16, 16, 16, wl.M, wl.N,
                          rt.UK_PACK_TYPE[4])
        else:
            k1 = wl.K // 2
            ctx.uk_mmt4d(ins[0], 0, k1 * 32, ins[1], 0, k1 * 32, out, 0, (wl.N // 16) * 256, wl.M // 16, wl.N // 16, k1,
                         16, 16, 2, rt.UK_MMT4D_S8S8S32, ws)

    def step(i):
        run(*sets[i % n_sets])

    def check():
        for (_, _, ws) in sets:
            if ws is not None:
                ctx.workspace_status(ws)

    pinned = [ctx.pinned_copy(x) for x in arrays]
    host_out = ctx.pinned_empty(out_shape, out_dtype)

    def e2e_step():
        ins, out, ws = sets[0]
        for d, h in zip(ins, pinned):
            rt.check(lib.iree_hal_b200_transfer_h2d(ctx.device, rt._vp(h), C.c_void_p(d.ptr), C.c_size_t(h.nbytes)))
        run(ins, out, ws)
        rt.check(lib.iree_hal_b200_transfer_d2h(ctx.device, C.c_void_p(out.ptr), rt._vp(host_out), C.c_size_t(host_out.nbytes)))
        ctx.synchronize()

    st.step, st.check, st.e2e_step = step, check, e2e_step
    st.h2d, st.d2h = in_bytes, host_out.nbytes
    st.desc = wl.desc
    st.l2_note = "operands rotate over %d sets (%.0f MB > 126 MB L2)" % (n_sets, n_sets * set_bytes / 1e6)
    return st
