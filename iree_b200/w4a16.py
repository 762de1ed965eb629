"""Host-side helpers for the fused int4 dequant + matmul dispatch (``iree_b200_w4a16*``)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import runtime as rt


def w4a16_numpy(ctx: rt.Context, a: np.ndarray, wq: np.ndarray, scales: np.ndarray, group: int = 128,
                variant: int = rt.W4A16_AUTO, tile_n: int = 0, out: np.ndarray = None, n_offset: int = 0) -> np.ndarray:
    """Host arrays in, host array out, through ``iree_b200_w4a16_host``.

    a [M, K] f16; wq [N, K/2] u8 (two int4 per byte, low nibble first); scales [N, K/group] f16.
    With ``out`` given (shape [M, ldo]) the N result columns land at ``n_offset``.
    """
    a = np.ascontiguousarray(a, np.float16)
    wq = np.ascontiguousarray(wq, np.uint8)
    scales = np.ascontiguousarray(scales, np.float16)
    M, K = a.shape
    N = wq.shape[0]
    assert wq.shape == (N, K // 2) and scales.shape == (N, K // group), (wq.shape, scales.shape)
    if out is None:
        out = np.empty((M, N), np.float16)
    assert out.dtype == np.float16 and out.flags.c_contiguous and out.shape[0] == M
    p = rt.W4A16Params(M, N, K, group, out.shape[1], n_offset, variant, tile_n)
    ctx.w4a16_host(p, a, wq, scales, out)
    return out


class _BenchState:
    pass


def bench_state(ctx: rt.Context, wl, rank: int, world: int, channel, make_peer_gather=None):
    """Buffers and step functions for bench.py's W4A16 workloads.

    With more than one rank the weight rows are sharded along N; every rank computes its
    [M, N/world] slice and the slices are all-gathered through the collective channel (the
    gathered buffer holds the slices rank after rank, i.e. the transposed-block layout that an
    all-gather along the outermost dimension produces).
    """
    from . import workloads as gen
    lib = rt.library()
    st = _BenchState()
    M, K = wl.M, wl.K
    sharded = getattr(wl, "sharded", False) and world > 1
    n_local = wl.N // world if sharded else wl.N
    if wl.name.startswith("c5"):
        a, wq, s = gen.c5_w4a16_sharded(M, world if sharded else 1, rank if sharded else 0, N=wl.N, K=K)
    else:
        a, wq, s = gen.c4_w4a16(M, N=wl.N, K=K)
    set_bytes = wq.nbytes + s.nbytes + a.nbytes + M * n_local * 2
    n_sets = int(np.ceil(2.2 * 126 * 2 ** 20 / set_bytes)) if set_bytes < 2 * 126 * 2 ** 20 else 1
    n_sets = max(2, min(n_sets, 24))
    sets = []
    for _ in range(n_sets):
        da, dw, ds = ctx.to_device(a), ctx.to_device(wq), ctx.to_device(s)
        dc = ctx.alloc(M * n_local * 2)
        ws = ctx.w4a16_workspace(n_local)
        p = rt.W4A16Params(M, n_local, K, 128, n_local, 0, rt.W4A16_AUTO, 0)
        variant, tile_n = ctx.w4a16_prepare(p, da, dw, ds, dc, ws)
        sets.append((p, da, dw, ds, dc, ws, variant, tile_n))
    gathers = [ctx.alloc(world * M * n_local * 2) for _ in sets] if channel is not None else None
    peer = make_peer_gather(ctx, channel, rank, world, gathers) if make_peer_gather else None

    def step(i):
        p, da, dw, ds, dc, ws, variant, tile_n = sets[i % n_sets]
        if channel is not None and i % n_sets == 0:
            rt.check(lib.iree_hal_b200_command_buffer_join_collectives(ctx.command_buffer))
        ctx.w4a16_run(p, da, dw, ds, dc, ws, variant, tile_n)
        if peer is not None:
            peer.gather(i % n_sets, dc, M * n_local * 2)   # copy engines, beside the following dispatches
        elif channel is not None:
            # overlaps the following dispatches on the device's second stream
            rt.check(lib.iree_hal_b200_command_buffer_all_gather_overlapped(
                ctx.command_buffer, channel, C.c_int32(1), C.c_void_p(dc.ptr), C.c_void_p(gathers[i % n_sets].ptr),
                C.c_size_t(M * n_local)))

    def check():
        for x in sets:
            ctx.workspace_status(x[5])

    pa, pw, ps = ctx.pinned_copy(a), ctx.pinned_copy(wq), ctx.pinned_copy(s)
    host_out = ctx.pinned_empty((M, n_local), np.float16)

    def e2e_step():
        p = rt.W4A16Params(M, n_local, K, 128, n_local, 0, rt.W4A16_AUTO, 0)
        ctx.w4a16_host(p, pa, pw, ps, host_out)

    st.step, st.check, st.e2e_step = step, check, e2e_step
    st.gathers, st.sets, st.peer = gathers, sets, peer
    st.ops = 2.0 * M * n_local * K
    st.bytes = float(wq.nbytes + s.nbytes + a.nbytes + M * n_local * 2)
    st.h2d = a.nbytes + wq.nbytes + s.nbytes
    st.d2h = host_out.nbytes
    st.variant = sets[0][6]
    st.desc = wl.desc + ("; rank slice N/world = %d, outputs all-gathered through the channel" % n_local
                         if channel is not None else "")
    st.l2_note = "operands rotate over %d sets (%.0f MB > 126 MB L2)" % (n_sets, n_sets * set_bytes / 1e6)
    return st
