"""Parity of the sm_100a contraction kernels with the CPU oracle, through the C ABI.

Integer results are bit-exact. Float results are exact on small-integer data and within
rtol = atol = 1e-2 (f16 out, f32 accumulate) on the benchmark distributions.
"""
import os

import numpy as np
import pytest

import iree_b200 as ib
import oracle
from iree_b200 import workloads
from iree_b200.runtime import MatmulParams, matmul_numpy

pytestmark = pytest.mark.gpu

RTOL = ATOL = 1e-2
THREADS = os.cpu_count() or 1

# tests/e2e/matmul/generate_e2e_matmul_tests.py:125-198 (small + a few large / gpu_large ones)
E2E_SHAPES = [(1, 1, 1), (9, 9, 9), (6, 13, 3), (15, 37, 7), (81, 19, 41), (1, 10, 10), (10, 1, 10), (10, 10, 1),
              (123, 456, 789), (1, 1000, 1000), (1000, 1, 1000), (512, 128, 512), (345, 456, 567)]


def oracle_matmul(t, a, b):
    """The reference's own ukernel chain when it was built, else the pinned restatement."""
    if oracle.have_ref():
        return oracle.matmul_ref(t, a, b, threads=THREADS)
    return oracle.matmul_port(t, a, b)


def small_ints(rng, kind, shape):
    if kind == ib.KIND_I8:
        return rng.integers(-128, 128, shape, dtype=np.int8)
    x = rng.integers(-4, 5, shape).astype(np.float32)
    if kind == ib.KIND_BF16:
        return (x.view(np.uint32) >> 16).astype(np.uint16)
    return x.astype(np.float16)


def as_f64(x, kind):
    if kind == ib.KIND_BF16 and x.dtype == np.uint16:
        return (x.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    return x.astype(np.float64)


@pytest.mark.parametrize("kind,epi", [(ib.KIND_F16, ib.EPILOGUE_CAST), (ib.KIND_F16, ib.EPILOGUE_ACCUMULATOR),
                                      (ib.KIND_BF16, ib.EPILOGUE_CAST), (ib.KIND_I8, ib.EPILOGUE_ACCUMULATOR)])
@pytest.mark.parametrize("layout", [ib.RHS_KN, ib.RHS_NK])
def test_e2e_shape_set_exact(ctx, kind, epi, layout):
    """Every shape of the reference's e2e matmul suites, whichever kernel it routes to (TMA +
    tcgen05 when pitches are 16-byte multiples, the SIMT kernel otherwise). Small-integer data,
    so results are exact for floats as well (iree-e2e-matmul-test.cc:28-131 policy)."""
    rng = np.random.default_rng(1)
    for (M, K, N) in E2E_SHAPES:
        a = small_ints(rng, kind, (M, K))
        b = small_ints(rng, kind, (K, N) if layout == ib.RHS_KN else (N, K))
        got = matmul_numpy(ctx, kind, epi, a, b, layout)
        bb = as_f64(b, kind) if layout == ib.RHS_KN else as_f64(b, kind).T
        want = as_f64(a, kind) @ bb                       # exact: integers well inside f32
        if epi == ib.EPILOGUE_CAST:                       # the truncf consumer rounds once
            want = as_f64(oracle.truncf(want.astype(np.float32), to_bf16=(kind == ib.KIND_BF16)), kind)
        assert (as_f64(got, kind) == want).all(), (M, K, N)


@pytest.mark.parametrize("kind", [ib.KIND_F16, ib.KIND_I8])
@pytest.mark.parametrize("layout", [ib.RHS_KN, ib.RHS_NK])
@pytest.mark.parametrize("tile_n", [0, 128, 256])
def test_tensor_core_path_tiles_and_ragged_edges(ctx, kind, layout, tile_n):
    rng = np.random.default_rng(2)
    epi = ib.EPILOGUE_ACCUMULATOR
    for (M, N, K) in [(128, 256, 128), (129, 384, 1040), (300, 528, 272), (1, 256, 4096), (640, 1280, 64)]:
        a = small_ints(rng, kind, (M, K))
        b = small_ints(rng, kind, (K, N) if layout == ib.RHS_KN else (N, K))
        got = matmul_numpy(ctx, kind, epi, a, b, layout, tile_n=tile_n)
        bb = as_f64(b, kind) if layout == ib.RHS_KN else as_f64(b, kind).T
        assert (got.astype(np.float64) == as_f64(a, kind) @ bb).all(), (M, N, K)


def test_generic_and_tensor_core_kernels_agree(ctx):
    rng = np.random.default_rng(3)
    a = small_ints(rng, ib.KIND_F16, (3, 200, 136))
    b = small_ints(rng, ib.KIND_F16, (3, 136, 264))
    fast = matmul_numpy(ctx, ib.KIND_F16, ib.EPILOGUE_CAST, a, b)
    slow = matmul_numpy(ctx, ib.KIND_F16, ib.EPILOGUE_CAST, a, b, flags=ib.FLAG_FORCE_GENERIC)
    assert (fast == slow).all()


def test_empty_dimensions(ctx):
    for (M, N, K) in [(0, 8, 8), (8, 0, 8)]:
        out = matmul_numpy(ctx, ib.KIND_F16, ib.EPILOGUE_CAST, np.zeros((M, K), np.float16), np.zeros((K, N), np.float16))
        assert out.shape == (M, N)
    out = matmul_numpy(ctx, ib.KIND_I8, ib.EPILOGUE_ACCUMULATOR, np.zeros((4, 0), np.int8), np.zeros((0, 5), np.int8))
    assert (out == 0).all()   # K = 0: the fill value


def test_c1_i8_matmul_bit_exact(ctx):
    a, b = workloads.c1_i8_matmul()
    got = matmul_numpy(ctx, ib.KIND_I8, ib.EPILOGUE_ACCUMULATOR, a, b)
    want = oracle_matmul(oracle.TYPE_S8S8S32, a, b)
    assert got.dtype == np.int32 and (got == want).all()


def test_c2_f16_matmul(ctx):
    a, b = workloads.c2_f16_matmul()
    got = matmul_numpy(ctx, ib.KIND_F16, ib.EPILOGUE_CAST, a, b)
    if oracle.have_ref():
        want = oracle.truncf(oracle.matmul_ref(oracle.TYPE_F16F16F32, a, b, threads=THREADS))
        np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32), rtol=RTOL, atol=ATOL)
    else:  # a strided subset of rows through the scalar restatement
        rows = np.arange(0, a.shape[0], 97)
        want = oracle.truncf(oracle.matmul_port(oracle.TYPE_F16F16F32, a[rows], b))
        np.testing.assert_allclose(got[rows].astype(np.float32), want.astype(np.float32), rtol=RTOL, atol=ATOL)


def test_c2_f16_batch_matmul(ctx):
    a, b = workloads.c2_f16_batch_matmul()
    got = matmul_numpy(ctx, ib.KIND_F16, ib.EPILOGUE_CAST, a, b)
    for i in range(a.shape[0]):
        want = oracle.truncf(oracle_matmul(oracle.TYPE_F16F16F32, a[i], b[i]))
        np.testing.assert_allclose(got[i].astype(np.float32), want.astype(np.float32), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("M", [1, 16, 512, 4096])
def test_c3_w8a8_requant(ctx, M):
    a, w, sa, sw = workloads.c3_w8a8(M)
    got = matmul_numpy(ctx, ib.KIND_I8, ib.EPILOGUE_REQUANT_F16, a, w, row_scale=sa, col_scale=sw)
    acc = matmul_numpy(ctx, ib.KIND_I8, ib.EPILOGUE_ACCUMULATOR, a, w)
    want_acc = oracle_matmul(oracle.TYPE_S8S8S32, a, w)
    assert (acc == want_acc).all()                       # i32 accumulator: bit-exact
    want = oracle.requant_f16(want_acc, sa, sw)
    np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32), rtol=RTOL, atol=ATOL)
    assert (got == want).all()                           # same operation order: identical in fact


@pytest.mark.parametrize("splits", [0, 2, 3, 5, 15])
def test_few_rows_products_with_their_k_range_split_over_ctas(ctx, splits):
    """Few-rows products whose tiles' K ranges are cut into work items (partial accumulators met through
    the workspace, last arriver applies the epilogue): i32 results bit-exact and the requant output
    identical to the unsplit kernel's, f16 exact on small integers, ragged N and K, both right-hand
    side layouts, a batch, and twice through the same workspace (the counters come back to zero)."""
    from iree_b200 import runtime as rt
    rng = np.random.default_rng(90 + splits)
    flags = rt.FLAG_SPLIT_K | (splits << 8)
    cases = [(ib.KIND_I8, ib.EPILOGUE_ACCUMULATOR, ib.RHS_KN, 16, 1280, 4096, 1),
             (ib.KIND_I8, ib.EPILOGUE_REQUANT_F16, ib.RHS_KN, 1, 11008, 4096, 1),
             (ib.KIND_I8, ib.EPILOGUE_ACCUMULATOR, ib.RHS_NK, 7, 200, 2064, 1),
             (ib.KIND_F16, ib.EPILOGUE_CAST, ib.RHS_KN, 32, 264, 1096, 1),
             (ib.KIND_F16, ib.EPILOGUE_ACCUMULATOR, ib.RHS_NK, 5, 96, 2048, 3)]
    for kind, epi, layout, M, N, K, B in cases:
        a = small_ints(rng, kind, (B, M, K))
        b = small_ints(rng, kind, (B, K, N) if layout == ib.RHS_KN else (B, N, K))
        if kind == ib.KIND_F16:
            a, b = (a / 4).astype(np.float16), (b / 4).astype(np.float16)      # keeps |result| exact in f16
        sa = rng.uniform(0.5, 1.5, M).astype(np.float32) / 64
        sw = rng.uniform(0.5, 1.5, N).astype(np.float32) / 64
        requant = epi == ib.EPILOGUE_REQUANT_F16
        da, db = ctx.to_device(a), ctx.to_device(b)
        odt = rt.out_dtype(kind, epi)
        dc = ctx.alloc(B * M * N * np.dtype(odt).itemsize)
        rs, cs = (ctx.to_device(sa), ctx.to_device(sw)) if requant else (None, None)
        p = MatmulParams(kind, epi, M, N, K, B, layout, 0, flags)
        ws = ctx.matmul_workspace(p)
        tile_n = ctx.matmul_prepare(p, da, db, ws)
        if splits:
            assert (tile_n >> 16) + 1 == min(splits, -(-K // (128 if kind == ib.KIND_I8 else 64)))
        t = {ib.KIND_I8: oracle.TYPE_S8S8S32, ib.KIND_F16: oracle.TYPE_F16F16F32}[kind]
        for round_ in range(2):
            dc.fill(0x55)
            ctx.matmul_run(p, da, db, dc, ws, tile_n, rs, cs)
            ctx.workspace_status(ws)
            got = dc.download(odt, (B, M, N))
            for i in range(B):
                bi = b[i] if layout == ib.RHS_KN else np.ascontiguousarray(b[i].T)
                acc = oracle_matmul(t, a[i], bi)
                want = oracle.requant_f16(acc, sa, sw) if requant else (oracle.truncf(acc) if epi == ib.EPILOGUE_CAST else acc)
                assert (got[i] == want).all(), (kind, epi, layout, M, N, K, i, round_, splits, tile_n >> 16)
        for x in (da, db, dc, ws) + ((rs, cs) if requant else ()):
            x.free()


def test_int8_linearity_at_full_size(ctx):
    """Size-independent property on the largest i8 configuration: C(A, B1 + B2) = C(A,B1) + C(A,B2)."""
    rng = np.random.default_rng(5)
    M, N, K = 4096, 11008, 4096
    a = rng.integers(-128, 128, (M, K), dtype=np.int8)
    b1 = rng.integers(-60, 60, (K, N), dtype=np.int8)
    b2 = rng.integers(-60, 60, (K, N), dtype=np.int8)
    c1 = matmul_numpy(ctx, ib.KIND_I8, ib.EPILOGUE_ACCUMULATOR, a, b1)
    c2 = matmul_numpy(ctx, ib.KIND_I8, ib.EPILOGUE_ACCUMULATOR, a, b2)
    c12 = matmul_numpy(ctx, ib.KIND_I8, ib.EPILOGUE_ACCUMULATOR, a, (b1 + b2).astype(np.int8))
    assert (c12 == c1 + c2).all()


def test_every_output_element_is_written(ctx):
    M, N, K = 200, 264, 128
    rng = np.random.default_rng(6)
    a = small_ints(rng, ib.KIND_F16, (M, K))
    b = small_ints(rng, ib.KIND_F16, (K, N))
    da, db = ctx.to_device(a), ctx.to_device(b)
    dc = ctx.alloc((M * N + 64) * 2).fill(0x7E)            # poison, with a guard band after the result
    ws = ctx.workspace()
    ctx.matmul(MatmulParams(ib.KIND_F16, ib.EPILOGUE_CAST, M, N, K, 1, ib.RHS_KN, 0, 0), da, db, dc, ws)
    ctx.workspace_status(ws)
    out = dc.download(np.uint16, (M * N + 64,))
    assert (out[M * N:] == 0x7E7E).all()                   # nothing past the end
    assert (out[:M * N].view(np.float16).reshape(M, N).astype(np.float64) == a.astype(np.float64) @ b.astype(np.float64)).all()
    for x in (da, db, dc, ws):
        x.free()


@pytest.mark.parametrize("kind", [ib.KIND_F16, ib.KIND_BF16, ib.KIND_I8])
@pytest.mark.parametrize("layout", [ib.RHS_KN, ib.RHS_NK])
def test_device_built_tensor_maps_equal_host_encoded(ctx, kind, layout):
    """b200_encode_tensormaps (the route for a runtime that never calls cuTensorMapEncodeTiled)
    must produce the bytes cuTensorMapEncodeTiled produces, and a matmul through them must work."""
    es = 1 if kind == ib.KIND_I8 else 2
    rng = np.random.default_rng(7)
    for (M, N, K, B, bn) in [(256, 384, 512, 1, 128), (130, 256, 1024, 3, 256), (4096, 4096, 4096, 1, 256)]:
        if M * N > 1 << 22:
            a = ctx.alloc(B * M * K * es); b = ctx.alloc(B * K * N * es)
        else:
            ah = small_ints(rng, kind, (B, M, K)); bh = small_ints(rng, kind, (B, K, N) if layout == ib.RHS_KN else (B, N, K))
            a, b = ctx.to_device(ah), ctx.to_device(bh)
        ws_h, ws_d = ctx.workspace(), ctx.workspace()
        p = MatmulParams(kind, ib.EPILOGUE_ACCUMULATOR, M, N, K, B, layout, bn, 0)
        bn_h = ctx.matmul_prepare(p, a, b, ws_h)
        p.flags = ib.FLAG_DEVICE_TENSORMAPS
        bn_d = ctx.matmul_prepare(p, a, b, ws_d)
        assert bn_h == bn_d == bn
        mh, md = ws_h.download(np.uint8, (256,)), ws_d.download(np.uint8, (256,))
        assert (mh == md).all(), (M, N, K, B, np.nonzero(mh != md)[0])
        if M * N <= 1 << 22:
            c = ctx.alloc(B * M * N * 4)
            ctx.matmul_run(p, a, b, c, ws_d, bn_d)
            ctx.workspace_status(ws_d)
            got = c.download(np.int32 if kind == ib.KIND_I8 else np.float32, (B, M, N))
            bb = as_f64(bh, kind) if layout == ib.RHS_KN else np.swapaxes(as_f64(bh, kind), -1, -2)
            assert (got.astype(np.float64) == as_f64(ah, kind) @ bb).all()
            c.free()
        for x in (a, b, ws_h, ws_d):
            x.free()


def test_bounded_wait_reports_deadline_and_context_survives(ctx):
    ws = ctx.workspace()
    ctx.dispatch("b200_selftest_wait_timeout", [ws], [20000], (1, 1, 1))   # 20 ms limit, nothing arrives
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.workspace_status(ws)
    assert e.value.code_name == "DEADLINE_EXCEEDED"
    # the context still works
    a = np.ones((8, 8), np.float16)
    assert (matmul_numpy(ctx, ib.KIND_F16, ib.EPILOGUE_CAST, a, a) == 8).all()
    ws.free()


def test_kernel_refuses_unaligned_tile_width(ctx):
    """A tile width the MMA cannot take is refused by the kernel itself (status word), not run."""
    a = ctx.alloc(128 * 64 * 2).fill(0); b = ctx.alloc(64 * 128 * 2).fill(0); c = ctx.alloc(128 * 128 * 2)
    ws = ctx.workspace()
    p = MatmulParams(ib.KIND_F16, ib.EPILOGUE_CAST, 128, 128, 64, 1, ib.RHS_NK, 0, 0)
    bn = ctx.matmul_prepare(p, a, b, ws)
    ctx.dispatch("b200_matmul_f16_f16", [c, ws], [128, 128, 64, 1, ib.RHS_NK, 48], (1, 1, 1))
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.workspace_status(ws)
    assert e.value.code_name == "INVALID_ARGUMENT" and bn
    for x in (a, b, c, ws):
        x.free()


def test_api_argument_errors(ctx):
    p = MatmulParams(ib.KIND_F16, ib.EPILOGUE_REQUANT_F16, 8, 8, 8, 1, ib.RHS_KN, 0, 0)
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.matmul_host(p, np.zeros((8, 8), np.float16), np.zeros((8, 8), np.float16), np.zeros((8, 8), np.float16))
    assert e.value.code_name == "UNIMPLEMENTED"           # requant is an i8 epilogue
    p = MatmulParams(ib.KIND_I8, ib.EPILOGUE_REQUANT_F16, 8, 8, 8, 1, ib.RHS_KN, 0, 0)
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.matmul_host(p, np.zeros((8, 8), np.int8), np.zeros((8, 8), np.int8), np.zeros((8, 8), np.float16))
    assert e.value.code_name == "INVALID_ARGUMENT"        # scales missing
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.dispatch("no_such_export", [], [], (1, 1, 1))
    assert e.value.code_name == "NOT_FOUND"


def test_graph_mode_replays_recorded_dispatches(ctx):
    """Graph command-buffer mode: dispatches recorded between begin_graph / end_graph run only
    when the graph executes, in order, and give the stream-mode result."""
    rng = np.random.default_rng(8)
    M, N, K = 256, 384, 512
    a = small_ints(rng, ib.KIND_F16, (M, K)); b = small_ints(rng, ib.KIND_F16, (K, N))
    da, db = ctx.to_device(a), ctx.to_device(b)
    c1, c2 = ctx.alloc(M * N * 2).fill(0), ctx.alloc(M * N * 2).fill(0)
    ws = ctx.workspace()
    p = MatmulParams(ib.KIND_F16, ib.EPILOGUE_CAST, M, N, K, 1, ib.RHS_KN, 0, 0)
    bn = ctx.matmul_prepare(p, da, db, ws)
    before = ctx.launch_count
    ctx.begin_graph()
    ctx.matmul_run(p, da, db, c1, ws, bn)
    with pytest.raises(ib.IreeB200Error) as e:                # a host-buffer call copies and waits: not recordable
        ctx.matmul_host(p, a, b, np.empty((M, N), np.float16))
    assert e.value.code_name == "FAILED_PRECONDITION"
    ctx.matmul_run(p, da, db, c2, ws, bn)
    graph = ctx.end_graph()
    ctx.synchronize()
    assert not c1.download(np.uint16, (M, N)).any()          # recorded, not executed
    assert ctx.launch_count == before
    graph.execute()
    ctx.workspace_status(ws)
    want = (a.astype(np.float64) @ b.astype(np.float64))
    for c in (c1, c2):
        assert (c.download(np.float16, (M, N)).astype(np.float64) == want).all()
    assert ctx.launch_count == before + 2
    graph.release()
    for x in (da, db, c1, c2, ws):
        x.free()


@pytest.mark.parametrize("M,graph", [(128, False), (512, True), (16, True), (300, False)])
def test_overlapped_matmul_chain_equals_the_serial_chain(ctx, M, graph):
    """A chain of f16 matmuls in which every step's left operand is the previous step's result
    (N = K), dispatched with overlap (programmatic dependent launch; stream mode and graph mode): a
    kernel may be launched, and set up its barriers and tensor memory, before the one ahead has
    finished, but must not read an operand early. The results are bit-identical to the serial
    chain (1-CTA kernel, its few-rows variant and the CTA-pair kernel)."""
    from iree_b200 import runtime as rt
    rng = np.random.default_rng(77 + M)
    N = K = 1024
    steps = 10
    a0 = (rng.standard_normal((M, K)) * 0.5).astype(np.float16)
    rhs = [ctx.to_device((rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16)) for _ in range(3)]
    bufs = [ctx.to_device(a0), ctx.alloc(M * N * 2), ctx.alloc(M * N * 2)]
    p = MatmulParams(ib.KIND_F16, ib.EPILOGUE_CAST, M, N, K, 1, ib.RHS_KN, 0, 0)
    # one workspace (its maps name the operands) per (source, right-hand side) pair in use
    prepared = {}

    def chain():
        bufs[0].upload(a0)
        if graph:
            ctx.begin_graph()
        src = 0
        for i in range(steps):
            dst = 1 + (i % 2)
            key = (src, i % 3)
            if key not in prepared:
                ws = ctx.matmul_workspace(p)
                prepared[key] = (ws, ctx.matmul_prepare(p, bufs[src], rhs[i % 3], ws))
            ws, bn = prepared[key]
            ctx.matmul_run(p, bufs[src], rhs[i % 3], bufs[dst], ws, bn)
            src = dst
        if graph:
            g = ctx.end_graph()
            g.execute()
            ctx.synchronize()
            g.release()
        for ws, _ in prepared.values():
            ctx.workspace_status(ws)
        return bufs[src].download(np.float16, (M, N))

    chain()                       # every workspace is prepared outside a recording
    serial = chain()
    ctx.set_dispatch_overlap(True)
    try:
        overlapped = chain()
    finally:
        ctx.set_dispatch_overlap(False)
    assert np.isfinite(serial.astype(np.float32)).all() and np.abs(serial.astype(np.float32)).max() > 1e-3
    assert np.array_equal(serial.view(np.uint16), overlapped.view(np.uint16))
    for b in bufs + rhs + [ws for ws, _ in prepared.values()]:
        b.free()
