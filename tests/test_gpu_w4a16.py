"""Parity of the fused int4 dequant + matmul kernels with the CPU oracle, through the C ABI.
Tolerance rtol = atol = 1e-2 (f16 out, f32 accumulate); the nibble order and group indexing
are additionally checked exactly on small-integer data."""
import numpy as np
import pytest

import iree_b200 as ib
import oracle
from iree_b200 import workloads
from iree_b200.w4a16 import w4a16_numpy

pytestmark = pytest.mark.gpu
RTOL = ATOL = 1e-2
import os
THREADS = os.cpu_count() or 1


def exact_case(rng, M, N, K, group=128):
    """Integer activations, power-of-two scales: every product and partial sum is exact in f32
    and every result fits f16, so all kernels must agree bit for bit with the oracle."""
    a = rng.integers(-2, 3, (M, K)).astype(np.float16)
    wq = workloads.pack_int4(rng.integers(-8, 8, (N, K), dtype=np.int8))
    s = (2.0 ** rng.integers(-3, 1, (N, K // group))).astype(np.float16)
    return a, wq, s


@pytest.mark.parametrize("variant", [ib.W4A16_GENERIC, ib.W4A16_DECODE, ib.W4A16_GEMM])
def test_exact_on_integer_data(ctx, variant):
    rng = np.random.default_rng(21)
    shapes = [(1, 16, 256), (8, 64, 512), (16, 256, 4096), (3, 48, 1024), (16, 32, 8192)]
    if variant == ib.W4A16_GEMM:
        shapes += [(128, 256, 256), (200, 384, 1024), (130, 264, 128)]
    if variant == ib.W4A16_GENERIC:
        shapes += [(5, 7, 128), (2, 33, 384)]
    for (M, N, K) in shapes:
        a, wq, s = exact_case(rng, M, N, K)
        got = w4a16_numpy(ctx, a, wq, s, variant=variant)
        want = oracle.w4a16(a, wq, s, threads=THREADS)
        assert (got == want).all(), (variant, M, N, K, np.abs(got.astype(np.float32) - want.astype(np.float32)).max())


def test_weights_in_tensor_memory_variant(ctx):
    """The many-rows kernel (weights as the tensor-memory operand, results by TMA stores): exact on
    integer data over ragged M and N, several tiles per CTA, column slices of a wider result, and
    equal to the shared-memory-operand kernel on the same inputs."""
    rng = np.random.default_rng(61)
    for (M, N, K) in [(256, 128, 128), (300, 264, 256), (520, 151 * 16, 384), (1024, 384, 1024), (257, 8, 128),
                      (128, 256, 512), (100, 264, 256), (17, 128, 1024), (129, 136, 128)]:
        a, wq, s = exact_case(rng, M, N, K)
        got = w4a16_numpy(ctx, a, wq, s, variant=ib.W4A16_GEMM_WT)
        want = oracle.w4a16(a, wq, s, threads=THREADS)
        assert (got == want).all(), (M, N, K, np.abs(got.astype(np.float32) - want.astype(np.float32)).max())
    # a column slice: neighbours of the slice must survive, also next to a ragged last tile
    M, N, K, ldo, off = 384, 200, 256, 512, 72
    a, wq, s = exact_case(rng, M, N, K)
    out = np.full((M, ldo), 7.0, np.float16)
    w4a16_numpy(ctx, a, wq, s, variant=ib.W4A16_GEMM_WT, out=out, n_offset=off)
    assert (out[:, off:off + N] == oracle.w4a16(a, wq, s, threads=THREADS)).all()
    assert (out[:, :off] == 7.0).all() and (out[:, off + N:] == 7.0).all()
    # real-valued data: same dequantised weights as the other tensor-core kernel, f32 accumulation
    a, wq, s = workloads.c4_w4a16(512, N=1024, K=2048, seed=62)
    wt = w4a16_numpy(ctx, a, wq, s, variant=ib.W4A16_GEMM_WT)
    ss = w4a16_numpy(ctx, a, wq, s, variant=ib.W4A16_GEMM)
    np.testing.assert_allclose(wt.astype(np.float32), ss.astype(np.float32), rtol=2e-3, atol=2e-3)
    np.testing.assert_allclose(wt.astype(np.float32), oracle.w4a16(a, wq, s, threads=THREADS).astype(np.float32),
                               rtol=RTOL, atol=ATOL)


def test_tensor_core_decode_variant(ctx):
    """The few-rows kernel on the tensor cores: exact on integer data over every M it takes, ragged
    N (tiles of 128 weight rows), K from one unit to several tiles' worth, shapes whose units
    divide evenly among the CTAs and shapes whose ranges start and end inside a tile (partial sums
    met through the workspace), twice through the same workspace; then real-valued data."""
    rng = np.random.default_rng(71)
    shapes = [(1, 128, 256), (16, 128, 256), (8, 64, 512), (3, 200, 1024), (16, 1000, 768), (16, 19 * 128, 8192),
              (5, 150 * 128, 512), (16, 149 * 128 + 8, 4096), (13, 8, 16384), (16, 2048, 2048)]
    for (M, N, K) in shapes:
        a, wq, s = exact_case(rng, M, N, K)
        want = oracle.w4a16(a, wq, s, threads=THREADS)
        da, dw, ds = ctx.to_device(a), ctx.to_device(wq), ctx.to_device(s)
        dc, ws = ctx.alloc(M * N * 2), ctx.w4a16_workspace(N)
        p = ib.W4A16Params(M, N, K, 128, N, 0, ib.W4A16_DECODE_TC, 0)
        variant, tile_n = ctx.w4a16_prepare(p, da, dw, ds, dc, ws)
        assert variant == ib.W4A16_DECODE_TC
        for round_ in range(2):
            dc.upload(np.full((M, N), 9.0, np.float16))
            ctx.w4a16_run(p, da, dw, ds, dc, ws, variant, tile_n)
            ctx.workspace_status(ws)
            got = dc.download(np.float16, (M, N))
            assert (got == want).all(), (M, N, K, round_, np.abs(got.astype(np.float32) - want.astype(np.float32)).max())
        for b in (da, dw, ds, dc, ws):
            b.free()
    # a column slice of a wider result
    M, N, K, ldo, off = 7, 200, 512, 512, 72
    a, wq, s = exact_case(rng, M, N, K)
    out = np.full((M, ldo), 7.0, np.float16)
    w4a16_numpy(ctx, a, wq, s, variant=ib.W4A16_DECODE_TC, out=out, n_offset=off)
    assert (out[:, off:off + N] == oracle.w4a16(a, wq, s, threads=THREADS)).all()
    assert (out[:, :off] == 7.0).all() and (out[:, off + N:] == 7.0).all()
    # real-valued data: the dequantised weights are the reference's, the accumulation is f32
    for M in (1, 16):
        a, wq, s = workloads.c4_w4a16(M, N=1536, K=4096, seed=72)
        got = w4a16_numpy(ctx, a, wq, s, variant=ib.W4A16_DECODE_TC)
        np.testing.assert_allclose(got.astype(np.float32), oracle.w4a16(a, wq, s, threads=THREADS).astype(np.float32),
                                   rtol=RTOL, atol=ATOL)
    # a workspace that was never prepared is refused by the kernel, not run through an empty tensor map
    a, wq, s = exact_case(rng, 4, 256, 512)
    da, dw, ds = ctx.to_device(a), ctx.to_device(wq), ctx.to_device(s)
    dc, ws = ctx.alloc(4 * 256 * 2), ctx.w4a16_workspace(256)
    ctx.w4a16_run(ib.W4A16Params(4, 256, 512, 128, 256, 0, ib.W4A16_DECODE_TC, 0), da, dw, ds, dc, ws, ib.W4A16_DECODE_TC, 0)
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.workspace_status(ws)
    assert e.value.code_name == "INVALID_ARGUMENT"
    for b in (da, dw, ds, dc, ws):
        b.free()


def test_pushing_dispatch_with_one_rank(ctx):
    """The N-sharded form with a channel of one: the kernel stores into the (only) destination,
    raises its arrival word, and the wait kernel sees it; a wait for a word nobody raises runs out
    and is reported as DEADLINE_EXCEEDED with the context still usable."""
    rng = np.random.default_rng(63)
    M, N, K = 512, 256, 256
    a, wq, s = exact_case(rng, M, N, K)
    da, dw, ds = ctx.to_device(a), ctx.to_device(wq), ctx.to_device(s)
    result, flags, ws = ctx.alloc(M * N * 2).fill(0x7E), ctx.alloc(256).fill(0), ctx.w4a16_workspace(N)
    p = ib.W4A16Params(M, N, K, 128, N, 0, ib.W4A16_GEMM_WT, 0)
    ctx.w4a16_prepare_push(p, da, dw, ds, [result], [flags], 0, ws)
    want = oracle.w4a16(a, wq, s, threads=THREADS)
    for epoch in (1, 2, 3):
        result.fill(0x7E)
        ctx.w4a16_run_push(p, ds, result, ws, 1, 0, epoch)
        ctx.w4a16_wait_arrivals(flags, ws, 1, epoch)
        ctx.workspace_status(ws)
        assert (result.download(np.float16, (M, N)) == want).all()
        assert flags.download(np.uint32, (1,))[0] == epoch
    ctx.w4a16_wait_arrivals(flags, ws, 1, 9)          # nothing will ever raise the word to 9
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.workspace_status(ws)
    assert e.value.code_name == "DEADLINE_EXCEEDED"
    ws.fill(0)
    ctx.w4a16_prepare_push(p, da, dw, ds, [result], [flags], 0, ws)
    ctx.w4a16_run_push(p, ds, result, ws, 1, 0, 4)
    ctx.w4a16_wait_arrivals(flags, ws, 1, 4)
    ctx.workspace_status(ws)
    for x in (da, dw, ds, result, flags, ws):
        x.free()


@pytest.mark.parametrize("tile_n", [16, 48, 80, 112, 128])
def test_tensor_core_tile_widths(ctx, tile_n):
    """Every tile width the tensor-core kernel accepts (multiples of 16 up to 128), on shapes with
    ragged edges in M and N, for the 128-row and the 256-row variant and several tiles per CTA."""
    rng = np.random.default_rng(40 + tile_n)
    for (M, N, K) in [(40, 3 * tile_n + 8, 384), (300, 2 * tile_n + 24, 256), (520, 151 * 16, 128)]:
        a, wq, s = exact_case(rng, M, N, K)
        got = w4a16_numpy(ctx, a, wq, s, variant=ib.W4A16_GEMM, tile_n=tile_n)
        want = oracle.w4a16(a, wq, s, threads=THREADS)
        assert (got == want).all(), (tile_n, M, N, K)


def test_generic_other_group_sizes(ctx):
    rng = np.random.default_rng(22)
    for group in (32, 64, 256):
        a, wq, s = exact_case(rng, 3, 40, 512, group)
        got = w4a16_numpy(ctx, a, wq, s, group=group)
        assert (got == oracle.w4a16(a, wq, s, group=group)).all(), group


@pytest.mark.parametrize("M", [1, 8, 16, 128, 2048])
def test_c4_w4a16(ctx, M):
    a, wq, s = workloads.c4_w4a16(M)
    got = w4a16_numpy(ctx, a, wq, s)
    if M <= 128:
        want = oracle.w4a16(a, wq, s, threads=THREADS)
        np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32), rtol=RTOL, atol=ATOL)
    else:  # a strided subset of rows keeps the CPU side to seconds
        rows = np.arange(0, M, 61)
        want = oracle.w4a16(a[rows], wq, s, threads=THREADS)
        np.testing.assert_allclose(got[rows].astype(np.float32), want.astype(np.float32), rtol=RTOL, atol=ATOL)


def test_host_call_in_units_equals_the_single_dispatch(ctx):
    """A many-rows product of tens of megabytes goes through the host-buffer call as units (growing
    rectangles of the result, computed as blocks of activation rows and of weight rows arrive), uploads and
    dispatches overlapping, the rectangles returning by pitched copies into a pageable or a page-locked
    result. Ragged row and column blocks; either way the result must equal, bit for bit, what the one
    dispatch of the same kernel leaves, and the oracle on a sample."""
    rng = np.random.default_rng(77)
    M, N, K = 1100, 4400, 12288
    a, wq, s = exact_case(rng, M, N, K)
    one = w4a16_numpy(ctx, a, wq, s, variant=ib.W4A16_GEMM_WT)           # explicit variant: one dispatch
    rows, cols = np.arange(0, M, 97), np.arange(0, N, 53)
    assert (one[np.ix_(rows, cols)] == oracle.w4a16(a[rows], wq[cols], s[cols], threads=THREADS)).all()
    pageable = np.full((M, N), 7.0, np.float16)
    w4a16_numpy(ctx, a, wq, s, out=pageable)                             # AUTO: in units
    assert (pageable == one).all(), np.argwhere(pageable != one)[:4]
    locked = ctx.pinned_empty((M, N), np.float16)
    try:
        locked[...] = 7.0
        w4a16_numpy(ctx, a, wq, s, out=locked)
        assert (locked == one).all(), np.argwhere(locked != one)[:4]
    finally:
        ib.runtime.library().iree_hal_b200_host_free(ctx.device, ib.runtime._vp(locked))


@pytest.mark.parametrize("M", [16, 4096])
def test_c5_w4a16_70b_shape(ctx, M):
    a, wq, s = workloads.c5_w4a16_sharded(M)
    got = w4a16_numpy(ctx, a, wq, s)
    if M <= 128:   # every output: 16 x 28672 dot products of length 8192 are seconds on the host cores
        want = oracle.w4a16(a, wq, s, threads=THREADS)
        np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32), rtol=RTOL, atol=ATOL)
        return
    cols = np.arange(0, wq.shape[0], 37)
    rows = np.arange(0, M, 257)
    want = oracle.w4a16(a[rows], wq[cols], s[cols], threads=THREADS)
    np.testing.assert_allclose(got[np.ix_(rows, cols)].astype(np.float32), want.astype(np.float32), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("variant", [ib.W4A16_DECODE, ib.W4A16_GEMM, ib.W4A16_DECODE_TC])
def test_distance_from_the_restated_dequant_is_measured(ctx, variant):
    """Data on which the rounding of f16(w * s) matters: integer activations (so every product
    a * w and every group sum is exact) and scales that are not powers of two. The restated
    dispatch rounds each dequantised weight to f16 before the contraction. The tensor-core kernels
    do the same and may differ from the oracle only through f32 summation order: at most one
    f16 unit in the last place of the result. The decode kernel multiplies the exact f32 group
    sum by the scale instead, so it differs from the oracle by the weights' rounding error, at
    most 2^-11 relative per weight: |got - oracle| <= 2^-11 * sum_k |a_k| |w_k s| plus the
    output's own rounding. Both bounds are asserted and the decode kernel must agree with the
    exactly scaled result to f32 accuracy."""
    rng = np.random.default_rng(77)
    M, N, K = 16, 256, 4096
    a = rng.integers(-2, 3, (M, K)).astype(np.float16)
    w = rng.integers(-8, 8, (N, K), dtype=np.int8)
    wq = workloads.pack_int4(w)
    s = rng.uniform(0.005, 0.05, (N, K // 128)).astype(np.float16)
    got = w4a16_numpy(ctx, a, wq, s, variant=variant).astype(np.float64)
    want = oracle.w4a16(a, wq, s, threads=THREADS).astype(np.float64)
    s_full = np.repeat(s.astype(np.float64), 128, axis=1)                      # [N, K]
    exact_scaled = a.astype(np.float64) @ (w.astype(np.float64) * s_full).T    # scale applied exactly
    magnitude = np.abs(a.astype(np.float64)) @ (np.abs(w.astype(np.float64)) * s_full).T
    ulp = np.spacing(np.abs(want).astype(np.float16)).astype(np.float64)
    if variant in (ib.W4A16_GEMM, ib.W4A16_DECODE_TC):    # the tensor-core kernels: exact dequant
        assert (np.abs(got - want) <= ulp).all()
        return
    bound = 2.0 ** -11 * magnitude + ulp
    assert (np.abs(got - want) <= bound).all(), (np.abs(got - want) / bound).max()
    # and it is the exactly scaled sum, rounded once to f16
    assert (np.abs(got - exact_scaled) <= 0.5 * ulp + 1e-5 * magnitude).all()
    assert (got != want).any()            # the data does exercise the difference


@pytest.mark.parametrize("M", [8, 256])
def test_sharded_slices_assemble_the_full_result(ctx, M):
    """N-sharding as the multi-GPU path does it: each rank's slice written at its column offset
    of the full-width buffer equals the unsharded result."""
    a, wq, s = workloads.c4_w4a16(M, N=1024, K=1024, seed=9)
    full = w4a16_numpy(ctx, a, wq, s)
    world = 4
    out = np.zeros((M, 1024), np.float16)
    for r in range(world):
        n0, n1 = r * 256, (r + 1) * 256
        w4a16_numpy(ctx, a, wq[n0:n1], s[n0:n1], out=out, n_offset=n0)
    assert (out == full).all()


def test_decode_slice_reduction_leaves_its_counters_clean(ctx):
    """K > 4096 is split over CTAs that meet through tile counters and f32 partial tiles in the
    workspace; repeated calls on the same workspace must give the same answer, and the counters
    (the part that has to start at zero) must be back at zero afterwards."""
    rng = np.random.default_rng(23)
    for (M, N, K) in [(16, 64, 8192), (7, 4752, 8192), (16, 48, 16384), (3, 32, 4096 + 768)]:
        a, wq, s = exact_case(rng, M, N, K)
        da, dw, ds = ctx.to_device(a), ctx.to_device(wq), ctx.to_device(s)
        dc = ctx.alloc(M * N * 2)
        ws = ctx.w4a16_workspace(N)
        p = ib.W4A16Params(M, N, K, 128, N, 0, ib.W4A16_DECODE, 0)
        want = oracle.w4a16(a, wq, s, threads=THREADS)
        for _ in range(3):
            dc.fill(0x7E)
            ctx.w4a16(p, da, dw, ds, dc, ws)
            ctx.workspace_status(ws)
            assert (dc.download(np.float16, (M, N)) == want).all(), (M, N, K)
        counters = ((N // 16) * 4 + 255) // 256 * 256
        raw = ws.download(np.uint8, (512 + counters,))
        assert not raw[384:448].any() and not raw[512:].any()     # status words 0..15 and the counters
        note = raw[448:464].view(np.uint32)                       # words 16..19: which weights the map describes
        assert (int(note[0]) | (int(note[1]) << 32), int(note[2]), int(note[3])) == (dw.ptr, N, K)
        for x in (da, dw, ds, dc, ws):
            x.free()


def test_decode_refuses_a_workspace_that_was_not_prepared(ctx):
    """K > 4096: the kernel fetches its weight tiles through a tensor map that prepare() leaves in the
    workspace. Running on a workspace that was never prepared, or that was prepared for other
    weights, must not reach the copy engine: nothing is computed and the status says so."""
    rng = np.random.default_rng(25)
    M, N, K = 4, 64, 8192
    a, wq, s = exact_case(rng, M, N, K)
    da, dw, ds, dw2 = ctx.to_device(a), ctx.to_device(wq), ctx.to_device(s), ctx.to_device(wq)
    dc, ws = ctx.alloc(M * N * 2).fill(0x7E), ctx.w4a16_workspace(N)
    p = ib.W4A16Params(M, N, K, 128, N, 0, ib.W4A16_DECODE, 0)
    ctx.w4a16_run(p, da, dw, ds, dc, ws, ib.W4A16_DECODE, 0)          # never prepared
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.workspace_status(ws)
    assert e.value.code_name == "INVALID_ARGUMENT"
    assert (dc.download(np.uint8, (M * N * 2,)) == 0x7E).all()
    ws.fill(0)
    ctx.w4a16_prepare(p, da, dw, ds, dc, ws)
    ctx.w4a16_run(p, da, dw2, ds, dc, ws, ib.W4A16_DECODE, 0)         # prepared, but for the other copy of the weights
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.workspace_status(ws)
    assert e.value.code_name == "INVALID_ARGUMENT"
    ws.fill(0)
    ctx.w4a16_prepare(p, da, dw2, ds, dc, ws)
    ctx.w4a16_run(p, da, dw2, ds, dc, ws, ib.W4A16_DECODE, 0)
    ctx.workspace_status(ws)
    assert (dc.download(np.float16, (M, N)) == oracle.w4a16(a, wq, s)).all()
    for x in (da, dw, ds, dw2, dc, ws):
        x.free()


def test_decode_refuses_misaligned_operands(ctx):
    """Operands the decode kernel would read with bulk copies / 16-byte loads must start on 16-byte
    boundaries: an explicit DECODE request is refused on the host (nothing is launched), and AUTO
    falls through to a kernel without that need and still computes the right answer."""
    rng = np.random.default_rng(24)
    M, N, K = 4, 32, 512
    a, wq, s = exact_case(rng, M, N, K)
    want = oracle.w4a16(a, wq, s)
    da, dw = ctx.to_device(a), ctx.to_device(wq)
    pad = ctx.alloc(s.nbytes + 64).fill(0)
    import ctypes as C
    from iree_b200 import runtime as rt
    shifted = pad.ptr + 8                      # 8-byte aligned only, like a sub-allocation at an odd offset
    rt.check(rt.library().iree_hal_b200_transfer_h2d(ctx.device, rt._vp(s), C.c_void_p(shifted), C.c_size_t(s.nbytes)))
    ctx.synchronize()
    dc, ws = ctx.alloc(M * N * 2), ctx.w4a16_workspace(N)
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.w4a16(ib.W4A16Params(M, N, K, 128, N, 0, ib.W4A16_DECODE, 0), da, dw, shifted, dc, ws)
    assert e.value.code_name == "INVALID_ARGUMENT" and "16-byte" in str(e.value)
    ctx.w4a16(ib.W4A16Params(M, N, K, 128, N, 0, ib.W4A16_AUTO, 0), da, dw, shifted, dc, ws)
    ctx.workspace_status(ws)
    assert (dc.download(np.float16, (M, N)) == want).all()
    for x in (da, dw, pad, dc, ws):
        x.free()


def test_argument_errors(ctx):
    a = np.zeros((2, 100), np.float16)
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.w4a16_host(ib.W4A16Params(2, 8, 100, 128, 8, 0, 0, 0), a, np.zeros((8, 50), np.uint8),
                       np.zeros((8, 1), np.float16), np.zeros((2, 8), np.float16))
    assert e.value.code_name == "INVALID_ARGUMENT"      # K not a multiple of the group size
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.w4a16_host(ib.W4A16Params(17, 16, 256, 128, 16, 0, ib.W4A16_DECODE, 0), np.zeros((17, 256), np.float16),
                       np.zeros((16, 128), np.uint8), np.zeros((16, 2), np.float16), np.zeros((17, 16), np.float16))
    assert e.value.code_name == "INVALID_ARGUMENT"      # decode kernel limit


@pytest.mark.parametrize("M,graph", [(1, False), (8, True), (16, False), (16, True)])
def test_overlapped_dispatch_chain_equals_the_serial_chain(ctx, M, graph):
    """A chain of decode dispatches in which every step's activations are the previous step's
    output (N = K), dispatched with overlap (programmatic dependent launch; stream mode and graph
    mode): each kernel may start, and prefetch weights, before the one ahead has finished, but
    must not read its activations early. The results are bit-identical to the serial chain."""
    from iree_b200 import runtime as rt
    rng = np.random.default_rng(33 + M)
    N = K = 4096
    steps = 12
    a0 = (rng.standard_normal((M, K)) * 0.5).astype(np.float16)
    layers = []
    for _ in range(3):
        wq = workloads.pack_int4(rng.integers(-7, 8, (N, K), dtype=np.int8))                 # zero mean
        s = (rng.uniform(0.5, 1.5, (N, K // 128)) / (4.5 * np.sqrt(K))).astype(np.float16)   # keeps the chain's scale near 1
        layers.append((ctx.to_device(wq), ctx.to_device(s)))
    bufs = [ctx.to_device(a0), ctx.alloc(M * N * 2), ctx.alloc(M * N * 2)]
    ws = ctx.w4a16_workspace(N)
    p = rt.W4A16Params(M, N, K, 128, N, 0, ib.W4A16_DECODE, 0)
    variant, tile_n = ctx.w4a16_prepare(p, bufs[0], layers[0][0], layers[0][1], bufs[1], ws)

    def chain():
        bufs[0].upload(a0)
        if graph:
            ctx.begin_graph()
        src = 0
        for i in range(steps):
            dst = 1 + (i % 2)
            wq, s = layers[i % 3]
            ctx.w4a16_run(p, bufs[src], wq, s, bufs[dst], ws, variant, tile_n)
            src = dst
        if graph:
            g = ctx.end_graph()
            g.execute()
            ctx.synchronize()
            g.release()
        ctx.workspace_status(ws)
        return bufs[src].download(np.float16, (M, N))

    serial = chain()
    ctx.set_dispatch_overlap(True)
    try:
        overlapped = chain()
    finally:
        ctx.set_dispatch_overlap(False)
    assert np.isfinite(serial.astype(np.float32)).all() and np.abs(serial.astype(np.float32)).max() > 1e-3
    assert np.array_equal(serial.view(np.uint16), overlapped.view(np.uint16))
    for b in bufs + [ws] + [x for l in layers for x in l]:
        b.free()
