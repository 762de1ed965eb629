"""Parity of the GPU pack / unpack / mmt4d entry points with the CPU oracle, through the C ABI.

pack and unpack move bytes, so every comparison is bit-exact; mmt4d is bit-exact for s8s8s32
and within rtol = atol = 1e-2 for the float types (exact on small-integer data).
"""
import numpy as np
import pytest

import iree_b200 as ib
import oracle
from iree_b200 import runtime as rt
from iree_b200.runtime import mmt4d_numpy, pack_numpy, unpack_numpy

pytestmark = pytest.mark.gpu

RTOL = ATOL = 1e-2

# builtins/ukernel/tools/pack_test.c:137-147 (outer shapes) and :214-245 (type / tile pairs), plus
# the tiles the x86-64 and generic tables choose for the benchmark types.
OUTER_SHAPES = [(0, 1), (1, 0), (1, 1), (3, 2), (9, 33)]
TYPE_TILES = [(np.float32, 3, 5), (np.int8, 4, 2), (np.int32, 3, 4), (np.float16, 6, 7), (np.uint16, 9, 2),
              (np.float32, 8, 1), (np.int8, 8, 2), (np.float32, 8, 8), (np.int32, 8, 8), (np.float32, 16, 1),
              (np.uint16, 16, 2), (np.int8, 16, 2), (np.float32, 16, 16), (np.int32, 16, 16), (np.int8, 1, 2),
              (np.float16, 16, 1)]


def random_array(rng, dtype, shape):
    dtype = np.dtype(dtype)
    return rng.integers(0, 256, (int(np.prod(shape)) * dtype.itemsize,), dtype=np.uint8).view(dtype).reshape(shape)


def cases():
    """(out_shape, in_shape, transpose_inner, transpose_outer) the way pack_test.c:152-190 builds them."""
    rng = np.random.default_rng(7)
    for (s0, s1) in OUTER_SHAPES:
        for ti in (False, True):
            for to in (False, True):
                for pad in ("none", "one_incomplete_tile", "a_lot"):
                    yield (s0, s1), ti, to, pad, rng


@pytest.mark.parametrize("dtype,tile0,tile1", TYPE_TILES)
def test_pack_matches_the_oracle_bit_for_bit(ctx, dtype, tile0, tile1):
    for (s0, s1), ti, to, pad, rng in cases():
        o0, o1 = (s0 + 16, s1 + 16) if pad == "a_lot" else (s0, s1)
        out_shape = ((o1, o0) if to else (o0, o1)) + (tile0, tile1)
        t0, t1 = (tile1, tile0) if ti else (tile0, tile1)
        in0, in1 = s0 * t0, s1 * t1
        if pad != "none":
            in0 = max(in0 - int(rng.integers(0, t0)), 0)
            in1 = max(in1 - int(rng.integers(0, t1)), 0)
        x = random_array(rng, dtype, (in0, in1))
        padding = int(rng.integers(0, 256)) * 0x01010101 & ((1 << (8 * np.dtype(dtype).itemsize)) - 1)
        want = oracle.pack_port(x, out_shape, ti, to, padding)
        got = pack_numpy(ctx, x, (t0, t1), ti, to, padding, out_shape=out_shape)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (dtype, out_shape, x.shape, ti, to, pad)


@pytest.mark.parametrize("dtype,tile0,tile1", TYPE_TILES)
def test_unpack_matches_the_oracle_and_leaves_the_rest_alone(ctx, dtype, tile0, tile1):
    for (s0, s1), ti, to, pad, rng in cases():
        o0, o1 = (s0 + 16, s1 + 16) if pad == "a_lot" else (s0, s1)
        in_shape = ((o1, o0) if to else (o0, o1)) + (tile0, tile1)
        t0, t1 = (tile1, tile0) if ti else (tile0, tile1)
        out0, out1 = s0 * t0, s1 * t1
        if pad != "none":
            out0 = max(out0 - int(rng.integers(0, t0)), 0)
            out1 = max(out1 - int(rng.integers(0, t1)), 0)
        x4 = random_array(rng, dtype, in_shape)
        want = oracle.unpack_port(x4, (out0, out1), ti, to)
        got = unpack_numpy(ctx, x4, (out0, out1), ti, to)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (dtype, in_shape, (out0, out1), ti, to, pad)


@pytest.mark.skipif(not oracle.have_ref(), reason="reference ukernels were not compiled")
def test_pack_and_unpack_match_the_reference_ukernels_on_operand_sized_matrices(ctx):
    """The three packs of one data-tiled matmul (pack.c / unpack.c as built from the reference's
    own sources): LHS, RHS with both transposes, and the accumulator round trip."""
    rng = np.random.default_rng(11)
    M, K, N = 300, 517, 260
    a = rng.integers(-128, 128, (M, K), dtype=np.int8)
    b = rng.integers(-128, 128, (K, N), dtype=np.int8)
    m0, n0, k0 = 16, 16, 2
    m1, n1, k1 = -(-M // m0), -(-N // n0), -(-K // k0)
    assert np.array_equal(pack_numpy(ctx, a, (m0, k0)), oracle.pack_ref(a, (m1, k1, m0, k0)))
    assert np.array_equal(pack_numpy(ctx, b, (k0, n0), True, True), oracle.pack_ref(b, (n1, k1, n0, k0), True, True))
    acc = rng.integers(-2 ** 31, 2 ** 31, (m1, n1, m0, n0)).astype(np.int32)
    assert np.array_equal(unpack_numpy(ctx, acc, (M, N)), oracle.unpack_ref(acc, (M, N)))
    f = rng.standard_normal((M, N)).astype(np.float32)
    assert np.array_equal(pack_numpy(ctx, f, (m0, n0)), oracle.pack_ref(f, (m1, n1, m0, n0)))


def test_pack_of_a_strided_view_and_tiles_too_large_to_stage(ctx):
    rng = np.random.default_rng(3)
    base = rng.integers(-128, 128, (70, 200), dtype=np.int8)
    view = base[3:60:2, 5:190:3]                       # in_offset, in_stride0 and in_stride1 all in play
    want = oracle.pack_port(np.ascontiguousarray(view), (-(-view.shape[0] // 8), -(-view.shape[1] // 4), 8, 4), padding=0x7F)
    assert np.array_equal(pack_numpy(ctx, view, (8, 4), padding=0x7F), want)
    big = rng.standard_normal((150, 700)).astype(np.float32)  # 100 x 300 tiles: the direct path
    want = oracle.pack_port(big, (2, 3, 100, 300), padding=0)
    assert np.array_equal(pack_numpy(ctx, big, (100, 300)), want)
    assert np.array_equal(unpack_numpy(ctx, want, (150, 700)), big)


def test_round_trip_at_benchmark_size(ctx):
    """unpack(pack(x)) == x on the weight matrix of the W8A8 configuration (4096 x 11008 int8),
    both operand roles; the padded tail of a ragged matrix holds the fill value."""
    rng = np.random.default_rng(5)
    w = rng.integers(-127, 128, (4096, 11008), dtype=np.int8)
    p = pack_numpy(ctx, w, (2, 16), True, True)                # RHS role: [N1, K1, N0, K0]
    assert p.shape == (688, 2048, 16, 2)
    assert np.array_equal(p[5, 7], w[14:16, 80:96].T)
    assert np.array_equal(unpack_numpy(ctx, p, w.shape, True, True), w)
    ragged = w[:4001, :1003]
    p = pack_numpy(ctx, ragged, (16, 2), padding=0x55)
    assert np.array_equal(unpack_numpy(ctx, p, ragged.shape), ragged)
    assert (p[-1, :, 1:, :] == 0x55).all() and (p[:, -1, :, 1] == 0x55).all()


def test_argument_errors(ctx):
    buf = ctx.alloc(1024)
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.uk_pack(buf, 0, 8, 1, buf, 0, 16, 7, 8, 8, 2, 2, 4, 2, 0, 0x02)   # out_stride1 != o2 * o3
    assert e.value.code_name == "INVALID_ARGUMENT"
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.uk_pack(buf, 0, 8, 1, buf, 0, 16, 8, 8, 8, 2, 2, 4, 2, 0, 0x07)   # no such type
    assert e.value.code_name == "INVALID_ARGUMENT"
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.uk_pack(buf, 0, 8, 1, buf, 0, 8, 8, 8, 8, 1, 1, 4, 2, 0, 0x02)    # tiles do not cover the matrix
    assert e.value.code_name == "INVALID_ARGUMENT"
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.uk_mmt4d(buf, 0, 8, buf, 0, 8, buf, 0, 8, 1, 1, 1, 2, 2, 2, 0x0B, buf)  # no such type
    assert e.value.code_name == "INVALID_ARGUMENT"
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.uk_mmt4d(buf, 0, 8, buf, 0, 8, buf, 0, 8, 1, 1, 1, 2, 2, 3, 0x0A, buf)  # s8s4s32 with an odd K0
    assert e.value.code_name == "INVALID_ARGUMENT"
    buf.free()


# ---- mmt4d ---------------------------------------------------------------------------------------------

# builtins/ukernel/tools/mmt4d_test.c:449-504: generic tiles, then the x86-64 tiles incl. narrow M0.
MMT4D_I8_TILES = [(4, 4, 2), (3, 5, 7), (9, 6, 3), (1, 16, 2), (2, 16, 2), (4, 16, 2), (8, 16, 2), (16, 16, 2), (8, 8, 2)]
MMT4D_SHAPES = [(1, 1, 1), (2, 3, 5), (3, 2, 17), (7, 9, 64)]  # outer M, N, K


@pytest.mark.parametrize("m0,n0,k0", MMT4D_I8_TILES)
def test_mmt4d_s8s8s32_bit_exact(ctx, m0, n0, k0):
    rng = np.random.default_rng(m0 * 100 + n0 * 10 + k0)
    for (M, N, K) in MMT4D_SHAPES:
        lhs = rng.integers(-128, 128, (M, K, m0, k0), dtype=np.int8)
        rhs = rng.integers(-128, 128, (N, K, n0, k0), dtype=np.int8)
        want = oracle.mmt4d_port(oracle.TYPE_S8S8S32, lhs, rhs)
        assert np.array_equal(mmt4d_numpy(ctx, rt.UK_MMT4D_S8S8S32, lhs, rhs), want), (M, N, K)
        acc = rng.integers(-10 ** 6, 10 ** 6, (M, N, m0, n0)).astype(np.int32)
        want = oracle.mmt4d_port(oracle.TYPE_S8S8S32, lhs, rhs, acc)
        assert np.array_equal(mmt4d_numpy(ctx, rt.UK_MMT4D_S8S8S32, lhs, rhs, acc), want), (M, N, K, "accumulate")


@pytest.mark.parametrize("type_flag,otype", [(rt.UK_MMT4D_F16F16F32, "F16F16F32"), (rt.UK_MMT4D_BF16BF16F32, "BF16BF16F32"),
                                             (rt.UK_MMT4D_F16F16F16, "F16F16F16")])
@pytest.mark.parametrize("m0,n0,k0", [(16, 16, 1), (8, 8, 1), (1, 16, 1), (3, 5, 7)])
def test_mmt4d_float_types(ctx, type_flag, otype, m0, n0, k0):
    # The 16-bit output type is the f32 result rounded once at the end (mmt4d_tile_generic.c:199-260
    # with SKIP_INTERMEDIATE_ROUNDINGS).
    ot = oracle.TYPE_BF16BF16F32 if otype.startswith("BF16") else oracle.TYPE_F16F16F32
    narrow = (lambda x: oracle.truncf(x)) if otype == "F16F16F16" else (lambda x: x)
    rng = np.random.default_rng(9)
    bf = type_flag == rt.UK_MMT4D_BF16BF16F32
    for (M, N, K) in [(2, 3, 40), (5, 4, 256)]:
        def draw(shape, small):
            x = (rng.integers(-4, 5, shape) if small else rng.standard_normal(shape) / np.sqrt(K * k0)).astype(np.float32)
            return (x.view(np.uint32) >> 16).astype(np.uint16) if bf else x.astype(np.float16)
        for small in (True, False):
            lhs, rhs = draw((M, K, m0, k0), small), draw((N, K, n0, k0), small)
            want = narrow(oracle.mmt4d_port(ot, lhs, rhs)).astype(np.float64)
            got = mmt4d_numpy(ctx, type_flag, lhs, rhs).astype(np.float64)
            if small:
                assert np.array_equal(got, want)
            else:
                assert np.allclose(got, want, rtol=RTOL, atol=ATOL)
            if type_flag != rt.UK_MMT4D_F16F16F16:
                acc = rng.standard_normal((M, N, m0, n0)).astype(np.float32)
                want = oracle.mmt4d_port(ot, lhs, rhs, acc)
                got = mmt4d_numpy(ctx, type_flag, lhs, rhs, acc)
                assert np.allclose(got, want, rtol=RTOL, atol=ATOL)


def test_mmt4d_empty_and_k_zero(ctx):
    lhs = np.zeros((2, 0, 4, 2), np.int8)
    rhs = np.zeros((3, 0, 4, 2), np.int8)
    assert (mmt4d_numpy(ctx, rt.UK_MMT4D_S8S8S32, lhs, rhs) == 0).all()            # K = 0: zero fill
    acc = np.arange(2 * 3 * 16, dtype=np.int32).reshape(2, 3, 4, 4)
    assert np.array_equal(mmt4d_numpy(ctx, rt.UK_MMT4D_S8S8S32, lhs, rhs, acc), acc)  # K = 0 + ACCUMULATE: untouched
    assert mmt4d_numpy(ctx, rt.UK_MMT4D_S8S8S32, np.zeros((0, 3, 4, 2), np.int8), np.zeros((3, 3, 4, 2), np.int8)).size == 0


def test_data_tiled_matmul_chain_on_the_gpu_equals_the_reference_chain(ctx):
    """Configuration 0 the way llvm-cpu runs it (pack, pack, mmt4d, unpack with the 16x16x2 VNNI
    tiles), every step on the GPU, bit-exact against the reference's own chain."""
    from iree_b200 import workloads
    a, b = workloads.c1_i8_matmul()
    M, K = a.shape
    N = b.shape[1]
    m0, n0, k0 = 16, 16, 2
    pl = pack_numpy(ctx, a, (m0, k0))
    pr = pack_numpy(ctx, b, (k0, n0), True, True)
    po = mmt4d_numpy(ctx, rt.UK_MMT4D_S8S8S32, pl, pr)
    got = unpack_numpy(ctx, po, (M, N))
    want = oracle.matmul_ref(oracle.TYPE_S8S8S32, a, b) if oracle.have_ref() else oracle.matmul_port(oracle.TYPE_S8S8S32, a, b)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("type_flag,tile", [(rt.UK_MMT4D_S8S8S32, (16, 16, 2)), (rt.UK_MMT4D_F16F16F32, (16, 16, 1)),
                                            (rt.UK_MMT4D_BF16BF16BF16, (16, 16, 1))])
def test_mmt4d_on_tiled_operands_is_one_launch_and_equals_the_untiling_path(ctx, type_flag, tile):
    """The kernel that reads tiled operands as they are (one launch) against the path that un-tiles both
    operands first (four launches): many tiles per CTA, K1 tails, outer extents that do not fill a CTA
    tile, operands and result inside larger buffers (offsets and outer strides), ACCUMULATE.
    Integer results are identical; float results are sums of the same products in another order."""
    m0, n0, k0 = tile
    rng = np.random.default_rng(5)
    i8 = type_flag == rt.UK_MMT4D_S8S8S32
    bf = type_flag == rt.UK_MMT4D_BF16BF16BF16
    idt = np.int8 if i8 else np.uint16 if bf else np.float16
    odt = np.int32 if i8 else np.uint16 if bf else np.float32

    def draw(shape, K):
        if i8:
            return rng.integers(-128, 128, shape, dtype=np.int8)
        x = (rng.standard_normal(shape) / np.sqrt(K)).astype(np.float32)
        return (x.view(np.uint32) >> 16).astype(np.uint16) if bf else x.astype(np.float16)

    for (M, N, K, pad) in [(9, 21, 130, 0), (40, 70, 257, 48), (3, 300, 64, 16), (33, 1, 1, 0)]:
        lhs, rhs = draw((M, K, m0, k0), K * k0), draw((N, K, n0, k0), K * k0)
        # rows of outer tiles `pad` elements apart from tight, operands 64 elements into their buffers
        ls, rs, os_ = K * m0 * k0 + pad, K * n0 * k0 + pad, N * m0 * n0 + pad
        lbuf = np.zeros(64 + M * ls, idt); rbuf = np.zeros(64 + N * rs, idt)
        for i in range(M):
            lbuf[64 + i * ls: 64 + i * ls + K * m0 * k0] = lhs[i].ravel()
        for i in range(N):
            rbuf[64 + i * rs: 64 + i * rs + K * n0 * k0] = rhs[i].ravel()
        acc = rng.integers(-10 ** 6, 10 ** 6, (M, N, m0, n0)).astype(np.int32) if i8 else rng.standard_normal((M, N, m0, n0)).astype(np.float32)
        dl, dr = ctx.to_device(lbuf), ctx.to_device(rbuf)
        results = {}
        for accumulate in ((False, True) if not bf else (False,)):
            for untile in (False, True):
                obuf = np.full(64 + M * os_, 0x55, odt)
                if accumulate:
                    for i in range(M):
                        obuf[64 + i * os_: 64 + i * os_ + N * m0 * n0] = acc[i].ravel().view(odt)
                do = ctx.to_device(obuf)
                flags = type_flag | (rt.UK_MMT4D_ACCUMULATE if accumulate else 0) | (rt.UK_MMT4D_UNTILE if untile else 0)
                ws = ctx.uk_mmt4d_workspace(M, N, K, m0, n0, k0, flags)
                before = ctx.launch_count
                ctx.uk_mmt4d(dl, 64, ls, dr, 64, rs, do, 64, os_, M, N, K, m0, n0, k0, flags, ws)
                launches = ctx.launch_count - before
                ctx.workspace_status(ws)
                assert launches == (4 if untile else 1), (M, N, K, untile, launches)
                got = do.download(odt, (64 + M * os_,))
                assert (got[:64] == 0x55).all()
                tiles = np.stack([got[64 + i * os_: 64 + i * os_ + N * m0 * n0] for i in range(M)]).reshape(M, N, m0, n0)
                if pad:
                    gaps = np.stack([got[64 + i * os_ + N * m0 * n0: 64 + (i + 1) * os_] for i in range(M)])
                    assert (gaps == 0x55).all()
                results[(accumulate, untile)] = tiles
                do.free(); ws.free()
            a, b = results[(accumulate, False)], results[(accumulate, True)]
            if i8:
                assert np.array_equal(a, b), (M, N, K, accumulate)
            elif bf:
                fa, fb = (a.astype(np.uint32) << 16).view(np.float32), (b.astype(np.uint32) << 16).view(np.float32)
                assert np.allclose(fa, fb, rtol=RTOL, atol=ATOL), (M, N, K)
            else:
                assert np.allclose(a, b, rtol=1e-4, atol=1e-4), (M, N, K, accumulate)
        if i8:
            want = oracle.mmt4d_port(oracle.TYPE_S8S8S32, lhs, rhs, acc)
            assert np.array_equal(results[(True, False)], want), (M, N, K)
        dl.free(); dr.free()


@pytest.mark.parametrize("dtype,tile", [(np.float32, (16, 16)), (np.int32, (8, 4)), (np.float16, (16, 8)), (np.int8, (7, 32)),
                                        (np.int8, (16, 16)), (np.float32, (1, 64))])
@pytest.mark.parametrize("transpose_outer", [False, True])
def test_pack_and_unpack_by_tma_copy_equal_the_staging_kernels(ctx, dtype, tile, transpose_outer):
    """Shapes the TMA-only copy takes (tile rows of whole 16-byte pieces, no inner transpose, a matrix
    the tiles cover exactly): bit-identical to the staging kernels and to the oracle, in both
    directions, one tile to many boxes per CTA, ragged last box along o1."""
    rng = np.random.default_rng(3)
    t0, t1 = tile
    for (n0, n1) in [(1, 1), (3, 5), (37, 70), (150, 301)]:
        x = rng.integers(-100, 100, (n0 * t0, n1 * t1)).astype(dtype)
        shape4 = ((n1, n0) if transpose_outer else (n0, n1)) + (t0, t1)
        want = oracle.pack_port(x, shape4, False, transpose_outer)
        got = pack_numpy(ctx, x, (t0, t1), False, transpose_outer)
        staged = pack_numpy(ctx, x, (t0, t1), False, transpose_outer, extra_flags=rt.UK_PACK_NO_TMA)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (n0, n1)
        assert np.array_equal(staged.view(np.uint8), want.view(np.uint8)), (n0, n1)
        back = unpack_numpy(ctx, got, x.shape, False, transpose_outer)
        back_staged = unpack_numpy(ctx, got, x.shape, False, transpose_outer, extra_flags=rt.UK_PACK_NO_TMA)
        assert np.array_equal(back.view(np.uint8), x.view(np.uint8)), (n0, n1)
        assert np.array_equal(back_staged.view(np.uint8), x.view(np.uint8)), (n0, n1)


@pytest.mark.parametrize("graph", [False, True])
def test_overlapped_data_tiled_chain_equals_the_reference(ctx, graph):
    """pack, pack, mmt4d, unpack as four dependent dispatches on device-resident buffers, launched
    early (programmatic dependent launch; stream mode and one recorded graph): every kernel of the
    chain waits on the device for the one ahead before it touches memory. Bit-exact against the
    reference's chain, several times over the same buffers."""
    from iree_b200 import workloads
    a, b = workloads.c1_i8_matmul()
    M, K = a.shape
    N = b.shape[1]
    want = oracle.matmul_ref(oracle.TYPE_S8S8S32, a, b) if oracle.have_ref() else oracle.matmul_port(oracle.TYPE_S8S8S32, a, b)
    da, db = ctx.to_device(a), ctx.to_device(b)
    pl, pr = ctx.alloc(M * K), ctx.alloc(N * K)
    po, out = ctx.alloc(M * N * 4), ctx.alloc(M * N * 4)
    ws = ctx.uk_mmt4d_workspace(M // 16, N // 16, K // 2, 16, 16, 2, rt.UK_MMT4D_S8S8S32)
    i8, i32 = rt.UK_PACK_TYPE[1], rt.UK_PACK_TYPE[4]

    def chain():
        ctx.uk_pack(da, 0, K, 1, pl, 0, (K // 2) * 32, 32, M, K, M // 16, K // 2, 16, 2, 0, i8)
        ctx.uk_pack(db, 0, N, 1, pr, 0, (K // 2) * 32, 32, K, N, N // 16, K // 2, 16, 2, 0,
                    i8 | rt.UK_TRANSPOSE_INNER | rt.UK_TRANSPOSE_OUTER)
        ctx.uk_mmt4d(pl, 0, (K // 2) * 32, pr, 0, (K // 2) * 32, po, 0, (N // 16) * 256, M // 16, N // 16, K // 2, 16, 16, 2,
                     rt.UK_MMT4D_S8S8S32, ws)
        ctx.uk_unpack(po, 0, (N // 16) * 256, 256, out, 0, N, 1, M // 16, N // 16, 16, 16, M, N, i32)

    chain()                     # first use allocates the context's scratch: keep that out of the recording
    ctx.synchronize()
    ctx.set_dispatch_overlap(True)
    try:
        for rounds in range(3):
            out.fill(0xEE)
            if graph:
                ctx.begin_graph()
                chain(); chain()
                g = ctx.end_graph()
                g.execute()
                ctx.synchronize()
                g.release()
            else:
                chain(); chain()
            got = out.download(np.int32, (M, N))
            assert np.array_equal(got, want), rounds
    finally:
        ctx.set_dispatch_overlap(False)
    ctx.workspace_status(ws)
    ctx.uk_status()
    for x in (da, db, pl, pr, po, out, ws):
        x.free()


@pytest.mark.parametrize("dtype,tile", [(np.int8, (16, 2)), (np.float16, (16, 1))])
def test_left_hand_side_pack_of_two_byte_tile_rows(ctx, dtype, tile):
    """[M, K] -> [M1, K1, 16, K0] without transposes where a tile row is two bytes (int8 16 x 2, f16
    16 x 1): the TMA-box / gather / bulk-copy kernel against the staging kernel and the oracle, whole and
    ragged matrices (zero padding), many regions per CTA."""
    rng = np.random.default_rng(8)
    t0, t1 = tile
    for (M, K) in [(16, 2), (128, 128), (100, 61 * t1), (512, 4096), (1000, 130 * t1)]:
        x = rng.integers(-100, 100, (M, K)).astype(dtype)
        shape4 = (-(-M // t0), -(-K // t1), t0, t1)
        want = oracle.pack_port(x, shape4, False, False)
        got = pack_numpy(ctx, x, (t0, t1))
        staged = pack_numpy(ctx, x, (t0, t1), extra_flags=rt.UK_PACK_NO_TMA)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (M, K)
        assert np.array_equal(staged.view(np.uint8), want.view(np.uint8)), (M, K)


def test_right_hand_side_pack_of_f16_tiles_is_a_tma_copy(ctx):
    """[K, N] f16 -> [N1, K1, 16, 1] with both transposes: a transposed tile one row high is that row, so
    the TMA-only copy takes it; equal to the staging kernel and the oracle."""
    rng = np.random.default_rng(9)
    for (K, N) in [(64, 16), (300, 160), (1024, 2048)]:
        x = rng.standard_normal((K, N)).astype(np.float16)
        want = oracle.pack_port(x, (N // 16, K, 16, 1), True, True)
        got = pack_numpy(ctx, x, (1, 16), True, True)
        staged = pack_numpy(ctx, x, (1, 16), True, True, extra_flags=rt.UK_PACK_NO_TMA)
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), (K, N)
        assert np.array_equal(staged.view(np.uint16), want.view(np.uint16)), (K, N)


def _unpack_nibbles(rhs_bytes, signed):
    """[N, K, N0, K0 / 2] bytes -> [N, K, N0, K0] integers: low nibble first (mmt4d_tile_generic.c:11-50, 108-143)."""
    lo = (rhs_bytes & 0xF).astype(np.int32)
    hi = (rhs_bytes >> 4).astype(np.int32)
    if signed:
        lo = np.where(lo >= 8, lo - 16, lo)
        hi = np.where(hi >= 8, hi - 16, hi)
    return np.stack([lo, hi], axis=-1).reshape(rhs_bytes.shape[:-1] + (rhs_bytes.shape[-1] * 2,))


@pytest.mark.parametrize("type_flag,ldt,rdt,tile", [
    (rt.UK_MMT4D_F32F32F32, np.float32, np.float32, (16, 16, 1)), (rt.UK_MMT4D_F32F32F32, np.float32, np.float32, (3, 5, 7)),
    (rt.UK_MMT4D_S16S16S32, np.int16, np.int16, (16, 16, 2)), (rt.UK_MMT4D_S16S8S32, np.int16, np.int8, (4, 8, 3)),
    (rt.UK_MMT4D_S16U4S32, np.int16, np.uint8, (1, 32, 8)), (rt.UK_MMT4D_S8S4S32, np.int8, np.uint8, (4, 16, 2)),
    (rt.UK_MMT4D_S8S4S32, np.int8, np.uint8, (3, 5, 6))])
def test_mmt4d_types_without_a_tensor_core_kernel(ctx, type_flag, ldt, rdt, tile):
    """f32f32f32 and the s16 / 4-bit types (exported_bits.h:29-42) through the one-thread-per-element kernel:
    integer types exact against a numpy restatement of the reference's generic tile functions (4-bit
    right-hand sides: two elements per byte, low nibble first, unsigned for u4 and sign-extended for s4),
    f32 within tolerance; with and without ACCUMULATE."""
    m0, n0, k0 = tile
    rng = np.random.default_rng(type_flag * 7 + m0)
    four_bit = type_flag in (rt.UK_MMT4D_S16U4S32, rt.UK_MMT4D_S8S4S32)
    for (M, N, K) in [(1, 1, 1), (2, 3, 5), (7, 9, 33)]:
        if ldt == np.float32:
            lhs = rng.standard_normal((M, K, m0, k0)).astype(np.float32)
            rhs = rng.standard_normal((N, K, n0, k0)).astype(np.float32)
            acc = rng.standard_normal((M, N, m0, n0)).astype(np.float32)
            l64, r64 = lhs.astype(np.float64), rhs.astype(np.float64)
        else:
            info = np.iinfo(ldt)
            lhs = rng.integers(info.min, info.max + 1, (M, K, m0, k0)).astype(ldt)
            if four_bit:
                rhs = rng.integers(0, 256, (N, K, n0, k0 // 2)).astype(np.uint8)
                r64 = _unpack_nibbles(rhs, signed=(type_flag == rt.UK_MMT4D_S8S4S32)).astype(np.int64)
            else:
                rinfo = np.iinfo(rdt)
                rhs = rng.integers(rinfo.min, rinfo.max + 1, (N, K, n0, k0)).astype(rdt)
                r64 = rhs.astype(np.int64)
            acc = rng.integers(-10 ** 6, 10 ** 6, (M, N, m0, n0)).astype(np.int32)
            l64 = lhs.astype(np.int64)
        prod = np.einsum("mkac,nkbc->mnab", l64, r64)
        for with_acc in (False, True):
            got = rt.mmt4d_numpy(ctx, type_flag, lhs, rhs, acc if with_acc else None)
            want = prod + (acc if with_acc else 0)
            if ldt == np.float32:
                assert np.allclose(got, want, rtol=1e-4, atol=1e-4), (M, N, K, with_acc)
            else:
                # 32-bit wrap-around like the reference's int32 accumulator
                assert np.array_equal(got, (want & 0xFFFFFFFF).astype(np.uint32).view(np.int32)), (M, N, K, with_acc)
                assert np.array_equal(got, oracle.mmt4d_int_types_port(type_flag, lhs, rhs, acc if with_acc else None))
            if oracle.have_ref():  # the reference's own ukernel (its generic tile functions) on the same operands
                ref = oracle.mmt4d_ref(type_flag, lhs, rhs, acc if with_acc else None)
                if ldt == np.float32:
                    assert np.allclose(got, ref, rtol=1e-4, atol=1e-4), (M, N, K, with_acc, "reference")
                else:
                    assert np.array_equal(got, ref), (M, N, K, with_acc, "reference")
