"""Pins the CPU oracle (oracle/contraction_oracle.c) before anything trusts it:

* against golden vectors produced by the reference's own ukernels (tests/golden/matmul_ref.npz,
  made by tests/golden/make_golden.py), on the shapes the reference's ukernel and e2e matmul
  tests use;
* against the reference ukernels live (oracle/_ref) when they are present: pack, mmt4d, unpack
  one at a time and chained, generic and architecture tile functions;
* the int4 nibble order against the reference's s8s4s32 tile function.
"""
import os

import numpy as np
import pytest

import oracle
from tests.golden.make_golden import SHAPES, inputs
from iree_b200 import workloads

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "matmul_ref.npz")
KINDS = (("s8s8s32", oracle.TYPE_S8S8S32), ("f16f16f32", oracle.TYPE_F16F16F32))
needs_ref = pytest.mark.skipif(not oracle.have_ref(), reason="oracle/_ref not built")


@pytest.fixture(scope="module")
def golden(built):
    return np.load(GOLDEN)


@pytest.mark.parametrize("kind,t", KINDS)
def test_port_matches_reference_golden_vectors(golden, kind, t):
    for i, (M, N, K) in enumerate(SHAPES):
        a, b = inputs(kind, M, N, K, 1000 + i)
        want = golden["%s_%dx%dx%d" % (kind, M, N, K)]
        got = oracle.matmul_port(t, a, b)
        assert got.dtype == want.dtype and (got == want).all(), (kind, M, N, K)
        # the naive whole-dispatch reference agrees too (exact: small-integer data)
        assert (oracle.matmul_naive(t, a, b) == want).all(), (kind, M, N, K)
        acc0 = np.random.default_rng(77 + i).integers(-5, 5, (M, N)).astype(want.dtype)
        want_acc = golden["%s_%dx%dx%d_acc" % (kind, M, N, K)]
        assert (oracle.matmul_port(t, a, b, acc=acc0) == want_acc).all(), (kind, M, N, K, "acc")


@pytest.mark.parametrize("kind,t", KINDS)
def test_port_is_tile_independent(built, kind, t):
    # Results do not depend on the data-tiling choice (narrow-M tiles included).
    a, b = inputs(kind, 7, 33, 50, 5)
    base = oracle.matmul_port(t, a, b, tile=(16, 16, 2 if kind == "s8s8s32" else 1))
    for tile in ((1, 16, 2), (8, 8, 2), (4, 16, 2), (8, 8, 1), (16, 16, 1), (2, 8, 1)):
        assert (oracle.matmul_port(t, a, b, tile=tile) == base).all(), tile


def test_x86_64_tile_choice():
    # CPUMaterializeEncodingPass.cpp:168-277 tables + narrow-M rule :284-377
    assert oracle.x86_64_tile(oracle.TYPE_S8S8S32, 1024, 1024) == (16, 16, 2)
    assert oracle.x86_64_tile(oracle.TYPE_F16F16F32, 4096, 4096) == (16, 16, 1)
    assert oracle.x86_64_tile(oracle.TYPE_S8S8S32, 1, 11008) == (1, 16, 2)
    assert oracle.x86_64_tile(oracle.TYPE_S8S8S32, 5, 11008) == (8, 16, 2)
    assert oracle.x86_64_tile(oracle.TYPE_S8S8S32, 16, 11008) == (16, 16, 2)


@needs_ref
def test_narrow_n_products_swap_their_operands(built):
    """SetEncoding records at most one narrow dimension (M wins a tie); a narrow-N result is
    materialised as the transposed product with the operands swapped, which must give the same
    numbers as the plain product."""
    assert oracle.matmul_narrow_sizes(1, 1000) == (1, None) and oracle.matmul_narrow_sizes(1000, 1) == (None, 1)
    assert oracle.matmul_narrow_sizes(8, 8) == (8, None) and oracle.matmul_narrow_sizes(9, 3) == (None, 3)
    assert oracle.matmul_narrow_sizes(16, 15) == (None, 15) and oracle.matmul_narrow_sizes(64, 64) == (None, None)
    assert oracle.is_narrow_n_result(1000, 1) and oracle.is_narrow_n_result(9, 3)
    assert not oracle.is_narrow_n_result(3, 9) and not oracle.is_narrow_n_result(8, 8)
    assert oracle.x86_64_tile(oracle.TYPE_S8S8S32, 3, 1000) == (4, 16, 2)       # the swapped problem of [1000, K] x [K, 3]
    rng = np.random.default_rng(12)
    for (M, N, K) in [(1000, 1, 64), (37, 3, 129), (9, 3, 10), (10, 1, 10)]:
        a = rng.integers(-128, 128, (M, K), dtype=np.int8)
        b = rng.integers(-128, 128, (K, N), dtype=np.int8)
        want = a.astype(np.int32) @ b.astype(np.int32)
        assert (oracle.matmul_port(oracle.TYPE_S8S8S32, a, b) == want).all()
        acc = rng.integers(-1000, 1000, (M, N), dtype=np.int32)
        assert (oracle.matmul_port(oracle.TYPE_S8S8S32, a, b, acc=acc) == want + acc).all()


@pytest.mark.parametrize("dtype", [np.int8, np.float16, np.float32, np.int32])
def test_pack_unpack_match_reference_ukernels(built, dtype):
    rng = np.random.default_rng(3)
    for (r, c, t0, t1) in [(5, 7, 2, 4), (16, 16, 16, 2), (33, 9, 8, 1), (1, 1, 16, 16), (10, 1000, 16, 2)]:
        x = rng.integers(-100, 100, (r, c)).astype(dtype)
        for ti in (False, True):
            for to in (False, True):
                tile0, tile1 = (t1, t0) if ti else (t0, t1)
                o0, o1 = -(-r // tile0), -(-c // tile1)
                if to:
                    o0, o1 = o1, o0
                tiles = (o0, o1, t0, t1)
                if dtype == np.int32 and (ti or to):
                    continue  # result tiles are never transposed on this path
                got = oracle.pack_port(x, tiles, ti, to)
                for mode in (0, 1):
                    want = oracle.pack_ref(x, tiles, ti, to, cpu_mode=mode)
                    assert (got == want).all(), (r, c, tiles, ti, to, mode)
                if dtype in (np.float32, np.int32, np.float16):
                    back = oracle.unpack_port(got, (r, c), ti, to)
                    assert (back == x).all()
                    assert (oracle.unpack_ref(got, (r, c), ti, to) == x).all()


@needs_ref
@pytest.mark.parametrize("kind,t", KINDS)
def test_mmt4d_matches_reference_ukernel(built, kind, t):
    rng = np.random.default_rng(9)
    k0 = 2 if kind == "s8s8s32" else 1
    for (M1, N1, K1, M0, N0) in [(1, 1, 1, 16, 16), (2, 3, 5, 16, 16), (3, 2, 10, 8, 8), (1, 4, 7, 1, 16), (2, 2, 3, 4, 16)]:
        if kind == "s8s8s32":
            l = rng.integers(-128, 128, (M1, K1, M0, k0), dtype=np.int8)
            r = rng.integers(-128, 128, (N1, K1, N0, k0), dtype=np.int8)
        else:
            l = rng.integers(-8, 8, (M1, K1, M0, k0)).astype(np.float16)
            r = rng.integers(-8, 8, (N1, K1, N0, k0)).astype(np.float16)
        got = oracle.mmt4d_port(t, l, r)
        for mode in (0, 1):
            assert (got == oracle.mmt4d_ref(t, l, r, cpu_mode=mode)).all(), (M1, N1, K1, M0, N0, mode)
        acc = rng.integers(-9, 9, got.shape).astype(got.dtype)
        assert (oracle.mmt4d_port(t, l, r, acc4=acc) == oracle.mmt4d_ref(t, l, r, acc4=acc)).all()


@needs_ref
def test_reference_has_architecture_tiles_for_the_configs(built):
    d0 = oracle.ref_lib().uk_chain_cpu_data0(1)
    if not (d0 >> 20) & 1:
        pytest.skip("host has no AVX-512")
    assert oracle.ref_has_arch_tile(oracle.TYPE_F16F16F32, 16, 16, 1)
    assert oracle.ref_has_arch_tile(oracle.TYPE_S8S8S32, 16, 16, 2)


@needs_ref
def test_int4_nibble_order_matches_reference_s8s4_tile(built):
    # iree_uk_mmt4d with type s8s4s32 (mmt4d_tile_generic.c:11-51) reads element 2i from the low
    # nibble of byte i. A one-hot left-hand side extracts each element of a packed row.
    import ctypes as C
    vals = np.array([-8, -7, -1, 0, 1, 5, 7, -3], np.int8)
    packed = workloads.pack_int4(vals[None, :])[0]          # 4 bytes
    K0 = 8
    lhs = np.eye(K0, dtype=np.int8).reshape(1, 1, K0, K0)    # [M1=1,K1=1,M0=8,K0=8]: row i0 selects k0
    rhs = packed.reshape(1, 1, 1, K0 // 2)                   # [N1=1,K1=1,N0=1,K0/2 bytes]
    out = np.zeros((1, 1, K0, 1), np.int32)
    flags = 0x0A | oracle.MMT4D_ALLOW_GENERIC
    oracle.ref_lib().uk_chain_mmt4d(lhs.ctypes.data_as(C.c_void_p), C.c_int64(K0 * K0),
                                    rhs.ctypes.data_as(C.c_void_p), C.c_int64(K0 // 2),
                                    out.ctypes.data_as(C.c_void_p), C.c_int64(K0), C.c_int64(1), C.c_int64(1),
                                    C.c_int64(1), C.c_int(K0), C.c_int(1), C.c_int(K0), C.c_uint32(flags), C.c_int(0))
    assert (out.reshape(-1) == vals).all()
    assert (oracle.unpack_i4(packed) == vals).all()
    assert (workloads.unpack_int4(packed[None, :])[0] == vals).all()


def test_subbyte_fixture_values(built):
    # tests/e2e/linalg/subbyte_to_fp.mlir: dense<[0..7]> : tensor<8xi4> extends to 0.0 .. 7.0.
    packed = workloads.pack_int4(np.arange(8, dtype=np.int8)[None, :])[0]
    assert (oracle.unpack_i4(packed) == np.arange(8, dtype=np.float32)).all()


def test_w4a16_port_against_numpy(built):
    rng = np.random.default_rng(11)
    M, N, K = 5, 48, 384
    a, wq, s = workloads.c4_w4a16(M, N=N, K=K, seed=11)
    got = oracle.w4a16(a, wq, s, threads=3)
    w = workloads.unpack_int4(wq).astype(np.float16).reshape(N, K // 128, 128)
    wd = (w * s[:, :, None]).astype(np.float16).reshape(N, K).astype(np.float64)
    want = a.astype(np.float64) @ wd.T
    np.testing.assert_allclose(got.astype(np.float64), want, rtol=2e-3, atol=2e-3)
    assert (oracle.w4a16(a, wq, s, threads=1) == got).all()   # threading does not change results


def test_requant_port(built):
    rng = np.random.default_rng(12)
    a, w, sa, sw = workloads.c3_w8a8(3, N=40, K=64, seed=12)
    acc = a.astype(np.int32) @ w.astype(np.int32)
    got = oracle.w8a8(a, w, sa, sw)
    want = ((acc.astype(np.float32) * sa[:, None]) * sw[None, :]).astype(np.float16)
    assert (got == want).all()


def test_f16_conversions_round_to_nearest_even(built):
    lib = oracle.port_lib()
    import ctypes as C
    lib.oracle_f32_to_f16.restype = C.c_uint16
    lib.oracle_f32_to_bf16.restype = C.c_uint16
    for v in (0.0, 1.0, -2.5, 65504.0, 65520.0, 1e-5, 0.1, 1.0009765625, 1.00048828125, 3.0e-8):
        assert lib.oracle_f32_to_f16(C.c_float(v)) == int(np.float32(v).astype(np.float16).view(np.uint16)), v
    x = np.float32(1.00390625)  # bf16 tie: rounds to even
    assert lib.oracle_f32_to_bf16(C.c_float(float(x))) == 0x3F80


def test_conversions_against_the_reference_routines(built):
    """The restatement's f16 / bf16 <-> f32 conversions (compiler _Float16) against the
    reference's own software routines (builtins/ukernel/common.h:664-790, compiled from the
    header where it lies) over all 65 536 16-bit patterns and a seeded f32 sample.

    They agree bit for bit on every value both can represent as a normal number. Where they
    differ is stated here and checked, so the difference cannot grow unnoticed:
      * 16 -> 32 bit: the reference routine returns zero for subnormal inputs (exponent field 0)
        and a canonical quiet NaN for every NaN; hardware conversion (and _Float16) keeps
        subnormals and NaN payloads.
      * 32 -> 16 bit: identical for 2^-14 <= |x| < 65520 and for zero and infinity. Below 2^-14
        the routine does not produce IEEE subnormals; in [65520, 131072) it leaves the exponent
        field saturated with mantissa bits set (a NaN pattern) where IEEE rounds to infinity.
    The reference's AVX-512 tile functions, which are what llvm-cpu runs on this host, convert in
    hardware (arch/x86_64/mmt4d_x86_64_avx512_base.c:68-131) like the restatement.
    """
    if not oracle.have_conv_ref():
        pytest.skip("oracle/_ref/libuk_conv.so not built (reference checkout absent)")
    patterns = np.arange(65536, dtype=np.uint16)
    for which, exp_shift, exp_max in (("f16_to_f32", 10, 31), ("bf16_to_f32", 7, 255)):
        mine = oracle.convert_port(which, patterns).view(np.uint32)
        ref = oracle.convert_ref(which, patterns).view(np.uint32)
        exp = (patterns >> exp_shift) & exp_max
        man = patterns & ((1 << exp_shift) - 1)
        special = ((exp == 0) & (man != 0)) | ((exp == exp_max) & (man != 0))   # subnormal or NaN
        assert (mine[~special] == ref[~special]).all(), which
        sub = (exp == 0) & (man != 0)
        assert (ref[sub] & 0x7fffffff == 0).all(), which + ": the reference routine flushes subnormals"
        assert (mine[sub] & 0x7fffffff != 0).all(), which + ": the restatement keeps them"
    rng = np.random.default_rng(0)
    f16_values = patterns.view(np.float16).astype(np.float32)
    finite = f16_values[np.isfinite(f16_values)]
    order = np.sort(finite)
    midpoints = ((order[:-1].astype(np.float64) + order[1:].astype(np.float64)) / 2).astype(np.float32)
    x = np.concatenate([rng.standard_normal(1 << 18).astype(np.float32) * s for s in (1e-6, 1e-4, 1e-2, 1, 100, 3e4, 1e5)]
                       + [finite, midpoints, np.array([0.0, -0.0, np.inf, -np.inf, 65504.0, 65519.99, 65520.0], np.float32)])
    mine, ref = oracle.convert_port("f32_to_f16", x), oracle.convert_ref("f32_to_f16", x)
    ax = np.abs(x)
    agree_zone = ((ax >= 2.0 ** -14) & (ax < 65520.0)) | (ax == 0) | np.isinf(x) | (ax >= 131072.0)
    assert (mine[agree_zone] == ref[agree_zone]).all()
    assert agree_zone.sum() > 1_000_000
    # every rounding tie inside the normal range is in the agree zone: both round to nearest even
    ties = midpoints[(np.abs(midpoints) >= 2.0 ** -14) & (np.abs(midpoints) < 65520.0)]
    assert (oracle.convert_port("f32_to_f16", ties) == oracle.convert_ref("f32_to_f16", ties)).all() and len(ties) > 60000
    differ = mine != ref
    assert ((ax[differ] < 2.0 ** -14) | ((ax[differ] >= 65520.0) & (ax[differ] < 131072.0))).all()
    # f32 -> bf16: no difference anywhere on the sample (NaN inputs excluded: payloads differ by design)
    assert (oracle.convert_port("f32_to_bf16", x) == oracle.convert_ref("f32_to_bf16", x)).all()


def test_conversion_difference_zone_is_outside_the_benchmark_data(built):
    """The value ranges the W4A16 / requant restatements are used on stay inside the zone where
    the restatement's conversions equal the reference's: dequantised weights f16(w * s) with
    |w| <= 8 and s in [0.005, 0.05] are either zero or at least 0.005 in magnitude, and outputs
    of the benchmark configurations are far below 65520."""
    a, wq, s = workloads.c4_w4a16(4, N=64, K=1024, seed=3)
    w = workloads.unpack_int4(wq).astype(np.float16).reshape(64, 8, 128)
    wd = (w * s[:, :, None]).astype(np.float16)
    mag = np.abs(wd.astype(np.float32))
    assert ((mag == 0) | (mag >= 2.0 ** -14)).all()
    out = oracle.w4a16(a, wq, s).astype(np.float32)
    assert np.abs(out).max() < 65520.0 and ((np.abs(out) == 0) | (np.abs(out) >= 2.0 ** -14)).mean() > 0.999


@pytest.mark.skipif(not oracle.have_ref(), reason="the reference's ukernels were not built")
@pytest.mark.parametrize("t,ldt,rdt,tile", [(oracle.TYPE_S16S16S32, np.int16, np.int16, (16, 16, 2)),
                                            (oracle.TYPE_S16S8S32, np.int16, np.int8, (4, 8, 3)),
                                            (oracle.TYPE_S16U4S32, np.int16, np.uint8, (1, 32, 8)),
                                            (oracle.TYPE_S8S4S32, np.int8, np.uint8, (4, 16, 2)),
                                            (oracle.TYPE_S8S4S32, np.int8, np.uint8, (3, 5, 6))])
def test_integer_mmt4d_types_restatement_equals_the_reference_ukernel(t, ldt, rdt, tile):
    """The s16 / 4-bit element types: the numpy restatement against iree_uk_mmt4d itself (generic tile
    functions and, where the host has them, the architecture-specific ones), with and without ACCUMULATE."""
    m0, n0, k0 = tile
    rng = np.random.default_rng(t)
    four_bit = t in (oracle.TYPE_S16U4S32, oracle.TYPE_S8S4S32)
    for (M, N, K) in [(1, 1, 1), (2, 3, 5), (5, 4, 17)]:
        li = np.iinfo(ldt)
        lhs = rng.integers(li.min, li.max + 1, (M, K, m0, k0)).astype(ldt)
        if four_bit:
            rhs = rng.integers(0, 256, (N, K, n0, k0 // 2)).astype(np.uint8)
        else:
            ri = np.iinfo(rdt)
            rhs = rng.integers(ri.min, ri.max + 1, (N, K, n0, k0)).astype(rdt)
        acc = rng.integers(-10 ** 6, 10 ** 6, (M, N, m0, n0)).astype(np.int32)
        for a in (None, acc):
            for mode in (0, 1):   # generic tile functions only / what the host CPU offers
                assert np.array_equal(oracle.mmt4d_int_types_port(t, lhs, rhs, a), oracle.mmt4d_ref(t, lhs, rhs, a, cpu_mode=mode))
