"""ctypes front end of the CPU oracle. TEST INFRASTRUCTURE ONLY.

Only tests/, ``__graft_entry__.smoke()`` and the CPU legs of ``bench.py`` may import this
package; the shipped package ``iree_b200`` never does.

Two checkers live here:

* ``port``  -- ``liboracle.so`` built from ``contraction_oracle.c``: a plain-C restatement of
  the reference's pack / mmt4d / unpack chain and of the linalg bodies of the fused
  dequant-int4 and requant dispatches.
* ``ref``   -- ``_ref/libuk_chain.so``: the reference's own ``iree_uk_pack`` /
  ``iree_uk_mmt4d`` / ``iree_uk_unpack`` compiled from the reference sources, chained by
  ``uk_chain.c``. Present whenever ``make -C oracle`` ran with the reference checkout
  available; the built files travel with the tree.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

TYPE_F32F32F32 = 1  # IREE_UK_FLAG_MMT4D_TYPE_* (builtins/ukernel/exported_bits.h:29-42)
TYPE_S8S8S32 = 2
TYPE_F16F16F32 = 3
TYPE_BF16BF16F32 = 5
TYPE_S16S16S32, TYPE_S16U4S32, TYPE_S16S8S32, TYPE_S8S4S32 = 7, 8, 9, 10   # the reference's ukernel only (mmt4d_ref)

PACK_F32, PACK_I8, PACK_I32, PACK_F16, PACK_BF16 = 1, 2, 3, 4, 5  # exported_bits.h:56-62
TRANSPOSE_INNER, TRANSPOSE_OUTER = 0x100, 0x200
MMT4D_ACCUMULATE, MMT4D_ALLOW_GENERIC, MMT4D_SKIP_ROUNDINGS = 0x100, 0x200, 0x400

_IN_DTYPE = {TYPE_F32F32F32: np.float32, TYPE_S8S8S32: np.int8, TYPE_F16F16F32: np.float16,
             TYPE_BF16BF16F32: np.uint16}
_ACC_DTYPE = {TYPE_F32F32F32: np.float32, TYPE_S8S8S32: np.int32, TYPE_F16F16F32: np.float32,
              TYPE_BF16BF16F32: np.float32, TYPE_S16S16S32: np.int32, TYPE_S16U4S32: np.int32,
              TYPE_S16S8S32: np.int32, TYPE_S8S4S32: np.int32}


def build(verbose: bool = False) -> None:
    """Compile liboracle.so and, when the reference checkout is present, oracle/_ref."""
    out = subprocess.run(["make", "-C", _HERE], capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + out.stdout + out.stderr)
    if verbose:
        print(out.stdout)


_port = None
_ref = None


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def port_lib():
    global _port
    if _port is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        _port = C.CDLL(path)
        _port.oracle_matmul_data_tiled.restype = C.c_int
        _port.oracle_w4a16.restype = C.c_int
    return _port


def have_ref() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libuk_chain.so"))


def ref_lib():
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libuk_chain.so")
        if not os.path.exists(path):
            build()
        _ref = C.CDLL(path)
        _ref.uk_chain_matmul.restype = C.c_int
        _ref.uk_chain_cpu_data0.restype = C.c_uint64
        _ref.uk_chain_mmt4d_info.restype = C.c_uint32
    return _ref


_conv = None


def have_conv_ref() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libuk_conv.so"))


def conv_ref_lib():
    """The reference's software f16 / bf16 conversions (builtins/ukernel/common.h:664-790)."""
    global _conv
    if _conv is None:
        path = os.path.join(_HERE, "_ref", "libuk_conv.so")
        if not os.path.exists(path):
            build()
        _conv = C.CDLL(path)
    return _conv


_CONV = {"f16_to_f32": (0, np.uint16, np.float32), "f32_to_f16": (1, np.float32, np.uint16),
         "bf16_to_f32": (2, np.uint16, np.float32), "f32_to_bf16": (3, np.float32, np.uint16)}


def convert_port(which: str, x: np.ndarray) -> np.ndarray:
    """The restatement's conversion `which` over an array (raw 16-bit patterns as uint16)."""
    code, din, dout = _CONV[which]
    x = np.ascontiguousarray(x, din)
    out = np.empty(x.shape, dout)
    port_lib().oracle_convert_n(C.c_int(code), _ptr(x), _ptr(out), C.c_int64(x.size))
    return out


def convert_ref(which: str, x: np.ndarray) -> np.ndarray:
    """The reference's own conversion `which` over an array."""
    _, din, dout = _CONV[which]
    x = np.ascontiguousarray(x, din)
    out = np.empty(x.shape, dout)
    getattr(conv_ref_lib(), "uk_conv_%s_n" % which)(_ptr(x), _ptr(out), C.c_int64(x.size))
    return out


# --------------------------------------------------------------------------------------
# Tile choice of the llvm-cpu data-tiling on x86-64 (restated from
# compiler/src/iree/compiler/Codegen/Common/CPU/CPUMaterializeEncodingPass.cpp:168-277 and
# the narrow-M rule :284-377 / GlobalOptimization/SetEncoding.cpp:101-142).
# --------------------------------------------------------------------------------------
def x86_64_tile(mmt4d_type: int, M: int, N: int, avx512: bool = True, vnni: bool = True):
    if mmt4d_type == TYPE_S8S8S32:
        m0, n0, k0 = (16, 16, 2) if avx512 else (8, 8, 2)
    elif mmt4d_type == TYPE_BF16BF16F32:
        m0, n0, k0 = (16, 16, 2) if avx512 else (8, 8, 1)
    else:
        m0, n0, k0 = (16, 16, 1) if avx512 else (8, 8, 1)
    # A statically narrow M (< 16) shrinks M0 to the next power of two >= M.
    if 0 < M < 16:
        p = 1
        while p < M:
            p *= 2
        m0 = min(m0, p)
    return m0, n0, k0


def matmul_narrow_sizes(M: int, N: int):
    """(narrow_M, narrow_N) as GlobalOptimization/SetEncoding.cpp:101-142 records them on the
    encoding: a static size below 16 is narrow; when both are, only the smaller is kept (M on a tie)."""
    nm = M if 0 < M < 16 else None
    nn = N if 0 < N < 16 else None
    if nm is not None and nn is not None:
        if nm <= nn:
            nn = None
        else:
            nm = None
    return nm, nn


def is_narrow_n_result(M: int, N: int) -> bool:
    """Codegen/Common/EncodingUtils.cpp:206-213: narrow N set and (narrow M unset or larger). The
    materialisation then swaps the operands and computes the transposed product, so that the narrow
    dimension becomes the mmt4d's M (MaterializeEncodingIntoPackUnPack.cpp:330-399)."""
    nm, nn = matmul_narrow_sizes(M, N)
    return nn is not None and (nm is None or nm > nn)


def _as_in(x, t):
    x = np.ascontiguousarray(x)
    if t == TYPE_BF16BF16F32:
        assert x.dtype == np.uint16, "bf16 travels as raw uint16 bit patterns"
    else:
        assert x.dtype == _IN_DTYPE[t], (x.dtype, t)
    return x


def matmul_port(t: int, lhs, rhs, tile=None, acc=None) -> np.ndarray:
    """pack -> mmt4d -> unpack through the plain-C restatement. Returns i32 / f32 [M,N]."""
    lhs, rhs = _as_in(lhs, t), _as_in(rhs, t)
    M, K = lhs.shape
    K2, N = rhs.shape
    assert K == K2
    if tile is None and is_narrow_n_result(M, N):
        # narrow N: out^T[N, M] = rhs^T[N, K] x lhs^T[K, M], tiles chosen for the swapped problem
        swapped = matmul_port(t, np.ascontiguousarray(rhs.T), np.ascontiguousarray(lhs.T), tile=x86_64_tile(t, N, M),
                              acc=None if acc is None else np.ascontiguousarray(np.asarray(acc).T))
        return np.ascontiguousarray(swapped.T)
    m0, n0, k0 = tile or x86_64_tile(t, M, N)
    out = np.zeros((M, N), _ACC_DTYPE[t]) if acc is None else np.ascontiguousarray(acc).copy()
    rc = port_lib().oracle_matmul_data_tiled(C.c_int(t), C.c_int64(M), C.c_int64(N), C.c_int64(K),
                                             _ptr(lhs), _ptr(rhs), _ptr(out), C.c_int(m0), C.c_int(n0),
                                             C.c_int(k0), C.c_int(0 if acc is None else 1))
    assert rc == 0
    return out


def matmul_naive(t: int, lhs, rhs, acc=None) -> np.ndarray:
    lhs, rhs = _as_in(lhs, t), _as_in(rhs, t)
    M, K = lhs.shape
    _, N = rhs.shape
    out = np.zeros((M, N), _ACC_DTYPE[t]) if acc is None else np.ascontiguousarray(acc).copy()
    port_lib().oracle_matmul_naive(C.c_int(t), C.c_int64(M), C.c_int64(N), C.c_int64(K), _ptr(lhs),
                                   _ptr(rhs), _ptr(out), C.c_int(0 if acc is None else 1))
    return out


def matmul_ref(t: int, lhs, rhs, tile=None, acc=None, cpu_mode: int = 1, threads: int = 1,
               times=None) -> np.ndarray:
    """The same chain through the reference's own ukernels (oracle/_ref)."""
    lhs, rhs = _as_in(lhs, t), _as_in(rhs, t)
    M, K = lhs.shape
    K2, N = rhs.shape
    assert K == K2
    m0, n0, k0 = tile or x86_64_tile(t, M, N)
    out = np.zeros((M, N), _ACC_DTYPE[t]) if acc is None else np.ascontiguousarray(acc).copy()
    tbuf = (C.c_double * 4)()
    rc = ref_lib().uk_chain_matmul(C.c_uint32(t), C.c_int64(M), C.c_int64(N), C.c_int64(K), _ptr(lhs),
                                   _ptr(rhs), _ptr(out), C.c_int(m0), C.c_int(n0), C.c_int(k0),
                                   C.c_int(0 if acc is None else 1), C.c_int(cpu_mode),
                                   C.c_int(threads), tbuf)
    assert rc == 0
    if times is not None:
        times[:] = list(tbuf)
    return out


def truncf(x: np.ndarray, to_bf16: bool = False) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    port_lib().oracle_truncf(_ptr(x), _ptr(out), C.c_int64(x.size), C.c_int(1 if to_bf16 else 0))
    return out if to_bf16 else out.view(np.float16)


def requant_f16(acc: np.ndarray, a_scale: np.ndarray, w_scale: np.ndarray) -> np.ndarray:
    acc = np.ascontiguousarray(acc, np.int32)
    a_scale = np.ascontiguousarray(a_scale, np.float32)
    w_scale = np.ascontiguousarray(w_scale, np.float32)
    M, N = acc.shape
    assert a_scale.shape == (M,) and w_scale.shape == (N,)
    out = np.empty((M, N), np.uint16)
    port_lib().oracle_requant_f16(_ptr(acc), _ptr(a_scale), _ptr(w_scale), _ptr(out), C.c_int64(M),
                                  C.c_int64(N))
    return out.view(np.float16)


def w8a8(a_i8, w_i8, a_scale, w_scale, use_ref: bool = False, threads: int = 1) -> np.ndarray:
    """W8A8 dispatch pair: data-tiled i8 matmul, then the requant consumer."""
    acc = (matmul_ref(TYPE_S8S8S32, a_i8, w_i8, threads=threads) if use_ref
           else matmul_port(TYPE_S8S8S32, a_i8, w_i8))
    return requant_f16(acc, a_scale, w_scale)


def w4a16(a_f16, wq_u8, scales_f16, group: int = 128, threads: int = 1) -> np.ndarray:
    """Fused dequant-int4 + grouped contraction. wq_u8 is [N, K/2] packed nibbles."""
    a = np.ascontiguousarray(a_f16, np.float16)
    wq = np.ascontiguousarray(wq_u8, np.uint8)
    s = np.ascontiguousarray(scales_f16, np.float16)
    M, K = a.shape
    N = wq.shape[0]
    assert wq.shape == (N, K // 2) and s.shape == (N, K // group)
    out = np.empty((M, N), np.uint16)
    rc = port_lib().oracle_w4a16(_ptr(a), _ptr(wq), _ptr(s), _ptr(out), C.c_int64(M), C.c_int64(N),
                                 C.c_int64(K), C.c_int(group), C.c_int(threads))
    assert rc == 0
    return out.view(np.float16)


def unpack_i4(bytes_u8: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(bytes_u8, np.uint8).reshape(-1)
    out = np.empty(b.size * 2, np.float32)
    port_lib().oracle_unpack_i4(_ptr(b), C.c_int64(b.size * 2), _ptr(out))
    return out


# Raw single-op entry points (used to pin each restated op against the reference ukernel).
def pack_port(x, tiles, transpose_inner=False, transpose_outer=False, padding=0):
    x = np.ascontiguousarray(x)
    o0, o1, o2, o3 = tiles
    out = np.zeros((o0, o1, o2, o3), x.dtype)
    port_lib().oracle_pack(_ptr(x), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]), C.c_int64(x.shape[1]),
                           _ptr(out), C.c_int64(o0), C.c_int64(o1), C.c_int64(o2), C.c_int64(o3),
                           C.c_int64(o1 * o2 * o3), C.c_int(x.dtype.itemsize), C.c_int(int(transpose_inner)),
                           C.c_int(int(transpose_outer)), C.c_uint64(padding))
    return out


_PACK_FLAG = {np.dtype(np.float32): PACK_F32, np.dtype(np.int8): PACK_I8, np.dtype(np.int32): PACK_I32,
              np.dtype(np.float16): PACK_F16}


def pack_ref(x, tiles, transpose_inner=False, transpose_outer=False, padding=0, cpu_mode=1):
    x = np.ascontiguousarray(x)
    o0, o1, o2, o3 = tiles
    out = np.zeros((o0, o1, o2, o3), x.dtype)
    flags = _PACK_FLAG[x.dtype] | (TRANSPOSE_INNER if transpose_inner else 0) | (
        TRANSPOSE_OUTER if transpose_outer else 0)
    ref_lib().uk_chain_pack(_ptr(x), C.c_int64(x.shape[1]), _ptr(out), C.c_int64(o1 * o2 * o3),
                            C.c_int64(x.shape[0]), C.c_int64(x.shape[1]), C.c_int64(o0), C.c_int64(o1),
                            C.c_int64(o2), C.c_int64(o3), C.c_uint64(padding), C.c_uint32(flags),
                            C.c_int(cpu_mode))
    return out


def unpack_port(x4, out_shape, transpose_inner=False, transpose_outer=False):
    x4 = np.ascontiguousarray(x4)
    i0, i1, i2, i3 = x4.shape
    out = np.zeros(out_shape, x4.dtype)
    port_lib().oracle_unpack(_ptr(x4), C.c_int64(i0), C.c_int64(i1), C.c_int64(i2), C.c_int64(i3),
                             C.c_int64(i1 * i2 * i3), _ptr(out), C.c_int64(out_shape[0]),
                             C.c_int64(out_shape[1]), C.c_int64(out_shape[1]), C.c_int(x4.dtype.itemsize),
                             C.c_int(int(transpose_inner)), C.c_int(int(transpose_outer)))
    return out


def unpack_ref(x4, out_shape, transpose_inner=False, transpose_outer=False, cpu_mode=1):
    x4 = np.ascontiguousarray(x4)
    i0, i1, i2, i3 = x4.shape
    out = np.zeros(out_shape, x4.dtype)
    flags = {np.dtype(np.float32): 1, np.dtype(np.int32): 3, np.dtype(np.float16): 4}[x4.dtype]
    flags |= (TRANSPOSE_INNER if transpose_inner else 0) | (TRANSPOSE_OUTER if transpose_outer else 0)
    ref_lib().uk_chain_unpack(_ptr(x4), C.c_int64(i1 * i2 * i3), _ptr(out), C.c_int64(out_shape[1]),
                              C.c_int64(i0), C.c_int64(i1), C.c_int64(i2), C.c_int64(i3),
                              C.c_int64(out_shape[0]), C.c_int64(out_shape[1]), C.c_uint32(flags),
                              C.c_int(cpu_mode))
    return out


def mmt4d_port(t, lhs4, rhs4, acc4=None):
    lhs4, rhs4 = np.ascontiguousarray(lhs4), np.ascontiguousarray(rhs4)
    M1, K1, M0, K0 = lhs4.shape
    N1, _, N0, _ = rhs4.shape
    out = (np.zeros((M1, N1, M0, N0), _ACC_DTYPE[t]) if acc4 is None
           else np.ascontiguousarray(acc4).copy())
    port_lib().oracle_mmt4d(C.c_int(t), _ptr(lhs4), C.c_int64(K1 * M0 * K0), _ptr(rhs4),
                            C.c_int64(K1 * N0 * K0), _ptr(out), C.c_int64(N1 * M0 * N0), C.c_int64(M1),
                            C.c_int64(N1), C.c_int64(K1), C.c_int(M0), C.c_int(N0), C.c_int(K0),
                            C.c_int(0 if acc4 is None else 1))
    return out


def mmt4d_ref(t, lhs4, rhs4, acc4=None, cpu_mode=1):
    lhs4, rhs4 = np.ascontiguousarray(lhs4), np.ascontiguousarray(rhs4)
    M1, K1, M0, K0 = lhs4.shape
    N1, _, N0, _ = rhs4.shape
    out = (np.zeros((M1, N1, M0, N0), _ACC_DTYPE[t]) if acc4 is None
           else np.ascontiguousarray(acc4).copy())
    flags = t | MMT4D_ALLOW_GENERIC | MMT4D_SKIP_ROUNDINGS | (0 if acc4 is None else MMT4D_ACCUMULATE)
    ref_lib().uk_chain_mmt4d(_ptr(lhs4), C.c_int64(K1 * M0 * K0), _ptr(rhs4), C.c_int64(K1 * N0 * K0),
                             _ptr(out), C.c_int64(N1 * M0 * N0), C.c_int64(M1), C.c_int64(N1),
                             C.c_int64(K1), C.c_int(M0), C.c_int(N0), C.c_int(K0), C.c_uint32(flags),
                             C.c_int(cpu_mode))
    return out


def ref_has_arch_tile(t, m0, n0, k0, cpu_mode=1) -> bool:
    flags = t | MMT4D_SKIP_ROUNDINGS
    return bool(ref_lib().uk_chain_mmt4d_info(C.c_int(m0), C.c_int(n0), C.c_int(k0), C.c_uint32(flags),
                                              C.c_int(cpu_mode)) & 1)


def mmt4d_int_types_port(t, lhs4, rhs4, acc4=None):
    """numpy restatement of the reference's generic tile functions for the s16 / 4-bit mmt4d types
    (builtins/ukernel/mmt4d_tile_generic.c:11-180): int32 accumulation with wrap-around; a 4-bit
    right-hand side holds two reduction elements per byte, low nibble first, unsigned for u4
    (S16U4S32) and sign-extended for s4 (S8S4S32). Pinned against the reference's own ukernel in
    tests/test_oracle.py."""
    lhs4, rhs4 = np.asarray(lhs4), np.asarray(rhs4)
    if t in (TYPE_S16U4S32, TYPE_S8S4S32):
        lo, hi = (rhs4 & 0xF).astype(np.int64), (rhs4 >> 4).astype(np.int64)
        if t == TYPE_S8S4S32:
            lo, hi = np.where(lo >= 8, lo - 16, lo), np.where(hi >= 8, hi - 16, hi)
        r = np.stack([lo, hi], axis=-1).reshape(rhs4.shape[:-1] + (rhs4.shape[-1] * 2,))
    else:
        r = rhs4.astype(np.int64)
    total = np.einsum("mkac,nkbc->mnab", lhs4.astype(np.int64), r)
    if acc4 is not None:
        total = total + np.asarray(acc4).astype(np.int64)
    return (total & 0xFFFFFFFF).astype(np.uint32).view(np.int32)
