"""The decode entry point that allocates nothing (``iree_b200_w4a16_decode_noalloc``).

It exists for callers that cannot allocate device memory at dispatch time, so it carries its
split-K scratch inside the library instead of taking a workspace. This test calls it through
the C ABI, twice in a row on the same stream, and requires its output to equal the regular
decode entry point's (same kernel body, so bit-equal; the tolerance of the other W4A16 tests,
rtol = atol = 1e-2, is the bar). Collected last on purpose: a run that stops at the first
failure has then already run every other test.
"""
import ctypes as C
import os

import numpy as np
import pytest

import iree_b200 as ib
import oracle
from iree_b200 import workloads

pytestmark = pytest.mark.gpu
RTOL = ATOL = 1e-2


def _noalloc(ctx, a, wq, s, out, M, N, K, ldo, n_off):
    lib = ib.library()
    code = lib.iree_b200_w4a16_decode_noalloc(C.c_void_p(a.ptr), C.c_void_p(wq.ptr), C.c_void_p(s.ptr),
                                              C.c_void_p(out.ptr), C.c_int32(M), C.c_int32(N), C.c_int32(K),
                                              C.c_int32(ldo), C.c_int32(n_off), C.c_void_p(ctx.stream))
    return code


@pytest.mark.parametrize("M,N,K", [(16, 512, 8192), (5, 1024, 8192), (8, 256, 4096), (16, 11008, 4096)])
def test_noalloc_matches_regular_entry_point_twice(ctx, M, N, K):
    a, wq, s = workloads.c4_w4a16(M, N=N, K=K, seed=31)
    da, dw, ds = ctx.to_device(a), ctx.to_device(wq), ctx.to_device(s)
    ref_out, ws = ctx.alloc(M * N * 2), ctx.w4a16_workspace(N)
    p = ib.W4A16Params(M, N, K, 128, N, 0, ib.W4A16_DECODE, 0)
    ctx.w4a16(p, da, dw, ds, ref_out, ws)
    ctx.workspace_status(ws)
    want = ref_out.download(np.float16, (M, N))
    # and directly against the CPU oracle, so the check does not rest on the other entry point alone
    cpu = oracle.w4a16(a, wq, s, threads=os.cpu_count() or 1)
    out = ctx.alloc(M * N * 2)
    for call in range(2):                      # the second call reuses whatever the first left in the scratch
        out.fill(0x7E)
        assert _noalloc(ctx, da, dw, ds, out, M, N, K, N, 0) == 0, ib.last_error()
        got = out.download(np.float16, (M, N))
        np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32), rtol=RTOL, atol=ATOL,
                                   err_msg="call %d" % call)
        assert (got == want).all(), "call %d" % call
        np.testing.assert_allclose(got.astype(np.float32), cpu.astype(np.float32), rtol=RTOL, atol=ATOL,
                                   err_msg="call %d against the CPU oracle" % call)
    for x in (da, dw, ds, ref_out, ws, out):
        x.free()


def test_noalloc_writes_a_column_slice(ctx):
    M, N, K, ldo, off = 4, 64, 8192, 256, 128
    a, wq, s = workloads.c4_w4a16(M, N=N, K=K, seed=32)
    da, dw, ds = ctx.to_device(a), ctx.to_device(wq), ctx.to_device(s)
    out = ctx.alloc(M * ldo * 2).fill(0)
    assert _noalloc(ctx, da, dw, ds, out, M, N, K, ldo, off) == 0, ib.last_error()
    got = out.download(np.float16, (M, ldo))
    ref_out, ws = ctx.alloc(M * N * 2), ctx.w4a16_workspace(N)
    ctx.w4a16(ib.W4A16Params(M, N, K, 128, N, 0, ib.W4A16_DECODE, 0), da, dw, ds, ref_out, ws)
    want = ref_out.download(np.float16, (M, N))
    assert (got[:, off:off + N] == want).all()
    assert not got[:, :off].any() and not got[:, off + N:].any()
    for x in (da, dw, ds, ref_out, ws, out):
        x.free()


def test_noalloc_rejects_sizes_beyond_its_scratch(ctx):
    d = ctx.alloc(256)
    big = 32768 + 16
    assert _noalloc(ctx, d, d, d, d, 1, big, 256, big, 0) == 11            # OUT_OF_RANGE
    assert "32768" in ib.last_error()
    assert _noalloc(ctx, d, d, d, d, 17, 16, 256, 16, 0) == 3              # INVALID_ARGUMENT: M > 16
    assert _noalloc(ctx, d, d, d, d, 1, 16, 100, 16, 0) == 3               # K not a multiple of 256
    assert _noalloc(ctx, d, d, d, d, 1, 16, 16384 + 256, 16, 0) == 3       # K above 16384
    assert _noalloc(ctx, d, d, d, d, 1, 16400, 16384, 16400, 0) == 11      # four K slices: half the columns at most
    d.free()


def test_noalloc_refuses_misaligned_operands_and_reports_status(ctx):
    """A caller that sub-allocates from its own pool may hand in a pointer at an 8-byte offset; the
    kernel would fault on it, so the entry point has to refuse it with a status (nothing runs)."""
    class Shifted:                                                       # stands in for a pool sub-allocation
        def __init__(self, ptr):
            self.ptr = ptr
    d = ctx.alloc(4096)
    odd = Shifted(d.ptr + 8)
    assert _noalloc(ctx, odd, d, d, d, 1, 16, 256, 16, 0) == 3 and "16-byte" in ib.last_error()
    assert _noalloc(ctx, d, odd, d, d, 1, 16, 256, 16, 0) == 3
    assert _noalloc(ctx, d, d, odd, d, 1, 16, 256, 16, 0) == 3
    # no dispatch of this process has given up a wait: the shared status record reads OK
    ctx.synchronize()
    assert ib.library().iree_b200_w4a16_decode_noalloc_status() == 0, ib.last_error()
    d.free()
