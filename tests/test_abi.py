"""Host-side checks that need no GPU: the C-ABI library loads, exports every symbol the header
declares, builds and verifies ExecutableDef flatbuffers the way the reference's loader does,
validates arguments, and reports UNAVAILABLE (never a CPU result) without a device."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import iree_b200
from iree_b200 import runtime

HEADER = os.path.join(os.path.dirname(os.path.dirname(__file__)), "include", "iree_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(iree_(?:hal_)?b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built):
    lib = iree_b200.library()
    names = declared_functions()
    assert len(names) >= 35
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_cubin_was_built_for_sm_100a_only(built):
    data = open(iree_b200.cubin_path(), "rb").read()
    assert data[:4] == b"\x7fELF"
    for export in ("b200_matmul_f16_f16", "b200_matmul_i8_i32", "b200_matmul_i8_requant_f16",
                   "b200_encode_tensormaps", "b200_matmul_generic_f16_f16"):
        assert export.encode() in data, export


def _build_def(names, blocks, smem, image):
    lib = iree_b200.library()
    arr = (C.c_char_p * len(names))(*[n.encode() for n in names])
    b = np.asarray(blocks, np.uint32).reshape(-1)
    s = np.asarray(smem, np.uint32)
    size = C.c_size_t()
    code = lib.iree_b200_executable_def_build(C.c_int32(len(names)), arr, b.ctypes.data_as(C.c_void_p),
                                              s.ctypes.data_as(C.c_void_p), image, C.c_size_t(len(image)), None,
                                              C.c_size_t(0), C.byref(size))
    assert code == 0
    buf = C.create_string_buffer(size.value)
    code = lib.iree_b200_executable_def_build(C.c_int32(len(names)), arr, b.ctypes.data_as(C.c_void_p),
                                              s.ctypes.data_as(C.c_void_p), image, C.c_size_t(len(image)), buf,
                                              C.c_size_t(size.value), C.byref(size))
    assert code == 0
    return buf.raw[:size.value]


def test_executable_def_layout(built):
    image = b"\x7fELF" + bytes(range(200)) + b"\x00\x01binary\x00tail"
    fb = _build_def(["k_one", "k_two"], [[64, 1, 1], [256, 2, 1]], [0, 4096], image)
    # file identifier of runtime/src/iree/schemas/cuda_executable_def.fbs
    assert fb[4:8] == b"CUDA"
    root = int.from_bytes(fb[0:4], "little")
    vt = root - int.from_bytes(fb[root:root + 4], "little", signed=True)
    vt_size = int.from_bytes(fb[vt:vt + 2], "little")
    assert vt_size >= 12
    fields = [int.from_bytes(fb[vt + 4 + 2 * i: vt + 6 + 2 * i], "little") for i in range((vt_size - 4) // 2)]

    def vec(field):
        pos = root + fields[field]
        pos += int.from_bytes(fb[pos:pos + 4], "little")
        return pos, int.from_bytes(fb[pos:pos + 4], "little")

    pos, n = vec(0)
    names = []
    for i in range(n):
        slot = pos + 4 + 4 * i
        s = slot + int.from_bytes(fb[slot:slot + 4], "little")
        ln = int.from_bytes(fb[s:s + 4], "little")
        names.append(fb[s + 4:s + 4 + ln].decode())
    assert names == ["k_one", "k_two"]
    pos, n = vec(1)
    assert n == 2 and np.frombuffer(fb[pos + 4:pos + 28], np.uint32).tolist() == [64, 1, 1, 256, 2, 1]
    pos, n = vec(2)
    assert n == 2 and np.frombuffer(fb[pos + 4:pos + 12], np.uint32).tolist() == [0, 4096]
    pos, n = vec(3)
    assert n == len(image) and fb[pos + 4:pos + 4 + n] == image      # binary-safe: explicit length


def _create(fb, fmt=b"PTXE"):
    lib = iree_b200.library()
    exe = C.c_void_p()
    code = lib.iree_hal_b200_executable_create(None, fmt, fb, C.c_size_t(len(fb)), C.byref(exe))
    return code, iree_b200.last_error()


def test_executable_loader_rejects_what_the_reference_rejects(built):
    # rules of runtime/src/iree/hal/drivers/cuda/native_executable.c:55-110 and the format gate
    # of nop_executable_cache.c:76-82; all decided before any device is touched
    good = _build_def(["k"], [[32, 1, 1]], [0], b"image")
    code, msg = _create(good, b"ELF")
    assert code == 5 and "format" in msg                                    # NOT_FOUND
    code, msg = _create(b"\x00" * 8)
    assert code == 3                                                        # INVALID_ARGUMENT
    code, msg = _create(good[:4] + b"XXXX" + good[8:])
    assert code == 3 and "CUDA" in msg
    code, msg = _create(_build_def([""], [[32, 1, 1]], [0], b"image"))
    assert code == 3 and "no name" in msg
    code, msg = _create(_build_def([], [], [], b"image"))
    assert code == 3 and "no block sizes" in msg
    code, msg = _create(_build_def(["k"], [[32, 1, 1]], [0], b""))
    assert code == 3 and "no PTX image" in msg
    code, msg = _create(good[: len(good) // 2])
    assert code == 3
    # a well-formed container passes verification and then needs a device
    code, msg = _create(good)
    assert code == 3 and "device is NULL" in msg


def test_command_buffer_argument_checks(built):
    lib = iree_b200.library()
    assert lib.iree_hal_b200_command_buffer_push_constants(None, C.c_size_t(0), None, C.c_size_t(0)) == 3
    assert lib.iree_hal_b200_command_buffer_dispatch(None, None, 0, 0, 0, 1, 1, 1) == 3
    assert lib.iree_hal_b200_channel_create(None, None, C.c_size_t(0), 0, 1, C.byref(C.c_void_p())) == 3
    assert lib.iree_b200_matmul(None, None, None, None, None, None, None, None) == 3


@pytest.mark.parametrize("M,N,K", [(4096, 28672, 8192), (2048, 11008, 4096), (1100, 4400, 12288), (256, 2048, 32768),
                                   (5000, 40000, 4096)])
def test_host_call_plan_covers_the_result_once_and_uploads_before_use(built, M, N, K):
    """The units of the host-buffer W4A16 call (planned without a device): their rectangles tile the
    [M, N] result exactly once, every rectangle only needs rows and columns whose upload precedes it, every
    operand block goes up exactly once, and block edges keep the kernel's alignment (256 rows / columns)."""
    p = runtime.W4A16Params(M, N, K, 128, N, 0, runtime.W4A16_AUTO, 0)
    units = runtime.Context.w4a16_host_plan(p)
    assert 2 <= len(units) <= 11
    covered = np.zeros((M, N), np.uint8)
    rows_up = np.zeros(M, bool)
    cols_up = np.zeros(N, bool)
    for (r0, rows, c0, cols, new_rows, new_cols) in units:
        assert rows > 0 and cols > 0 and r0 % 256 == 0 and c0 % 256 == 0
        if new_rows:
            assert not rows_up[r0:r0 + rows].any()
            rows_up[r0:r0 + rows] = True
        if new_cols:
            assert not cols_up[c0:c0 + cols].any()
            cols_up[c0:c0 + cols] = True
        assert new_rows or new_cols
        assert rows_up[r0:r0 + rows].all() and cols_up[c0:c0 + cols].all()
        covered[r0:r0 + rows, c0:c0 + cols] += 1
    assert (covered == 1).all() and rows_up.all() and cols_up.all()
    # the first result leaves after a part of the operands has arrived (a fifth at most on the large shapes)
    first = units[0]
    if M >= 2048:
        assert first[1] * K * 2 + first[3] * (K // 2 + K // 64) <= 0.2 * (M * K * 2 + N * (K // 2 + K // 64))


def test_host_call_plan_leaves_small_and_unsuitable_products_alone(built):
    plan = runtime.Context.w4a16_host_plan
    assert plan(runtime.W4A16Params(16, 28672, 8192, 128, 28672, 0, runtime.W4A16_AUTO, 0)) == []      # few rows
    assert plan(runtime.W4A16Params(512, 2048, 1024, 128, 2048, 0, runtime.W4A16_AUTO, 0)) == []        # small
    assert plan(runtime.W4A16Params(4096, 28676, 8192, 128, 28676, 0, runtime.W4A16_AUTO, 0)) == []     # N % 8
    assert plan(runtime.W4A16Params(4096, 28672, 8192, 128, 28672, 0, runtime.W4A16_GEMM, 0)) == []     # explicit variant
    assert plan(runtime.W4A16Params(4096, 14336, 8192, 128, 28672, 14336, runtime.W4A16_AUTO, 0)) == [] # a column slice
    with pytest.raises(ValueError):
        plan(runtime.W4A16Params(4096, 28672, 100, 128, 28672, 0, runtime.W4A16_AUTO, 0))


def _has_gpu():
    try:
        c = iree_b200.Context(0)
        c.close()
        return True
    except iree_b200.IreeB200Error:
        return False


def test_no_cpu_fallback_without_a_device(built):
    if _has_gpu():
        pytest.skip("a GPU is present")
    with pytest.raises(iree_b200.IreeB200Error) as e:
        iree_b200.Context(0)
    assert e.value.code_name == "UNAVAILABLE"
    dev = C.c_void_p()
    assert iree_b200.library().iree_hal_b200_device_create(0, C.byref(dev)) == 14


def test_product_never_imports_the_oracle():
    root = os.path.dirname(os.path.dirname(__file__))
    for dirpath, _, files in os.walk(os.path.join(root, "iree_b200")):
        for f in files:
            if f.endswith((".py", ".cc", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text and "liboracle" not in text, f
