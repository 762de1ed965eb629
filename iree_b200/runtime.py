"""ctypes host side of ``libiree_b200.so`` (declared in ``include/iree_b200.h``).

Mirrors the reference's runtime surface for one dispatch: a context owns the device, the
loaded executable (an ``ExecutableDef`` flatbuffer wrapped around the sm_100a cubin) and a
stream command buffer; operators push constants, bind buffers and dispatch. Failures raise
:class:`IreeB200Error` carrying the reference's status code name.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

KIND_F16, KIND_BF16, KIND_I8 = 0, 1, 2
EPILOGUE_CAST, EPILOGUE_ACCUMULATOR, EPILOGUE_REQUANT_F16 = 0, 1, 2
RHS_KN, RHS_NK = 0, 1
FLAG_FORCE_GENERIC, FLAG_DEVICE_TENSORMAPS, FLAG_PAIR_CTAS, FLAG_SINGLE_CTA, FLAG_SPLIT_K = 1, 2, 4, 8, 16
WORKSPACE_BYTES = 512

_STATUS_NAMES = {0: "OK", 1: "CANCELLED", 2: "UNKNOWN", 3: "INVALID_ARGUMENT", 4: "DEADLINE_EXCEEDED",
                 5: "NOT_FOUND", 6: "ALREADY_EXISTS", 7: "PERMISSION_DENIED", 8: "RESOURCE_EXHAUSTED",
                 9: "FAILED_PRECONDITION", 10: "ABORTED", 11: "OUT_OF_RANGE", 12: "UNIMPLEMENTED",
                 13: "INTERNAL", 14: "UNAVAILABLE", 15: "DATA_LOSS", 16: "UNAUTHENTICATED"}


class IreeB200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        self.code = code
        self.code_name = _STATUS_NAMES.get(code, str(code))
        super().__init__("%s: %s" % (self.code_name, message))


class MatmulParams(C.Structure):
    _fields_ = [("kind", C.c_int32), ("epilogue", C.c_int32), ("M", C.c_int32), ("N", C.c_int32),
                ("K", C.c_int32), ("batch", C.c_int32), ("rhs_layout", C.c_int32), ("tile_n", C.c_int32),
                ("flags", C.c_int32)]


class W4A16Params(C.Structure):
    _fields_ = [("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32), ("group_size", C.c_int32),
                ("ldo", C.c_int32), ("n_offset", C.c_int32), ("variant", C.c_int32), ("tile_n", C.c_int32)]


W4A16_AUTO, W4A16_DECODE, W4A16_GEMM, W4A16_GENERIC, W4A16_GEMM_WT, W4A16_DECODE_TC = 0, 1, 2, 3, 4, 5


class _Binding(C.Structure):
    _fields_ = [("binding", C.c_uint32), ("device_ptr", C.c_void_p)]


def library_path() -> str:
    return os.path.join(_HERE, "libiree_b200.so")


def cubin_path() -> str:
    return os.path.join(_HERE, "csrc", "b200_contraction.cubin")


_lib = None


def library():
    """Loads libiree_b200.so. Raises if it was not built: there is no fallback."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise IreeB200Error(14, "libiree_b200.so is not built (run `python -m iree_b200.build`)")
        lib = C.CDLL(path)
        lib.iree_b200_last_error.restype = C.c_char_p
        lib.iree_hal_b200_device_stream.restype = C.c_void_p
        lib.iree_b200_context_device.restype = C.c_void_p
        lib.iree_b200_context_executable.restype = C.c_void_p
        lib.iree_b200_context_command_buffer.restype = C.c_void_p
        lib.iree_hal_b200_command_buffer_launch_count.restype = C.c_uint64
        lib.iree_b200_w4a16_workspace_bytes.restype = C.c_size_t
        lib.iree_b200_uk_mmt4d_workspace_bytes.restype = C.c_size_t
        _lib = lib
    return _lib


def last_error() -> str:
    return library().iree_b200_last_error().decode()


def check(code: int) -> None:
    if code != 0:
        raise IreeB200Error(code, last_error())


def _vp(x) -> C.c_void_p:
    if x is None:
        return C.c_void_p(0)
    if isinstance(x, DeviceBuffer):
        return C.c_void_p(x.ptr)
    if isinstance(x, int):
        return C.c_void_p(x)
    if isinstance(x, np.ndarray):
        return C.c_void_p(x.ctypes.data)
    if hasattr(x, "data_ptr"):  # a torch tensor on this device
        return C.c_void_p(x.data_ptr())
    raise TypeError(type(x))


class DeviceBuffer:
    """A raw device allocation (what a HAL buffer resolves to before a launch)."""

    def __init__(self, ctx: "Context", nbytes: int):
        self.ctx, self.nbytes = ctx, int(nbytes)
        p = C.c_void_p()
        check(library().iree_hal_b200_buffer_allocate(ctx.device, C.c_size_t(self.nbytes), C.byref(p)))
        self.ptr = p.value or 0

    def upload(self, host: np.ndarray) -> "DeviceBuffer":
        host = np.ascontiguousarray(host)
        assert host.nbytes <= self.nbytes
        check(library().iree_hal_b200_transfer_h2d(self.ctx.device, _vp(host), C.c_void_p(self.ptr),
                                                   C.c_size_t(host.nbytes)))
        self.ctx.synchronize()  # the pageable source may be released by the caller
        return self

    def download(self, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype)
        assert out.nbytes <= self.nbytes
        check(library().iree_hal_b200_transfer_d2h(self.ctx.device, C.c_void_p(self.ptr), _vp(out),
                                                   C.c_size_t(out.nbytes)))
        self.ctx.synchronize()
        return out

    def fill(self, byte: int) -> "DeviceBuffer":
        check(library().iree_hal_b200_fill_buffer(self.ctx.device, C.c_void_p(self.ptr), C.c_size_t(self.nbytes),
                                                  C.c_uint8(byte)))
        return self

    def free(self) -> None:
        if self.ptr:
            library().iree_hal_b200_buffer_free(self.ctx.device, C.c_void_p(self.ptr))
            self.ptr = 0


class Event:
    """A CUevent on the context's dispatch stream."""

    def __init__(self, ctx: "Context"):
        self.ctx = ctx
        h = C.c_void_p()
        check(library().iree_hal_b200_event_create(ctx.device, C.byref(h)))
        self.handle = h

    def record(self) -> "Event":
        check(library().iree_hal_b200_event_record(self.ctx.device, self.handle))
        return self

    def elapsed_ms(self, end: "Event") -> float:
        ms = C.c_float()
        check(library().iree_hal_b200_event_elapsed_ms(self.ctx.device, self.handle, end.handle, C.byref(ms)))
        return float(ms.value)


class Graph:
    """A recorded sequence of dispatches replayed with one cuGraphLaunch."""

    def __init__(self, ctx: "Context", handle):
        self.ctx, self.handle = ctx, handle

    def execute(self) -> None:
        check(library().iree_hal_b200_graph_execute(self.ctx.command_buffer, self.handle))

    def release(self) -> None:
        if self.handle:
            library().iree_hal_b200_graph_release(self.handle)
            self.handle = None


class Context:
    """Device + loaded contraction executable + command buffer (``iree_b200_context_t``)."""

    def __init__(self, device_ordinal: int = 0, cubin: Optional[str] = None):
        lib = library()
        cubin = cubin or cubin_path()
        h = C.c_void_p()
        check(lib.iree_b200_context_create(C.c_int32(device_ordinal), cubin.encode(), C.byref(h)))
        self.handle = h
        self.device = C.c_void_p(lib.iree_b200_context_device(h))
        self.executable = C.c_void_p(lib.iree_b200_context_executable(h))
        self.command_buffer = C.c_void_p(lib.iree_b200_context_command_buffer(h))
        name = C.create_string_buffer(128)
        sm, cc, smem = C.c_int32(), C.c_int32(), C.c_int32()
        check(lib.iree_hal_b200_device_query(self.device, name, C.c_size_t(128), C.byref(sm), C.byref(cc),
                                             C.byref(smem)))
        self.device_name, self.sm_count, self.compute_capability = name.value.decode(), sm.value, cc.value
        self.max_shared_memory = smem.value

    # -- plumbing ------------------------------------------------------------------------
    def close(self) -> None:
        if self.handle:
            library().iree_b200_context_release(self.handle)
            self.handle = None

    def synchronize(self) -> None:
        check(library().iree_hal_b200_device_synchronize(self.device))

    @property
    def stream(self) -> int:
        return library().iree_hal_b200_device_stream(self.device) or 0

    @property
    def launch_count(self) -> int:
        return int(library().iree_hal_b200_command_buffer_launch_count(self.command_buffer))

    def set_dispatch_overlap(self, enable: bool) -> None:
        """Lets exports that order themselves on the device start before the dispatch ahead has finished."""
        check(library().iree_b200_context_set_dispatch_overlap(self.handle, C.c_int32(1 if enable else 0)))

    def set_reserved_sms(self, count: int) -> None:
        """Leaves `count` SMs free of the persistent kernels (for collectives running beside them)."""
        check(library().iree_b200_context_set_reserved_sms(self.handle, C.c_int32(count)))

    def begin_graph(self) -> None:
        check(library().iree_hal_b200_command_buffer_begin_graph(self.command_buffer))

    def end_graph(self) -> Graph:
        h = C.c_void_p()
        check(library().iree_hal_b200_command_buffer_end_graph(self.command_buffer, C.byref(h)))
        return Graph(self, h)

    def event(self) -> "Event":
        return Event(self)

    def alloc(self, nbytes: int) -> DeviceBuffer:
        return DeviceBuffer(self, nbytes)

    def to_device(self, host: np.ndarray) -> DeviceBuffer:
        host = np.ascontiguousarray(host)
        return DeviceBuffer(self, max(host.nbytes, 1)).upload(host)

    def pinned_empty(self, shape, dtype) -> np.ndarray:
        """A numpy array over page-locked host memory (freed with the context's device)."""
        nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        check(library().iree_hal_b200_host_allocate(self.device, C.c_size_t(max(nbytes, 1)), C.byref(p)))
        buf = (C.c_uint8 * max(nbytes, 1)).from_address(p.value)
        return np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)

    def pinned_copy(self, host: np.ndarray) -> np.ndarray:
        out = self.pinned_empty(host.shape, host.dtype)
        out[...] = host
        return out

    def workspace(self) -> DeviceBuffer:
        return DeviceBuffer(self, WORKSPACE_BYTES).fill(0)

    def matmul_workspace(self, params: MatmulParams) -> DeviceBuffer:
        """A workspace of the size this product asks for (more than the header when FLAG_SPLIT_K applies)."""
        library().iree_b200_matmul_workspace_bytes.restype = C.c_size_t
        nbytes = int(library().iree_b200_matmul_workspace_bytes(self.handle, C.byref(params)))
        return DeviceBuffer(self, nbytes).fill(0)

    def workspace_status(self, ws) -> None:
        check(library().iree_b200_workspace_status(self.handle, _vp(ws)))

    # -- raw HAL-level dispatch ------------------------------------------------------------
    def lookup(self, entry_name: str) -> int:
        return library().iree_hal_b200_executable_lookup(self.executable, entry_name.encode())

    def dispatch(self, entry_name: str, bindings, constants, grid) -> None:
        """push_descriptor_set + push_constants + dispatch, as a compiled host program would."""
        lib = library()
        ordinal = self.lookup(entry_name)
        if ordinal < 0:
            raise IreeB200Error(5, "no export named " + entry_name)
        arr = (_Binding * len(bindings))()
        for i, b in enumerate(bindings):
            arr[i].binding, arr[i].device_ptr = i, _vp(b).value
        check(lib.iree_hal_b200_command_buffer_push_descriptor_set(self.command_buffer, C.c_uint32(0),
                                                                   C.c_size_t(len(bindings)), arr))
        consts = np.asarray(constants, dtype=np.int32)
        check(lib.iree_hal_b200_command_buffer_push_constants(self.command_buffer, C.c_size_t(0), _vp(consts),
                                                              C.c_size_t(consts.nbytes)))
        gx, gy, gz = grid
        check(lib.iree_hal_b200_command_buffer_dispatch(self.command_buffer, self.executable, C.c_int32(ordinal),
                                                        C.c_uint32(len(bindings)), C.c_uint32(len(constants)),
                                                        C.c_uint32(gx), C.c_uint32(gy), C.c_uint32(gz)))

    # -- operators ---------------------------------------------------------------------------
    def matmul_prepare(self, params: MatmulParams, lhs, rhs, ws) -> int:
        tile_n = C.c_int32()
        check(library().iree_b200_matmul_prepare(self.handle, C.byref(params), _vp(lhs), _vp(rhs), _vp(ws),
                                                 C.byref(tile_n)))
        return tile_n.value

    def matmul_run(self, params: MatmulParams, lhs, rhs, out, ws, tile_n: int, row_scale=None,
                   col_scale=None) -> None:
        check(library().iree_b200_matmul_run(self.handle, C.byref(params), _vp(lhs), _vp(rhs), _vp(out),
                                             _vp(row_scale), _vp(col_scale), _vp(ws), C.c_int32(tile_n)))

    def matmul(self, params: MatmulParams, lhs, rhs, out, ws, row_scale=None, col_scale=None) -> None:
        check(library().iree_b200_matmul(self.handle, C.byref(params), _vp(lhs), _vp(rhs), _vp(out),
                                         _vp(row_scale), _vp(col_scale), _vp(ws)))

    def matmul_host(self, params: MatmulParams, lhs: np.ndarray, rhs: np.ndarray, out: np.ndarray,
                    row_scale=None, col_scale=None) -> None:
        check(library().iree_b200_matmul_host(self.handle, C.byref(params), _vp(lhs), _vp(rhs), _vp(out),
                                              _vp(row_scale), _vp(col_scale)))

    # fused int4 dequant + matmul
    def w4a16_workspace(self, N: int) -> DeviceBuffer:
        nbytes = int(library().iree_b200_w4a16_workspace_bytes(C.c_int32(N)))
        return DeviceBuffer(self, nbytes).fill(0)

    def w4a16_prepare(self, params: W4A16Params, a, wq, scales, out, ws):
        variant, tile_n = C.c_int32(), C.c_int32()
        check(library().iree_b200_w4a16_prepare(self.handle, C.byref(params), _vp(a), _vp(wq), _vp(scales), _vp(out),
                                                _vp(ws), C.byref(variant), C.byref(tile_n)))
        return variant.value, tile_n.value

    def w4a16_run(self, params: W4A16Params, a, wq, scales, out, ws, variant: int, tile_n: int) -> None:
        check(library().iree_b200_w4a16_run(self.handle, C.byref(params), _vp(a), _vp(wq), _vp(scales), _vp(out),
                                            _vp(ws), C.c_int32(variant), C.c_int32(tile_n)))

    def w4a16(self, params: W4A16Params, a, wq, scales, out, ws) -> None:
        check(library().iree_b200_w4a16(self.handle, C.byref(params), _vp(a), _vp(wq), _vp(scales), _vp(out), _vp(ws)))

    # N-sharded dispatch whose epilogue stores its column block into every rank's result
    def w4a16_prepare_push(self, params: W4A16Params, a, wq, scales, results, flags, rank: int, ws) -> None:
        """results / flags: one entry per rank (this rank's own buffers at index `rank`, the others as imported)."""
        world = len(results)
        check(library().iree_b200_w4a16_prepare_push(self.handle, C.byref(params), _vp(a), _vp(wq), _vp(scales),
                                                     self._ptr_array(results), self._ptr_array(flags), C.c_int32(world),
                                                     C.c_int32(rank), _vp(ws)))

    def w4a16_run_push(self, params: W4A16Params, scales, result, ws, world: int, rank: int, epoch: int) -> None:
        check(library().iree_b200_w4a16_run_push(self.handle, C.byref(params), _vp(scales), _vp(result), _vp(ws),
                                                 C.c_int32(world), C.c_int32(rank), C.c_int32(epoch)))

    def w4a16_wait_arrivals(self, own_flags, ws, world: int, epoch: int) -> None:
        check(library().iree_b200_w4a16_wait_arrivals(self.handle, _vp(own_flags), _vp(ws), C.c_int32(world),
                                                      C.c_int32(epoch)))

    def w4a16_host(self, params: W4A16Params, a, wq, scales, out) -> None:
        check(library().iree_b200_w4a16_host(self.handle, C.byref(params), _vp(a), _vp(wq), _vp(scales), _vp(out)))

    @staticmethod
    def w4a16_host_plan(params: W4A16Params):
        """The dispatches ``w4a16_host`` cuts a product into: a list of (row0, rows, col0, cols, uploads_rows,
        uploads_cols); empty when it runs as one dispatch. Needs no device."""
        units = (C.c_int32 * (6 * 32))()
        n = library().iree_b200_w4a16_host_plan(C.byref(params), units, C.c_int32(32))
        if n < 0:
            raise ValueError("invalid W4A16 parameters")
        return [tuple(units[6 * u:6 * u + 6]) for u in range(n)]

    @staticmethod
    def _ptr_array(items):
        arr = (C.c_void_p * len(items))()
        for i, x in enumerate(items):
            arr[i] = _vp(x).value
        return arr

    def matmul_run_sequence(self, params: MatmulParams, sets, tile_n: int, first: int, count: int) -> None:
        """sets: list of (lhs, rhs, out, workspace, row_scale, col_scale); issued from C in one call."""
        cols = list(zip(*sets))
        scales = cols[4][0] is not None
        check(library().iree_b200_matmul_run_sequence(
            self.handle, C.byref(params), C.c_int32(len(sets)), self._ptr_array(cols[0]), self._ptr_array(cols[1]),
            self._ptr_array(cols[2]), self._ptr_array(cols[4]) if scales else None,
            self._ptr_array(cols[5]) if scales else None, self._ptr_array(cols[3]), C.c_int32(tile_n), C.c_int32(first),
            C.c_int32(count)))

    def w4a16_run_sequence(self, params: W4A16Params, sets, variant: int, tile_n: int, first: int, count: int) -> None:
        """sets: list of (a, wq, scales, out, workspace)."""
        cols = list(zip(*sets))
        check(library().iree_b200_w4a16_run_sequence(
            self.handle, C.byref(params), C.c_int32(len(sets)), self._ptr_array(cols[0]), self._ptr_array(cols[1]),
            self._ptr_array(cols[2]), self._ptr_array(cols[3]), self._ptr_array(cols[4]), C.c_int32(variant),
            C.c_int32(tile_n), C.c_int32(first), C.c_int32(count)))

    # data-tiled entry points (argument order of iree_uk_pack / iree_uk_unpack / iree_uk_mmt4d)
    def uk_pack(self, in_buffer, in_offset, in_stride0, in_stride1, out_buffer, out_offset, out_stride0, out_stride1,
                in_size0, in_size1, out_size0, out_size1, out_size2, out_size3, padding_value, flags) -> None:
        i64 = C.c_int64
        check(library().iree_b200_uk_pack(
            self.handle, _vp(in_buffer), i64(in_offset), i64(in_stride0), i64(in_stride1), _vp(out_buffer),
            i64(out_offset), i64(out_stride0), i64(out_stride1), i64(in_size0), i64(in_size1), i64(out_size0),
            i64(out_size1), i64(out_size2), i64(out_size3), C.c_uint64(padding_value), C.c_uint32(flags)))

    def uk_unpack(self, in_buffer, in_offset, in_stride0, in_stride1, out_buffer, out_offset, out_stride0, out_stride1,
                  in_size0, in_size1, in_size2, in_size3, out_size0, out_size1, flags) -> None:
        i64 = C.c_int64
        check(library().iree_b200_uk_unpack(
            self.handle, _vp(in_buffer), i64(in_offset), i64(in_stride0), i64(in_stride1), _vp(out_buffer),
            i64(out_offset), i64(out_stride0), i64(out_stride1), i64(in_size0), i64(in_size1), i64(in_size2),
            i64(in_size3), i64(out_size0), i64(out_size1), C.c_uint32(flags)))

    # -- transfer commands, barriers, layouts (the reference's command-buffer API beyond dispatch) ----
    def begin(self) -> None:
        check(library().iree_hal_b200_command_buffer_begin(self.command_buffer))

    def end(self) -> None:
        check(library().iree_hal_b200_command_buffer_end(self.command_buffer))

    def execution_barrier(self) -> None:
        check(library().iree_hal_b200_command_buffer_execution_barrier(self.command_buffer, C.c_uint32(0), C.c_uint32(0),
                                                                        C.c_uint32(0)))

    def fill_buffer(self, target, offset: int, length: int, pattern: bytes) -> None:
        check(library().iree_hal_b200_command_buffer_fill_buffer(self.command_buffer, _vp(target), C.c_size_t(offset),
                                                                  C.c_size_t(length), pattern, C.c_size_t(len(pattern))))

    def copy_buffer(self, source, source_offset: int, target, target_offset: int, length: int) -> None:
        check(library().iree_hal_b200_command_buffer_copy_buffer(self.command_buffer, _vp(source), C.c_size_t(source_offset),
                                                                  _vp(target), C.c_size_t(target_offset), C.c_size_t(length)))

    def pipeline_layout(self, push_constant_count: int, set_binding_counts) -> C.c_void_p:
        """A pipeline layout of len(set_binding_counts) descriptor sets; free with release_pipeline_layout."""
        lib = library()
        sets = (C.c_void_p * max(len(set_binding_counts), 1))()
        for i, n in enumerate(set_binding_counts):
            h = C.c_void_p()
            check(lib.iree_hal_b200_descriptor_set_layout_create(self.device, C.c_uint32(n), C.byref(h)))
            sets[i] = h
        out = C.c_void_p()
        try:
            check(lib.iree_hal_b200_pipeline_layout_create(self.device, C.c_uint32(push_constant_count),
                                                           C.c_uint32(len(set_binding_counts)), sets, C.byref(out)))
        finally:
            for i in range(len(set_binding_counts)):
                lib.iree_hal_b200_descriptor_set_layout_release(C.c_void_p(sets[i]))
        return out

    def release_pipeline_layout(self, layout) -> None:
        library().iree_hal_b200_pipeline_layout_release(layout)

    def push_descriptor_set(self, set_index: int, pointers) -> None:
        arr = (_Binding * len(pointers))()
        for i, b in enumerate(pointers):
            arr[i].binding, arr[i].device_ptr = i, _vp(b).value
        check(library().iree_hal_b200_command_buffer_push_descriptor_set(self.command_buffer, C.c_uint32(set_index),
                                                                         C.c_size_t(len(pointers)), arr))

    def dispatch_with_layout(self, entry_name: str, layout, constants, grid) -> None:
        lib = library()
        ordinal = self.lookup(entry_name)
        if ordinal < 0:
            raise IreeB200Error(5, "no export named " + entry_name)
        consts = np.asarray(constants, dtype=np.int32)
        check(lib.iree_hal_b200_command_buffer_push_constants(self.command_buffer, C.c_size_t(0), _vp(consts),
                                                              C.c_size_t(consts.nbytes)))
        gx, gy, gz = grid
        check(lib.iree_hal_b200_command_buffer_dispatch_with_layout(self.command_buffer, self.executable, C.c_int32(ordinal),
                                                                    layout, C.c_uint32(gx), C.c_uint32(gy), C.c_uint32(gz)))

    def uk_status(self) -> None:
        """Raises if a pack / unpack kernel reported a rejected argument or a wait that ran out."""
        check(library().iree_b200_uk_status(self.handle))

    def uk_mmt4d_workspace(self, M, N, K, M0, N0, K0, flags) -> DeviceBuffer:
        nbytes = int(library().iree_b200_uk_mmt4d_workspace_bytes(C.c_int64(M), C.c_int64(N), C.c_int64(K), C.c_int32(M0),
                                                                  C.c_int32(N0), C.c_int32(K0), C.c_uint32(flags)))
        return DeviceBuffer(self, max(nbytes, 512)).fill(0)

    def uk_mmt4d(self, lhs, lhs_offset, lhs_stride0, rhs, rhs_offset, rhs_stride0, out, out_offset, out_stride0,
                 M, N, K, M0, N0, K0, flags, workspace) -> None:
        i64 = C.c_int64
        check(library().iree_b200_uk_mmt4d(
            self.handle, _vp(lhs), i64(lhs_offset), i64(lhs_stride0), _vp(rhs), i64(rhs_offset), i64(rhs_stride0),
            _vp(out), i64(out_offset), i64(out_stride0), i64(M), i64(N), i64(K), C.c_int32(M0), C.c_int32(N0),
            C.c_int32(K0), C.c_uint32(flags), _vp(workspace)))

    def encode_tensor_map(self, elem_bytes, is_bf16, ptr, dim0, dim1, dim2, box0, box1) -> bytes:
        out = C.create_string_buffer(128)
        check(library().iree_b200_encode_tensor_map(self.handle, C.c_int32(elem_bytes), C.c_int32(int(is_bf16)),
                                                    _vp(ptr), C.c_uint32(dim0), C.c_uint32(dim1), C.c_uint32(dim2),
                                                    C.c_uint32(box0), C.c_uint32(box1), out))
        return out.raw


_IN_DTYPE = {KIND_F16: np.float16, KIND_BF16: np.uint16, KIND_I8: np.int8}


def out_dtype(kind: int, epilogue: int):
    if epilogue == EPILOGUE_ACCUMULATOR:
        return np.int32 if kind == KIND_I8 else np.float32
    return np.uint16 if (kind == KIND_BF16 and epilogue == EPILOGUE_CAST) else np.float16


def matmul_numpy(ctx: Context, kind: int, epilogue: int, lhs: np.ndarray, rhs: np.ndarray, rhs_layout: int = RHS_KN,
                 row_scale=None, col_scale=None, tile_n: int = 0, flags: int = 0) -> np.ndarray:
    """Convenience for tests: host arrays in, host array out, through iree_b200_matmul_host.

    lhs is [M,K] or [B,M,K]; rhs is [K,N] / [B,K,N] (RHS_KN) or [N,K] / [B,N,K] (RHS_NK).
    bf16 travels as raw uint16 bit patterns.
    """
    lhs = np.ascontiguousarray(lhs)
    rhs = np.ascontiguousarray(rhs)
    assert lhs.dtype == _IN_DTYPE[kind] and rhs.dtype == _IN_DTYPE[kind], (lhs.dtype, rhs.dtype)
    batched = lhs.ndim == 3
    B = lhs.shape[0] if batched else 1
    M, K = lhs.shape[-2:]
    N = rhs.shape[-1] if rhs_layout == RHS_KN else rhs.shape[-2]
    p = MatmulParams(kind, epilogue, M, N, K, B, rhs_layout, tile_n, flags)
    out = np.empty((B, M, N) if batched else (M, N), out_dtype(kind, epilogue))
    rs = None if row_scale is None else np.ascontiguousarray(row_scale, np.float32)
    cs = None if col_scale is None else np.ascontiguousarray(col_scale, np.float32)
    ctx.matmul_host(p, lhs, rhs, out, rs, cs)
    return out


# ---- data tiling conveniences (tests and the bench) -------------------------------------------------

UK_PACK_TYPE = {1: 0x02, 2: 0x04, 4: 0x03}  # element bytes -> I8I8 / F16F16 / I32I32 (pure data movement)
UK_TRANSPOSE_INNER, UK_TRANSPOSE_OUTER = 0x100, 0x200
UK_PACK_NO_TMA = 0x40000     # this library's own: the staging kernels even where the TMA unit alone could copy
UK_MMT4D_S8S8S32, UK_MMT4D_F16F16F32, UK_MMT4D_F16F16F16 = 0x02, 0x03, 0x04
UK_MMT4D_BF16BF16F32, UK_MMT4D_BF16BF16BF16, UK_MMT4D_ACCUMULATE = 0x05, 0x06, 0x100
UK_MMT4D_F32F32F32, UK_MMT4D_S16S16S32, UK_MMT4D_S16U4S32, UK_MMT4D_S16S8S32, UK_MMT4D_S8S4S32 = 0x01, 0x07, 0x08, 0x09, 0x0A
UK_MMT4D_UNTILE = 0x10000   # this library's own: take the un-tiling path even where the tiled-operand kernel applies


def pack_numpy(ctx: Context, x: np.ndarray, tile, transpose_inner=False, transpose_outer=False, padding: int = 0,
               out_shape=None, extra_flags: int = 0) -> np.ndarray:
    """Host [S0,S1] array in, tiled [o0,o1,o2,o3] array out, through iree_b200_uk_pack. `tile` is the
    (rows, cols) tile extent in matrix terms; x may be a strided 2-D view."""
    assert x.ndim == 2
    es = x.dtype.itemsize
    t0, t1 = tile
    n0, n1 = -(-x.shape[0] // t0), -(-x.shape[1] // t1)
    if out_shape is None:
        outer = (n1, n0) if transpose_outer else (n0, n1)
        inner = (t1, t0) if transpose_inner else (t0, t1)
        out_shape = outer + inner
    # A strided view travels as its whole (contiguous) base plus offset and strides, in elements.
    base = x
    while base.base is not None and isinstance(base.base, np.ndarray):
        base = base.base
    if not base.flags.c_contiguous:
        base = x = np.ascontiguousarray(x)
    offset = (x.__array_interface__["data"][0] - base.__array_interface__["data"][0]) // es
    stride0, stride1 = x.strides[0] // es, x.strides[1] // es
    dev_in = ctx.to_device(base.reshape(-1).view(np.uint8)) if base.size else ctx.alloc(16)
    count = int(np.prod(out_shape))
    dev_out = ctx.alloc(max(count * es, 16)).fill(0xCD)
    flags = UK_PACK_TYPE[es] | (UK_TRANSPOSE_INNER if transpose_inner else 0) | (UK_TRANSPOSE_OUTER if transpose_outer else 0)
    flags |= extra_flags
    ctx.uk_pack(dev_in, offset, stride0, stride1, dev_out, 0, out_shape[1] * out_shape[2] * out_shape[3],
                out_shape[2] * out_shape[3], x.shape[0], x.shape[1], *out_shape, padding, flags)
    out = dev_out.download(x.dtype, out_shape)
    ctx.uk_status()
    dev_in.free()
    dev_out.free()
    return out


def unpack_numpy(ctx: Context, x4: np.ndarray, out_shape, transpose_inner=False, transpose_outer=False,
                 fill: int = 0xCD, extra_flags: int = 0) -> np.ndarray:
    """Tiled host array in, row-major [S0,S1] out, through iree_b200_uk_unpack; untouched output bytes keep `fill`."""
    x4 = np.ascontiguousarray(x4)
    es = x4.dtype.itemsize
    dev_in = ctx.to_device(x4) if x4.size else ctx.alloc(16)
    count = int(out_shape[0] * out_shape[1])
    dev_out = ctx.alloc(max(count * es, 16)).fill(fill)
    flags = UK_PACK_TYPE[es] | (UK_TRANSPOSE_INNER if transpose_inner else 0) | (UK_TRANSPOSE_OUTER if transpose_outer else 0)
    flags |= extra_flags
    ctx.uk_unpack(dev_in, 0, x4.shape[1] * x4.shape[2] * x4.shape[3], x4.shape[2] * x4.shape[3], dev_out, 0, out_shape[1], 1,
                  *x4.shape, out_shape[0], out_shape[1], flags)
    out = dev_out.download(x4.dtype, tuple(out_shape))
    ctx.uk_status()
    dev_in.free()
    dev_out.free()
    return out


def mmt4d_numpy(ctx: Context, type_flag: int, lhs4: np.ndarray, rhs4: np.ndarray, acc4=None) -> np.ndarray:
    """lhs4 [M,K,M0,K0], rhs4 [N,K,N0,K0] -> [M,N,M0,N0] through iree_b200_uk_mmt4d (acc4 given: ACCUMULATE)."""
    lhs4, rhs4 = np.ascontiguousarray(lhs4), np.ascontiguousarray(rhs4)
    M, K, M0, K0 = lhs4.shape
    N, K2, N0, K02 = rhs4.shape
    four_bit = type_flag in (UK_MMT4D_S16U4S32, UK_MMT4D_S8S4S32)   # right-hand side: two elements per byte
    assert (K, K0) == (K2, K02 * 2 if four_bit else K02)
    odt = {UK_MMT4D_S8S8S32: np.int32, UK_MMT4D_F16F16F32: np.float32, UK_MMT4D_BF16BF16F32: np.float32,
           UK_MMT4D_F16F16F16: np.float16, UK_MMT4D_BF16BF16BF16: np.uint16, UK_MMT4D_F32F32F32: np.float32,
           UK_MMT4D_S16S16S32: np.int32, UK_MMT4D_S16U4S32: np.int32, UK_MMT4D_S16S8S32: np.int32,
           UK_MMT4D_S8S4S32: np.int32}[type_flag]
    flags = type_flag | (UK_MMT4D_ACCUMULATE if acc4 is not None else 0)
    out_shape = (M, N, M0, N0)
    count = int(np.prod(out_shape))
    dl = ctx.to_device(lhs4) if lhs4.size else ctx.alloc(16)
    dr = ctx.to_device(rhs4) if rhs4.size else ctx.alloc(16)
    if acc4 is not None:
        do = ctx.to_device(np.ascontiguousarray(acc4, odt)) if count else ctx.alloc(16)
    else:
        do = ctx.alloc(max(count * np.dtype(odt).itemsize, 16)).fill(0xCD)
    ws = ctx.uk_mmt4d_workspace(M, N, K, M0, N0, K0, flags)
    ctx.uk_mmt4d(dl, 0, K * M0 * K0, dr, 0, K * N0 * K0, do, 0, N * M0 * N0, M, N, K, M0, N0, K0, flags, ws)
    ctx.workspace_status(ws)
    out = do.download(odt, out_shape)
    for b in (dl, dr, do, ws):
        b.free()
    return out
