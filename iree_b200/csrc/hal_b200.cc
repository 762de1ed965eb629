// Host side of libiree_b200.so: the HAL-shaped runtime slice (device, buffers, ExecutableDef
// loader, stream command buffer, NCCL channel) and the operator-level contraction entry points
// declared in include/iree_b200.h. Host code only: the kernels live in a separate sm_100a cubin
// that enters through the same ExecutableDef container the reference's CUDA driver loads.
//
// libcuda.so and libnccl.so are opened at run time, as the reference's
// cuda_dynamic_symbols.c / nccl_dynamic_symbols.c do, so this library loads (and its symbols
// can be inspected) on a machine without a GPU; every call that needs the device then
// returns UNAVAILABLE. There is no CPU execution path.
#include <cuda.h>
#include <dlfcn.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <chrono>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/iree_b200.h"
#include "hal_b200_internal.h"
#include "w4a16_decode_tc.h"

namespace {

thread_local std::string g_last_error;

iree_b200_status_t fail(iree_b200_status_t code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

#define B200_RETURN_IF_ERROR(expr)                     \
  do {                                                 \
    iree_b200_status_t status__ = (expr);              \
    if (status__ != IREE_B200_STATUS_OK) return status__; \
  } while (0)

// ------------------------------------------------------------------------------------------
// Dynamic CUDA driver symbols.
// ------------------------------------------------------------------------------------------
struct CudaSymbols {
  void* handle = nullptr;
  bool tried = false;
  std::string error;
#define CU_FN(name, ...) CUresult (*name)(__VA_ARGS__) = nullptr;
  CU_FN(cuInit, unsigned)
  CU_FN(cuDeviceGet, CUdevice*, int)
  CU_FN(cuDeviceGetCount, int*)
  CU_FN(cuDeviceGetName, char*, int, CUdevice)
  CU_FN(cuDeviceGetAttribute, int*, CUdevice_attribute, CUdevice)
  CU_FN(cuDevicePrimaryCtxRetain, CUcontext*, CUdevice)
  CU_FN(cuDevicePrimaryCtxRelease, CUdevice)
  CU_FN(cuCtxSetCurrent, CUcontext)
  CU_FN(cuStreamCreate, CUstream*, unsigned)
  CU_FN(cuStreamDestroy, CUstream)
  CU_FN(cuStreamSynchronize, CUstream)
  CU_FN(cuStreamWaitEvent, CUstream, CUevent, unsigned)
  CU_FN(cuMemAlloc, CUdeviceptr*, size_t)
  CU_FN(cuMemFree, CUdeviceptr)
  CU_FN(cuMemHostAlloc, void**, size_t, unsigned)
  CU_FN(cuMemFreeHost, void*)
  CU_FN(cuMemcpyHtoDAsync, CUdeviceptr, const void*, size_t, CUstream)
  CU_FN(cuMemcpyDtoHAsync, void*, CUdeviceptr, size_t, CUstream)
  CU_FN(cuMemsetD8Async, CUdeviceptr, unsigned char, size_t, CUstream)
  CU_FN(cuModuleLoadDataEx, CUmodule*, const void*, unsigned, CUjit_option*, void**)
  CU_FN(cuModuleUnload, CUmodule)
  CU_FN(cuModuleGetFunction, CUfunction*, CUmodule, const char*)
  CU_FN(cuFuncSetAttribute, CUfunction, CUfunction_attribute, int)
  CU_FN(cuLaunchKernel, CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
        void**, void**)
  CU_FN(cuEventCreate, CUevent*, unsigned)
  CU_FN(cuEventDestroy, CUevent)
  CU_FN(cuEventRecord, CUevent, CUstream)
  CU_FN(cuEventSynchronize, CUevent)
  CU_FN(cuEventElapsedTime, float*, CUevent, CUevent)
  CU_FN(cuGraphCreate, CUgraph*, unsigned)
  CU_FN(cuGraphDestroy, CUgraph)
  CU_FN(cuGraphAddKernelNode, CUgraphNode*, CUgraph, const CUgraphNode*, size_t, const CUDA_KERNEL_NODE_PARAMS*)
  CU_FN(cuGraphInstantiateWithFlags, CUgraphExec*, CUgraph, unsigned long long)
  CU_FN(cuGraphLaunch, CUgraphExec, CUstream)
  CU_FN(cuGraphExecDestroy, CUgraphExec)
  // optional (programmatic dependent launch); dispatch overlap is refused when they are missing
  CU_FN(cuIpcGetMemHandle, CUipcMemHandle*, CUdeviceptr)
  CU_FN(cuIpcOpenMemHandle, CUdeviceptr*, CUipcMemHandle, unsigned)
  CU_FN(cuIpcCloseMemHandle, CUdeviceptr)
  CU_FN(cuMemcpyDtoDAsync, CUdeviceptr, CUdeviceptr, size_t, CUstream)
  CU_FN(cuLaunchKernelEx, const CUlaunchConfig*, CUfunction, void**, void**)
  CU_FN(cuGraphAddDependencies_v2, CUgraph, const CUgraphNode*, const CUgraphNode*, const CUgraphEdgeData*, size_t)
  CU_FN(cuEventQuery, CUevent)
  // optional (transfer commands)
  CU_FN(cuMemsetD16Async, CUdeviceptr, unsigned short, size_t, CUstream)
  CU_FN(cuMemsetD32Async, CUdeviceptr, unsigned int, size_t, CUstream)
  CU_FN(cuGraphAddMemcpyNode, CUgraphNode*, CUgraph, const CUgraphNode*, size_t, const CUDA_MEMCPY3D*, CUcontext)
  CU_FN(cuGraphAddMemsetNode, CUgraphNode*, CUgraph, const CUgraphNode*, size_t, const CUDA_MEMSET_NODE_PARAMS*, CUcontext)
  CU_FN(cuMemcpy2DAsync, const CUDA_MEMCPY2D*, CUstream)
  CU_FN(cuGetErrorName, CUresult, const char**)
  CU_FN(cuGetErrorString, CUresult, const char**)
  CU_FN(cuTensorMapEncodeTiled, CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
        const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
        CUtensorMapL2promotion, CUtensorMapFloatOOBfill)
#undef CU_FN
};
CudaSymbols g_cu;
std::mutex g_cu_mutex;

template <typename T>
bool load_sym(void* handle, const char* name, T& out) {
  out = reinterpret_cast<T>(dlsym(handle, name));
  return out != nullptr;
}

iree_b200_status_t ensure_cuda() {
  std::lock_guard<std::mutex> lock(g_cu_mutex);
  if (!g_cu.tried) {
    g_cu.tried = true;
    const char* names[] = {"libcuda.so.1", "libcuda.so"};
    for (const char* n : names) {
      g_cu.handle = dlopen(n, RTLD_NOW | RTLD_LOCAL);
      if (g_cu.handle) break;
    }
    if (!g_cu.handle) {
      g_cu.error = "CUDA driver library (libcuda.so.1) could not be loaded; no GPU on this machine?";
    } else {
      bool ok = true;
#define LOAD(field, symbol) ok = load_sym(g_cu.handle, symbol, g_cu.field) && ok;
      LOAD(cuInit, "cuInit")
      LOAD(cuDeviceGet, "cuDeviceGet")
      LOAD(cuDeviceGetCount, "cuDeviceGetCount")
      LOAD(cuDeviceGetName, "cuDeviceGetName")
      LOAD(cuDeviceGetAttribute, "cuDeviceGetAttribute")
      LOAD(cuDevicePrimaryCtxRetain, "cuDevicePrimaryCtxRetain")
      LOAD(cuDevicePrimaryCtxRelease, "cuDevicePrimaryCtxRelease_v2")
      LOAD(cuCtxSetCurrent, "cuCtxSetCurrent")
      LOAD(cuStreamCreate, "cuStreamCreate")
      LOAD(cuStreamDestroy, "cuStreamDestroy_v2")
      LOAD(cuStreamSynchronize, "cuStreamSynchronize")
      LOAD(cuStreamWaitEvent, "cuStreamWaitEvent")
      LOAD(cuMemAlloc, "cuMemAlloc_v2")
      LOAD(cuMemFree, "cuMemFree_v2")
      LOAD(cuMemHostAlloc, "cuMemHostAlloc")
      LOAD(cuMemFreeHost, "cuMemFreeHost")
      LOAD(cuMemcpyHtoDAsync, "cuMemcpyHtoDAsync_v2")
      LOAD(cuMemcpyDtoHAsync, "cuMemcpyDtoHAsync_v2")
      LOAD(cuMemsetD8Async, "cuMemsetD8Async")
      LOAD(cuModuleLoadDataEx, "cuModuleLoadDataEx")
      LOAD(cuModuleUnload, "cuModuleUnload")
      LOAD(cuModuleGetFunction, "cuModuleGetFunction")
      LOAD(cuFuncSetAttribute, "cuFuncSetAttribute")
      LOAD(cuLaunchKernel, "cuLaunchKernel")
      LOAD(cuEventCreate, "cuEventCreate")
      LOAD(cuEventDestroy, "cuEventDestroy_v2")
      LOAD(cuEventRecord, "cuEventRecord")
      LOAD(cuEventSynchronize, "cuEventSynchronize")
      LOAD(cuEventElapsedTime, "cuEventElapsedTime")
      LOAD(cuGraphCreate, "cuGraphCreate")
      LOAD(cuGraphDestroy, "cuGraphDestroy")
      LOAD(cuGraphAddKernelNode, "cuGraphAddKernelNode_v2")
      LOAD(cuGraphInstantiateWithFlags, "cuGraphInstantiateWithFlags")
      LOAD(cuGraphLaunch, "cuGraphLaunch")
      LOAD(cuGraphExecDestroy, "cuGraphExecDestroy")
      LOAD(cuGetErrorName, "cuGetErrorName")
      LOAD(cuGetErrorString, "cuGetErrorString")
      LOAD(cuTensorMapEncodeTiled, "cuTensorMapEncodeTiled")
#undef LOAD
      load_sym(g_cu.handle, "cuIpcGetMemHandle", g_cu.cuIpcGetMemHandle);
      load_sym(g_cu.handle, "cuIpcOpenMemHandle_v2", g_cu.cuIpcOpenMemHandle);
      load_sym(g_cu.handle, "cuIpcCloseMemHandle", g_cu.cuIpcCloseMemHandle);
      load_sym(g_cu.handle, "cuMemcpyDtoDAsync_v2", g_cu.cuMemcpyDtoDAsync);
      load_sym(g_cu.handle, "cuLaunchKernelEx", g_cu.cuLaunchKernelEx);
      load_sym(g_cu.handle, "cuGraphAddDependencies_v2", g_cu.cuGraphAddDependencies_v2);
      load_sym(g_cu.handle, "cuEventQuery", g_cu.cuEventQuery);
      load_sym(g_cu.handle, "cuMemsetD16Async", g_cu.cuMemsetD16Async);
      load_sym(g_cu.handle, "cuMemsetD32Async", g_cu.cuMemsetD32Async);
      load_sym(g_cu.handle, "cuGraphAddMemcpyNode", g_cu.cuGraphAddMemcpyNode);
      load_sym(g_cu.handle, "cuGraphAddMemsetNode", g_cu.cuGraphAddMemsetNode);
      load_sym(g_cu.handle, "cuMemcpy2DAsync_v2", g_cu.cuMemcpy2DAsync);
      if (!ok) {
        g_cu.error = "CUDA driver library is missing required symbols";
        g_cu.handle = nullptr;
      } else {
        CUresult r = g_cu.cuInit(0);
        if (r != CUDA_SUCCESS) {
          g_cu.error = "cuInit failed (" + std::to_string(static_cast<int>(r)) + ")";
          g_cu.handle = nullptr;
        }
      }
    }
  }
  if (!g_cu.handle) return fail(IREE_B200_STATUS_UNAVAILABLE, "%s", g_cu.error.c_str());
  return IREE_B200_STATUS_OK;
}

// CUresult -> status with the driver's own name and text, like cuda_status_util.c.
iree_b200_status_t cu_check(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return IREE_B200_STATUS_OK;
  const char *name = "?", *text = "?";
  if (g_cu.cuGetErrorName) g_cu.cuGetErrorName(r, &name);
  if (g_cu.cuGetErrorString) g_cu.cuGetErrorString(r, &text);
  iree_b200_status_t code = IREE_B200_STATUS_INTERNAL;
  if (r == CUDA_ERROR_OUT_OF_MEMORY) code = IREE_B200_STATUS_RESOURCE_EXHAUSTED;
  if (r == CUDA_ERROR_INVALID_VALUE) code = IREE_B200_STATUS_INVALID_ARGUMENT;
  if (r == CUDA_ERROR_NOT_FOUND) code = IREE_B200_STATUS_NOT_FOUND;
  return fail(code, "%s: %s (%s)", what, name ? name : "?", text ? text : "?");
}
#define CU_RETURN_IF_ERROR(expr, what) B200_RETURN_IF_ERROR(cu_check((expr), what))

// ------------------------------------------------------------------------------------------
// Dynamic NCCL symbols (only touched when a channel is created).
// ------------------------------------------------------------------------------------------
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
struct NcclSymbols {
  void* handle = nullptr;
  bool tried = false;
  std::string error;
  int (*ncclGetVersion)(int*) = nullptr;
  int (*ncclGetUniqueId)(ncclUniqueId*) = nullptr;
  int (*ncclCommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  int (*ncclCommDestroy)(ncclComm_t) = nullptr;
  int (*ncclAllGather)(const void*, void*, size_t, int, ncclComm_t, CUstream) = nullptr;
  int (*ncclAllReduce)(const void*, void*, size_t, int, int, ncclComm_t, CUstream) = nullptr;  // optional
  int (*ncclGroupStart)() = nullptr;
  int (*ncclGroupEnd)() = nullptr;
  int (*ncclCommSplit)(ncclComm_t, int, int, ncclComm_t*, void*) = nullptr;  // optional (NCCL >= 2.18)
  // optional: the collective kinds beyond all-gather
  int (*ncclBroadcast)(const void*, void*, size_t, int, int, ncclComm_t, CUstream) = nullptr;
  int (*ncclReduce)(const void*, void*, size_t, int, int, int, ncclComm_t, CUstream) = nullptr;
  int (*ncclReduceScatter)(const void*, void*, size_t, int, int, ncclComm_t, CUstream) = nullptr;
  int (*ncclSend)(const void*, size_t, int, int, ncclComm_t, CUstream) = nullptr;
  int (*ncclRecv)(void*, size_t, int, int, ncclComm_t, CUstream) = nullptr;
  int (*ncclCommCount)(const ncclComm_t, int*) = nullptr;                   // optional
  int (*ncclCommUserRank)(const ncclComm_t, int*) = nullptr;                // optional
  const char* (*ncclGetErrorString)(int) = nullptr;
};
NcclSymbols g_nccl;

iree_b200_status_t ensure_nccl() {
  std::lock_guard<std::mutex> lock(g_cu_mutex);
  if (!g_nccl.tried) {
    g_nccl.tried = true;
    // A copy already loaded into the process (for instance by a Python framework) is preferred,
    // so that one NCCL instance owns the NVLink resources.
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      g_nccl.handle = dlopen(n, RTLD_NOW | RTLD_NOLOAD | RTLD_LOCAL);
      if (g_nccl.handle) break;
    }
    const char* env = getenv("IREE_B200_NCCL_LIBRARY");
    if (!g_nccl.handle && env) g_nccl.handle = dlopen(env, RTLD_NOW | RTLD_LOCAL);
    for (const char* n : names) {
      if (g_nccl.handle) break;
      g_nccl.handle = dlopen(n, RTLD_NOW | RTLD_LOCAL);
    }
    if (!g_nccl.handle) {
      g_nccl.error = "NCCL library (libnccl.so.2) could not be loaded";
    } else {
      bool ok = true;
      ok = load_sym(g_nccl.handle, "ncclGetVersion", g_nccl.ncclGetVersion) && ok;
      ok = load_sym(g_nccl.handle, "ncclGetUniqueId", g_nccl.ncclGetUniqueId) && ok;
      ok = load_sym(g_nccl.handle, "ncclCommInitRank", g_nccl.ncclCommInitRank) && ok;
      ok = load_sym(g_nccl.handle, "ncclCommDestroy", g_nccl.ncclCommDestroy) && ok;
      ok = load_sym(g_nccl.handle, "ncclAllGather", g_nccl.ncclAllGather) && ok;
      load_sym(g_nccl.handle, "ncclAllReduce", g_nccl.ncclAllReduce);
      load_sym(g_nccl.handle, "ncclCommSplit", g_nccl.ncclCommSplit);
      load_sym(g_nccl.handle, "ncclBroadcast", g_nccl.ncclBroadcast);
      load_sym(g_nccl.handle, "ncclReduce", g_nccl.ncclReduce);
      load_sym(g_nccl.handle, "ncclReduceScatter", g_nccl.ncclReduceScatter);
      load_sym(g_nccl.handle, "ncclSend", g_nccl.ncclSend);
      load_sym(g_nccl.handle, "ncclRecv", g_nccl.ncclRecv);
      load_sym(g_nccl.handle, "ncclCommCount", g_nccl.ncclCommCount);
      load_sym(g_nccl.handle, "ncclCommUserRank", g_nccl.ncclCommUserRank);
      ok = load_sym(g_nccl.handle, "ncclGroupStart", g_nccl.ncclGroupStart) && ok;
      ok = load_sym(g_nccl.handle, "ncclGroupEnd", g_nccl.ncclGroupEnd) && ok;
      ok = load_sym(g_nccl.handle, "ncclGetErrorString", g_nccl.ncclGetErrorString) && ok;
      if (!ok) {
        g_nccl.error = "NCCL library is missing required symbols";
        g_nccl.handle = nullptr;
      }
    }
  }
  if (!g_nccl.handle) return fail(IREE_B200_STATUS_UNAVAILABLE, "%s", g_nccl.error.c_str());
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t nccl_check(int r, const char* what) {
  if (r == 0) return IREE_B200_STATUS_OK;
  return fail(IREE_B200_STATUS_INTERNAL, "%s: NCCL error %d (%s)", what, r,
              g_nccl.ncclGetErrorString ? g_nccl.ncclGetErrorString(r) : "?");
}

// ------------------------------------------------------------------------------------------
// Minimal flatbuffer reader / writer for ExecutableDef.
// ------------------------------------------------------------------------------------------
struct ExecutableDefView {
  std::vector<std::string> entry_points;
  std::vector<uint32_t> block_sizes;  // 3 per entry
  std::vector<uint32_t> shared_memory;
  const uint8_t* image = nullptr;
  size_t image_size = 0;
};

struct FbReader {
  const uint8_t* data;
  size_t size;
  bool in(size_t pos, size_t len) const { return pos <= size && len <= size - pos; }
  bool u16(size_t pos, uint16_t* v) const {
    if (!in(pos, 2)) return false;
    memcpy(v, data + pos, 2);
    return true;
  }
  bool u32(size_t pos, uint32_t* v) const {
    if (!in(pos, 4)) return false;
    memcpy(v, data + pos, 4);
    return true;
  }
  bool i32(size_t pos, int32_t* v) const {
    if (!in(pos, 4)) return false;
    memcpy(v, data + pos, 4);
    return true;
  }
};

// Resolves table field `index` to the absolute position of its value (0 when absent).
bool fb_field(const FbReader& r, size_t table, int index, size_t* out_pos) {
  int32_t soff;
  if (!r.i32(table, &soff)) return false;
  int64_t vt = static_cast<int64_t>(table) - soff;
  if (vt < 0 || !r.in(static_cast<size_t>(vt), 4)) return false;
  uint16_t vt_size, field_off = 0;
  if (!r.u16(static_cast<size_t>(vt), &vt_size)) return false;
  size_t slot = 4 + 2 * static_cast<size_t>(index);
  if (slot + 2 <= vt_size && !r.u16(static_cast<size_t>(vt) + slot, &field_off)) return false;
  *out_pos = field_off ? table + field_off : 0;
  return true;
}
// Follows the uoffset stored at pos.
bool fb_indirect(const FbReader& r, size_t pos, size_t* out) {
  uint32_t off;
  if (!r.u32(pos, &off)) return false;
  *out = pos + off;
  return r.in(*out, 4);
}

iree_b200_status_t parse_executable_def(const void* data, size_t size, ExecutableDefView* view) {
  if (!data) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "flatbuffer data is not present");
  FbReader r{static_cast<const uint8_t*>(data), size};
  const char* bad = "flatbuffer verification failed";
  if (size < 12 || memcmp(r.data + 4, "CUDA", 4) != 0)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "%s: file identifier is not 'CUDA'", bad);
  size_t table;
  if (!fb_indirect(r, 0, &table)) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "%s: root out of range", bad);
  size_t f_entries, f_blocks, f_smem, f_image;
  if (!fb_field(r, table, 0, &f_entries) || !fb_field(r, table, 1, &f_blocks) || !fb_field(r, table, 2, &f_smem) ||
      !fb_field(r, table, 3, &f_image))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "%s: vtable out of range", bad);
  if (f_entries) {
    size_t vec;
    uint32_t n;
    if (!fb_indirect(r, f_entries, &vec) || !r.u32(vec, &n) || !r.in(vec + 4, 4ull * n))
      return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "%s: entry_points out of range", bad);
    for (uint32_t i = 0; i < n; ++i) {
      size_t str;
      uint32_t len;
      if (!fb_indirect(r, vec + 4 + 4ull * i, &str) || !r.u32(str, &len) || !r.in(str + 4, static_cast<size_t>(len) + 1))
        return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "%s: entry point %u out of range", bad, i);
      view->entry_points.emplace_back(reinterpret_cast<const char*>(r.data + str + 4), len);
    }
  }
  if (f_blocks) {
    size_t vec;
    uint32_t n;
    if (!fb_indirect(r, f_blocks, &vec) || !r.u32(vec, &n) || !r.in(vec + 4, 12ull * n))
      return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "%s: block_sizes out of range", bad);
    view->block_sizes.resize(3ull * n);
    memcpy(view->block_sizes.data(), r.data + vec + 4, 12ull * n);
  }
  if (f_smem) {
    size_t vec;
    uint32_t n;
    if (!fb_indirect(r, f_smem, &vec) || !r.u32(vec, &n) || !r.in(vec + 4, 4ull * n))
      return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "%s: shared_memory_size out of range", bad);
    view->shared_memory.resize(n);
    memcpy(view->shared_memory.data(), r.data + vec + 4, 4ull * n);
  }
  if (f_image) {
    size_t str;
    uint32_t len;
    if (!fb_indirect(r, f_image, &str) || !r.u32(str, &len) || !r.in(str + 4, static_cast<size_t>(len) + 1))
      return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "%s: ptx_image out of range", bad);
    view->image = r.data + str + 4;
    view->image_size = len;
  }
  // Content rules of native_executable.c:76-108.
  for (size_t i = 0; i < view->entry_points.size(); ++i)
    if (view->entry_points[i].empty())
      return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "executable entry point %zu has no name", i);
  if (view->block_sizes.empty()) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "no block sizes present");
  if (view->entry_points.size() != view->block_sizes.size() / 3)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "entry points (%zu) and block sizes (%zu) count mismatch",
                view->entry_points.size(), view->block_sizes.size() / 3);
  if (view->image_size == 0) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "no PTX image present");
  return IREE_B200_STATUS_OK;
}

void put_u32(std::vector<uint8_t>& b, size_t pos, uint32_t v) { memcpy(b.data() + pos, &v, 4); }
size_t align_up(std::vector<uint8_t>& b, size_t a) {
  while (b.size() % a) b.push_back(0);
  return b.size();
}

}  // namespace

// ==========================================================================================
// Objects
// ==========================================================================================
struct iree_hal_b200_device_t {
  CUdevice device = 0;
  CUcontext context = nullptr;
  CUstream stream = nullptr;
  // Second stream for collectives that may overlap later dispatches, with the two events that
  // order it against the dispatch stream (created on first use).
  CUstream collective_stream = nullptr;
  CUevent dispatch_done = nullptr, collective_done = nullptr;
  // peer-copy all-gather: copies fan out over these streams (one copy engine each) between two
  // events on the collective stream
  static constexpr int kCopyStreams = 8;
  CUstream copy_streams[kCopyStreams] = {};
  CUevent copy_done[kCopyStreams] = {};
  CUevent copies_go = nullptr;
  // Third stream for device -> host copies that run under the next host -> device copy in the
  // host-buffer entry points (created on first use).
  CUstream readback_stream = nullptr;
  CUevent readback_ready = nullptr;
  CUstream upload_stream = nullptr;  // host -> device copies that run beside the dispatch stream's kernels
  CUevent upload_ready = nullptr;
  int sm_count = 0, cc = 0, max_smem = 0;
  char name[128] = {0};
};

struct iree_hal_b200_executable_t {
  std::atomic<int> references{1};  // iree_hal_resource_t's count (native_executable.c:21-25)
  iree_hal_b200_device_t* device = nullptr;
  CUmodule module = nullptr;
  struct Entry {
    std::string name;
    CUfunction fn;
    uint32_t block[3];
    uint32_t smem;
  };
  std::vector<Entry> entries;
};

struct iree_hal_b200_graph_t {
  iree_hal_b200_device_t* device = nullptr;
  CUgraph graph = nullptr;
  CUgraphExec exec = nullptr;
  uint64_t kernel_nodes = 0;
};

struct iree_hal_b200_command_buffer_t {
  std::atomic<int> references{1};
  iree_hal_b200_device_t* device = nullptr;
  // Graph mode: dispatches become kernel nodes chained one after the other instead of launches.
  CUgraph recording = nullptr;
  CUgraphNode last_node = nullptr;
  uint64_t recorded_nodes = 0;
  // The next dispatches may start before the dispatch ahead of them has finished (programmatic
  // dependent launch); the caller vouches that their exports order themselves on the device.
  bool overlap = false;
  bool open = false;             // between begin and end
  bool barrier_pending = false;  // an execution barrier was recorded: the next dispatch takes a full dependency
  uint32_t constants[IREE_HAL_B200_MAX_PUSH_CONSTANT_COUNT] = {0};
  void* bindings[IREE_HAL_B200_MAX_DESCRIPTOR_SET_COUNT][IREE_HAL_B200_MAX_DESCRIPTOR_SET_BINDING_COUNT] = {{nullptr}};
  uint64_t launches = 0;
};

struct iree_hal_b200_descriptor_set_layout_t {
  uint32_t binding_count = 0;
};
struct iree_hal_b200_pipeline_layout_t {
  // what pipeline_layout.c:178-188 records: every set's binding count and, through the running sum, the
  // index of its first kernel parameter; the push constants follow the last set
  std::vector<uint32_t> set_binding_counts;
  uint32_t push_constant_count = 0;
};

// A timeline semaphore (hal/semaphore.h): a 64-bit payload that only grows. Values are reached by a host
// signal or by the device passing an event that queue_execute recorded behind the work it submitted.
struct iree_hal_b200_semaphore_t {
  std::atomic<int> references{1};
  iree_hal_b200_device_t* device = nullptr;
  std::mutex mutex;
  uint64_t value = 0;
  struct Pending {
    uint64_t value;
    CUevent event;
  };
  std::vector<Pending> pending;  // in submission order: values grow
};

struct iree_hal_b200_channel_t {
  std::atomic<int> references{1};
  iree_hal_b200_device_t* device = nullptr;
  ncclComm_t comm = nullptr;
  int32_t rank = 0, count = 1;
  void* barrier_word = nullptr;  // 4 bytes reduced by the channel barrier (allocated on first use)
};

extern "C" {

const char* iree_b200_last_error(void) { return g_last_error.c_str(); }

int32_t iree_b200_internal_set_error(int32_t code, const char* message) {
  g_last_error = message ? message : "";
  return code;
}

static iree_b200_status_t encode_decode_weight_map(const void* wq, int32_t N, int32_t K, void* out_map);
int32_t iree_b200_internal_encode_decode_weight_map(const void* wq, int32_t N, int32_t K, void* out_map) {
  return encode_decode_weight_map(wq, N, K, out_map);
}

// ---- device ----------------------------------------------------------------------------------
iree_b200_status_t iree_hal_b200_device_create(int32_t ordinal, iree_hal_b200_device_t** out_device) {
  if (!out_device) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "out_device is NULL");
  *out_device = nullptr;
  B200_RETURN_IF_ERROR(ensure_cuda());
  int count = 0;
  CU_RETURN_IF_ERROR(g_cu.cuDeviceGetCount(&count), "cuDeviceGetCount");
  if (ordinal < 0 || ordinal >= count)
    return fail(IREE_B200_STATUS_NOT_FOUND, "device ordinal %d out of range (%d devices)", ordinal, count);
  auto* d = new iree_hal_b200_device_t();
  iree_b200_status_t st = cu_check(g_cu.cuDeviceGet(&d->device, ordinal), "cuDeviceGet");
  if (!st) st = cu_check(g_cu.cuDevicePrimaryCtxRetain(&d->context, d->device), "cuDevicePrimaryCtxRetain");
  if (st) {
    delete d;
    return st;
  }
  st = cu_check(g_cu.cuCtxSetCurrent(d->context), "cuCtxSetCurrent");
  if (!st) st = cu_check(g_cu.cuStreamCreate(&d->stream, CU_STREAM_NON_BLOCKING), "cuStreamCreate");
  int major = 0, minor = 0;
  if (!st) {
    g_cu.cuDeviceGetName(d->name, sizeof d->name, d->device);
    g_cu.cuDeviceGetAttribute(&d->sm_count, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, d->device);
    g_cu.cuDeviceGetAttribute(&major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, d->device);
    g_cu.cuDeviceGetAttribute(&minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, d->device);
    g_cu.cuDeviceGetAttribute(&d->max_smem, CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN, d->device);
    d->cc = major * 10 + minor;
  }
  if (st) {
    g_cu.cuDevicePrimaryCtxRelease(d->device);
    delete d;
    return st;
  }
  *out_device = d;
  return IREE_B200_STATUS_OK;
}

void iree_hal_b200_device_release(iree_hal_b200_device_t* device) {
  if (!device) return;
  g_cu.cuCtxSetCurrent(device->context);
  for (int i = 0; i < iree_hal_b200_device_t::kCopyStreams; ++i) {
    if (device->copy_streams[i]) {
      g_cu.cuStreamSynchronize(device->copy_streams[i]);
      g_cu.cuStreamDestroy(device->copy_streams[i]);
      g_cu.cuEventDestroy(device->copy_done[i]);
    }
  }
  if (device->copies_go) g_cu.cuEventDestroy(device->copies_go);
  if (device->collective_stream) {
    g_cu.cuStreamSynchronize(device->collective_stream);
    g_cu.cuStreamDestroy(device->collective_stream);
    g_cu.cuEventDestroy(device->dispatch_done);
    g_cu.cuEventDestroy(device->collective_done);
  }
  if (device->readback_stream) {
    g_cu.cuStreamSynchronize(device->readback_stream);
    g_cu.cuStreamDestroy(device->readback_stream);
    g_cu.cuEventDestroy(device->readback_ready);
  }
  if (device->upload_stream) {
    g_cu.cuStreamSynchronize(device->upload_stream);
    g_cu.cuStreamDestroy(device->upload_stream);
    g_cu.cuEventDestroy(device->upload_ready);
  }
  if (device->stream) {
    g_cu.cuStreamSynchronize(device->stream);
    g_cu.cuStreamDestroy(device->stream);
  }
  g_cu.cuDevicePrimaryCtxRelease(device->device);
  delete device;
}

iree_b200_status_t iree_hal_b200_device_query(iree_hal_b200_device_t* device, char* name, size_t name_capacity,
                                              int32_t* out_sm_count, int32_t* out_compute_capability,
                                              int32_t* out_max_shared_memory) {
  if (!device) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "device is NULL");
  if (name && name_capacity) snprintf(name, name_capacity, "%s", device->name);
  if (out_sm_count) *out_sm_count = device->sm_count;
  if (out_compute_capability) *out_compute_capability = device->cc;
  if (out_max_shared_memory) *out_max_shared_memory = device->max_smem;
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_device_synchronize(iree_hal_b200_device_t* device) {
  if (!device) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "device is NULL");
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  CU_RETURN_IF_ERROR(g_cu.cuStreamSynchronize(device->stream), "cuStreamSynchronize");
  return IREE_B200_STATUS_OK;
}

void* iree_hal_b200_device_stream(iree_hal_b200_device_t* device) { return device ? device->stream : nullptr; }

// ---- events ----------------------------------------------------------------------------------
iree_b200_status_t iree_hal_b200_event_create(iree_hal_b200_device_t* device, void** out_event) {
  if (!device || !out_event) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  CUevent e = nullptr;
  CU_RETURN_IF_ERROR(g_cu.cuEventCreate(&e, CU_EVENT_DEFAULT), "cuEventCreate");
  *out_event = e;
  return IREE_B200_STATUS_OK;
}
void iree_hal_b200_event_release(iree_hal_b200_device_t* device, void* event) {
  if (device && event) g_cu.cuEventDestroy(static_cast<CUevent>(event));
}
iree_b200_status_t iree_hal_b200_event_record(iree_hal_b200_device_t* device, void* event) {
  if (!device || !event) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  CU_RETURN_IF_ERROR(g_cu.cuEventRecord(static_cast<CUevent>(event), device->stream), "cuEventRecord");
  return IREE_B200_STATUS_OK;
}
iree_b200_status_t iree_hal_b200_event_elapsed_ms(iree_hal_b200_device_t* device, void* start, void* end,
                                                  float* out_ms) {
  if (!device || !start || !end || !out_ms) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  CU_RETURN_IF_ERROR(g_cu.cuEventSynchronize(static_cast<CUevent>(end)), "cuEventSynchronize");
  CU_RETURN_IF_ERROR(g_cu.cuEventElapsedTime(out_ms, static_cast<CUevent>(start), static_cast<CUevent>(end)),
                     "cuEventElapsedTime");
  return IREE_B200_STATUS_OK;
}

// ---- buffers ---------------------------------------------------------------------------------
iree_b200_status_t iree_hal_b200_buffer_allocate(iree_hal_b200_device_t* device, size_t byte_length,
                                                 void** out_device_ptr) {
  if (!device || !out_device_ptr) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  CUdeviceptr p = 0;
  CU_RETURN_IF_ERROR(g_cu.cuMemAlloc(&p, byte_length ? byte_length : 1), "cuMemAlloc");
  *out_device_ptr = reinterpret_cast<void*>(p);
  return IREE_B200_STATUS_OK;
}
iree_b200_status_t iree_hal_b200_buffer_free(iree_hal_b200_device_t* device, void* device_ptr) {
  if (!device) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "device is NULL");
  if (!device_ptr) return IREE_B200_STATUS_OK;
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  CU_RETURN_IF_ERROR(g_cu.cuMemFree(reinterpret_cast<CUdeviceptr>(device_ptr)), "cuMemFree");
  return IREE_B200_STATUS_OK;
}
iree_b200_status_t iree_hal_b200_host_allocate(iree_hal_b200_device_t* device, size_t byte_length,
                                               void** out_pinned_host_ptr) {
  if (!device || !out_pinned_host_ptr) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  CU_RETURN_IF_ERROR(g_cu.cuMemHostAlloc(out_pinned_host_ptr, byte_length ? byte_length : 1, 0), "cuMemHostAlloc");
  return IREE_B200_STATUS_OK;
}
iree_b200_status_t iree_hal_b200_host_free(iree_hal_b200_device_t* device, void* pinned_host_ptr) {
  if (!device) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "device is NULL");
  if (!pinned_host_ptr) return IREE_B200_STATUS_OK;
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  CU_RETURN_IF_ERROR(g_cu.cuMemFreeHost(pinned_host_ptr), "cuMemFreeHost");
  return IREE_B200_STATUS_OK;
}
iree_b200_status_t iree_hal_b200_transfer_h2d(iree_hal_b200_device_t* device, const void* source,
                                              void* target_device_ptr, size_t byte_length) {
  if (!device || (byte_length && (!source || !target_device_ptr)))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if (!byte_length) return IREE_B200_STATUS_OK;
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  CU_RETURN_IF_ERROR(g_cu.cuMemcpyHtoDAsync(reinterpret_cast<CUdeviceptr>(target_device_ptr), source, byte_length,
                                            device->stream),
                     "cuMemcpyHtoDAsync");
  return IREE_B200_STATUS_OK;
}
iree_b200_status_t iree_hal_b200_transfer_d2h(iree_hal_b200_device_t* device, const void* source_device_ptr,
                                              void* target, size_t byte_length) {
  if (!device || (byte_length && (!source_device_ptr || !target)))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if (!byte_length) return IREE_B200_STATUS_OK;
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  CU_RETURN_IF_ERROR(g_cu.cuMemcpyDtoHAsync(target, reinterpret_cast<CUdeviceptr>(source_device_ptr), byte_length,
                                            device->stream),
                     "cuMemcpyDtoHAsync");
  return IREE_B200_STATUS_OK;
}
iree_b200_status_t iree_hal_b200_fill_buffer(iree_hal_b200_device_t* device, void* device_ptr, size_t byte_length,
                                             uint8_t pattern) {
  if (!device || (byte_length && !device_ptr)) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if (!byte_length) return IREE_B200_STATUS_OK;
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  CU_RETURN_IF_ERROR(g_cu.cuMemsetD8Async(reinterpret_cast<CUdeviceptr>(device_ptr), pattern, byte_length,
                                          device->stream),
                     "cuMemsetD8Async");
  return IREE_B200_STATUS_OK;
}

// ---- ExecutableDef writer ----------------------------------------------------------------------
iree_b200_status_t iree_b200_executable_def_build(int32_t entry_count, const char* const* entry_names,
                                                  const uint32_t* block_sizes_xyz,
                                                  const uint32_t* shared_memory_sizes, const void* image,
                                                  size_t image_size, void* out_data, size_t out_capacity,
                                                  size_t* out_size) {
  if (entry_count < 0 || (entry_count && (!entry_names || !block_sizes_xyz || !shared_memory_sizes)) || !out_size)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  // Laid out front to back: header, vtable, table, then the vectors / strings it points at.
  std::vector<uint8_t> b;
  b.resize(8, 0);
  memcpy(b.data() + 4, "CUDA", 4);
  // vtable: size 14 (4 + 5 fields * 2), table size 24 (soffset + 5 uoffsets), field offsets.
  const size_t vt = b.size();
  const uint16_t vtable[7] = {14, 24, 4, 8, 12, 16, 0 /* source_locations absent */};
  b.insert(b.end(), reinterpret_cast<const uint8_t*>(vtable), reinterpret_cast<const uint8_t*>(vtable) + 14);
  b.resize(b.size() + 2, 0);  // pad so the table is 4-byte aligned
  const size_t table = b.size();
  b.resize(table + 24, 0);
  const int32_t soff = static_cast<int32_t>(table - vt);
  memcpy(b.data() + table, &soff, 4);
  put_u32(b, 0, static_cast<uint32_t>(table));

  // entry_points: vector of offsets to strings.
  const size_t vec_entries = align_up(b, 4);
  b.resize(vec_entries + 4 + 4ull * entry_count, 0);
  put_u32(b, vec_entries, static_cast<uint32_t>(entry_count));
  put_u32(b, table + 4, static_cast<uint32_t>(vec_entries - (table + 4)));
  for (int32_t i = 0; i < entry_count; ++i) {
    const char* name = entry_names[i] ? entry_names[i] : "";
    const size_t str = align_up(b, 4);
    const uint32_t len = static_cast<uint32_t>(strlen(name));
    b.resize(str + 4 + len + 1, 0);
    put_u32(b, str, len);
    memcpy(b.data() + str + 4, name, len);
    const size_t slot = vec_entries + 4 + 4ull * i;
    put_u32(b, slot, static_cast<uint32_t>(str - slot));
  }
  // block_sizes: vector of inline structs {x, y, z}.
  const size_t vec_blocks = align_up(b, 4);
  b.resize(vec_blocks + 4 + 12ull * entry_count, 0);
  put_u32(b, vec_blocks, static_cast<uint32_t>(entry_count));
  if (entry_count) memcpy(b.data() + vec_blocks + 4, block_sizes_xyz, 12ull * entry_count);
  put_u32(b, table + 8, static_cast<uint32_t>(vec_blocks - (table + 8)));
  // shared_memory_size: vector of u32.
  const size_t vec_smem = align_up(b, 4);
  b.resize(vec_smem + 4 + 4ull * entry_count, 0);
  put_u32(b, vec_smem, static_cast<uint32_t>(entry_count));
  if (entry_count) memcpy(b.data() + vec_smem + 4, shared_memory_sizes, 4ull * entry_count);
  put_u32(b, table + 12, static_cast<uint32_t>(vec_smem - (table + 12)));
  // ptx_image: a string with an explicit length, so binary images are safe.
  const size_t str_image = align_up(b, 4);
  b.resize(str_image + 4 + image_size + 1, 0);
  put_u32(b, str_image, static_cast<uint32_t>(image_size));
  if (image_size) memcpy(b.data() + str_image + 4, image, image_size);
  put_u32(b, table + 16, static_cast<uint32_t>(str_image - (table + 16)));

  *out_size = b.size();
  if (!out_data) return IREE_B200_STATUS_OK;
  if (out_capacity < b.size())
    return fail(IREE_B200_STATUS_OUT_OF_RANGE, "output buffer too small: %zu < %zu", out_capacity, b.size());
  memcpy(out_data, b.data(), b.size());
  return IREE_B200_STATUS_OK;
}

// ---- executable ---------------------------------------------------------------------------------
iree_b200_status_t iree_hal_b200_executable_create(iree_hal_b200_device_t* device, const char* executable_format,
                                                   const void* executable_data, size_t executable_data_size,
                                                   iree_hal_b200_executable_t** out_executable) {
  if (!out_executable) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "out_executable is NULL");
  *out_executable = nullptr;
  if (!executable_format || strcmp(executable_format, "PTXE") != 0)
    return fail(IREE_B200_STATUS_NOT_FOUND, "no executable implementation registered for the given format '%s'",
                executable_format ? executable_format : "(null)");
  ExecutableDefView view;
  B200_RETURN_IF_ERROR(parse_executable_def(executable_data, executable_data_size, &view));
  if (!device) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "device is NULL");
  for (size_t i = 0; i < view.entry_points.size(); ++i) {
    const uint32_t smem = i < view.shared_memory.size() ? view.shared_memory[i] : 0;
    if (smem > static_cast<uint32_t>(device->max_smem))
      return fail(IREE_B200_STATUS_RESOURCE_EXHAUSTED,
                  "function '%s' requested shared memory size of %u bytes larger than allowed size of %d bytes",
                  view.entry_points[i].c_str(), smem, device->max_smem);
  }
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  auto* exe = new iree_hal_b200_executable_t();
  exe->device = device;
  // The image may be PTX text or a cubin; the driver tells them apart (native_executable.c:174-176).
  std::vector<uint8_t> image(view.image, view.image + view.image_size);
  image.push_back(0);
  iree_b200_status_t st = cu_check(g_cu.cuModuleLoadDataEx(&exe->module, image.data(), 0, nullptr, nullptr),
                                   "cuModuleLoadDataEx");
  for (size_t i = 0; !st && i < view.entry_points.size(); ++i) {
    iree_hal_b200_executable_t::Entry e;
    e.name = view.entry_points[i];
    memcpy(e.block, &view.block_sizes[3 * i], 12);
    e.smem = i < view.shared_memory.size() ? view.shared_memory[i] : 0;
    st = cu_check(g_cu.cuModuleGetFunction(&e.fn, exe->module, e.name.c_str()), e.name.c_str());
    if (!st && e.smem)
      st = cu_check(g_cu.cuFuncSetAttribute(e.fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                            static_cast<int>(e.smem)),
                    "cuFuncSetAttribute(MAX_DYNAMIC_SHARED_SIZE_BYTES)");
    if (!st) exe->entries.push_back(e);
  }
  if (st) {
    if (exe->module) g_cu.cuModuleUnload(exe->module);
    delete exe;
    return st;
  }
  *out_executable = exe;
  return IREE_B200_STATUS_OK;
}

void iree_hal_b200_executable_retain(iree_hal_b200_executable_t* executable) {
  if (executable) executable->references.fetch_add(1);
}
void iree_hal_b200_executable_release(iree_hal_b200_executable_t* executable) {
  if (!executable || executable->references.fetch_sub(1) != 1) return;
  g_cu.cuCtxSetCurrent(executable->device->context);
  if (executable->module) g_cu.cuModuleUnload(executable->module);
  delete executable;
}
int32_t iree_hal_b200_executable_entry_count(const iree_hal_b200_executable_t* executable) {
  return executable ? static_cast<int32_t>(executable->entries.size()) : 0;
}
int32_t iree_hal_b200_executable_lookup(const iree_hal_b200_executable_t* executable, const char* entry_name) {
  if (!executable || !entry_name) return -1;
  for (size_t i = 0; i < executable->entries.size(); ++i)
    if (executable->entries[i].name == entry_name) return static_cast<int32_t>(i);
  return -1;
}

// ---- command buffer -------------------------------------------------------------------------------
iree_b200_status_t iree_hal_b200_command_buffer_create(iree_hal_b200_device_t* device,
                                                       iree_hal_b200_command_buffer_t** out_command_buffer) {
  if (!device || !out_command_buffer) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  auto* cb = new iree_hal_b200_command_buffer_t();
  cb->device = device;
  *out_command_buffer = cb;
  return IREE_B200_STATUS_OK;
}
void iree_hal_b200_command_buffer_retain(iree_hal_b200_command_buffer_t* command_buffer) {
  if (command_buffer) command_buffer->references.fetch_add(1);
}
void iree_hal_b200_command_buffer_release(iree_hal_b200_command_buffer_t* command_buffer) {
  if (command_buffer && command_buffer->references.fetch_sub(1) == 1) delete command_buffer;
}

iree_b200_status_t iree_hal_b200_command_buffer_push_constants(iree_hal_b200_command_buffer_t* command_buffer,
                                                               size_t offset, const void* values,
                                                               size_t values_length) {
  if (!command_buffer || (values_length && !values)) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if ((offset % 4) || (values_length % 4))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "push constant offset/length must be multiples of 4 bytes");
  if (offset + values_length > sizeof command_buffer->constants)
    return fail(IREE_B200_STATUS_OUT_OF_RANGE, "push constant range [%zu, %zu) exceeds the %d-constant limit", offset,
                offset + values_length, IREE_HAL_B200_MAX_PUSH_CONSTANT_COUNT);
  memcpy(reinterpret_cast<uint8_t*>(command_buffer->constants) + offset, values, values_length);
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_command_buffer_push_descriptor_set(
    iree_hal_b200_command_buffer_t* command_buffer, uint32_t set, size_t binding_count,
    const iree_hal_b200_descriptor_set_binding_t* bindings) {
  if (!command_buffer || (binding_count && !bindings)) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if (set >= IREE_HAL_B200_MAX_DESCRIPTOR_SET_COUNT)
    return fail(IREE_B200_STATUS_OUT_OF_RANGE, "descriptor set %u out of range", set);
  for (size_t i = 0; i < binding_count; ++i) {
    if (bindings[i].binding >= IREE_HAL_B200_MAX_DESCRIPTOR_SET_BINDING_COUNT)
      return fail(IREE_B200_STATUS_OUT_OF_RANGE, "binding %u out of range", bindings[i].binding);
    command_buffer->bindings[set][bindings[i].binding] = bindings[i].device_ptr;
  }
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_command_buffer_dispatch(iree_hal_b200_command_buffer_t* command_buffer,
                                                         iree_hal_b200_executable_t* executable, int32_t entry_point,
                                                         uint32_t binding_count, uint32_t constant_count,
                                                         uint32_t workgroup_x, uint32_t workgroup_y,
                                                         uint32_t workgroup_z) {
  if (!command_buffer || !executable) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if (entry_point < 0 || entry_point >= static_cast<int32_t>(executable->entries.size()))
    return fail(IREE_B200_STATUS_OUT_OF_RANGE, "entry point ordinal %d out of range (%zu entries)", entry_point,
                executable->entries.size());
  if (binding_count > IREE_HAL_B200_MAX_DESCRIPTOR_SET_BINDING_COUNT ||
      constant_count > IREE_HAL_B200_MAX_PUSH_CONSTANT_COUNT)
    return fail(IREE_B200_STATUS_OUT_OF_RANGE, "binding / constant count exceeds the pipeline layout limits");
  if (!workgroup_x || !workgroup_y || !workgroup_z) return IREE_B200_STATUS_OK;  // empty dispatch
  const auto& e = executable->entries[entry_point];
  // Kernel parameters: every binding as a device pointer, then each constant on its own
  // (stream_command_buffer.c:538-594).
  void* params[IREE_HAL_B200_MAX_DESCRIPTOR_SET_BINDING_COUNT + IREE_HAL_B200_MAX_PUSH_CONSTANT_COUNT];
  for (uint32_t i = 0; i < binding_count; ++i) params[i] = &command_buffer->bindings[0][i];
  for (uint32_t i = 0; i < constant_count; ++i) params[binding_count + i] = &command_buffer->constants[i];
  iree_hal_b200_device_t* d = command_buffer->device;
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(d->context), "cuCtxSetCurrent");
  if (command_buffer->recording) {
    // Same parameter packing, recorded as a graph node (graph_command_buffer.c:747-829); the
    // driver copies the parameter values when the node is added.
    CUDA_KERNEL_NODE_PARAMS np;
    memset(&np, 0, sizeof np);
    np.func = e.fn;
    np.gridDimX = workgroup_x;
    np.gridDimY = workgroup_y;
    np.gridDimZ = workgroup_z;
    np.blockDimX = e.block[0];
    np.blockDimY = e.block[1];
    np.blockDimZ = e.block[2];
    np.sharedMemBytes = e.smem;
    np.kernelParams = params;
    CUgraphNode node = nullptr;
    const bool programmatic = command_buffer->overlap && command_buffer->last_node && !command_buffer->barrier_pending;
    command_buffer->barrier_pending = false;
    CU_RETURN_IF_ERROR(g_cu.cuGraphAddKernelNode(&node, command_buffer->recording,
                                                 command_buffer->last_node && !programmatic ? &command_buffer->last_node : nullptr,
                                                 command_buffer->last_node && !programmatic ? 1 : 0, &np),
                       "cuGraphAddKernelNode");
    if (programmatic) {
      // The edge leaves the upstream kernel's programmatic port: this node may be launched once
      // every upstream block has released its dependents (or exited), and waits on the device
      // (griddepcontrol.wait) before it touches anything the upstream kernel produces.
      CUgraphEdgeData edge;
      memset(&edge, 0, sizeof edge);
      edge.from_port = CU_GRAPH_KERNEL_NODE_PORT_PROGRAMMATIC;
      edge.to_port = 0;
      edge.type = CU_GRAPH_DEPENDENCY_TYPE_PROGRAMMATIC;
      CU_RETURN_IF_ERROR(g_cu.cuGraphAddDependencies_v2(command_buffer->recording, &command_buffer->last_node, &node,
                                                        &edge, 1),
                         "cuGraphAddDependencies");
    }
    command_buffer->last_node = node;
    ++command_buffer->recorded_nodes;
    return IREE_B200_STATUS_OK;
  }
  const bool early = command_buffer->overlap && !command_buffer->barrier_pending;
  command_buffer->barrier_pending = false;
  if (early) {
    CUlaunchConfig config;
    memset(&config, 0, sizeof config);
    config.gridDimX = workgroup_x;
    config.gridDimY = workgroup_y;
    config.gridDimZ = workgroup_z;
    config.blockDimX = e.block[0];
    config.blockDimY = e.block[1];
    config.blockDimZ = e.block[2];
    config.sharedMemBytes = e.smem;
    config.hStream = d->stream;
    CUlaunchAttribute attr;
    memset(&attr, 0, sizeof attr);
    attr.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
    attr.value.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attr;
    config.numAttrs = 1;
    CU_RETURN_IF_ERROR(g_cu.cuLaunchKernelEx(&config, e.fn, params, nullptr), e.name.c_str());
  } else {
    CU_RETURN_IF_ERROR(g_cu.cuLaunchKernel(e.fn, workgroup_x, workgroup_y, workgroup_z, e.block[0], e.block[1],
                                           e.block[2], e.smem, d->stream, params, nullptr),
                       e.name.c_str());
  }
  ++command_buffer->launches;
  return IREE_B200_STATUS_OK;
}

// ---- begin / end, barriers, transfer commands ---------------------------------------------------------
iree_b200_status_t iree_hal_b200_command_buffer_begin(iree_hal_b200_command_buffer_t* command_buffer) {
  if (!command_buffer) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "command_buffer is NULL");
  if (command_buffer->open) return fail(IREE_B200_STATUS_FAILED_PRECONDITION, "command buffer is already recording");
  command_buffer->open = true;
  return IREE_B200_STATUS_OK;
}
iree_b200_status_t iree_hal_b200_command_buffer_end(iree_hal_b200_command_buffer_t* command_buffer) {
  if (!command_buffer) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "command_buffer is NULL");
  if (!command_buffer->open) return fail(IREE_B200_STATUS_FAILED_PRECONDITION, "command buffer is not recording");
  command_buffer->open = false;
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_command_buffer_execution_barrier(iree_hal_b200_command_buffer_t* command_buffer,
                                                                  uint32_t source_stage_mask, uint32_t target_stage_mask,
                                                                  uint32_t flags) {
  if (!command_buffer) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "command_buffer is NULL");
  (void)source_stage_mask;
  (void)target_stage_mask;
  (void)flags;
  // Commands already execute in recording order (one stream; a linear chain of graph nodes). What a
  // barrier changes here: the dispatch after it is not launched early, whatever the overlap setting.
  command_buffer->barrier_pending = true;
  return IREE_B200_STATUS_OK;
}

// A transfer command as a node of the recording (after the previous node) or on the dispatch stream.
static iree_b200_status_t chain_node(iree_hal_b200_command_buffer_t* cb, CUgraphNode node) {
  cb->last_node = node;
  ++cb->recorded_nodes;
  cb->barrier_pending = true;  // a kernel may not be launched early behind a copy or a fill
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_command_buffer_fill_buffer(iree_hal_b200_command_buffer_t* command_buffer,
                                                            void* target_device_ptr, size_t target_offset, size_t length,
                                                            const void* pattern, size_t pattern_length) {
  if (!command_buffer || !pattern) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if (pattern_length != 1 && pattern_length != 2 && pattern_length != 4)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "fill patterns must be 1, 2 or 4 bytes long (got %zu)", pattern_length);
  if ((target_offset % pattern_length) || (length % pattern_length))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "fill offset and length must be aligned to the pattern length");
  if (!length) return IREE_B200_STATUS_OK;
  if (!target_device_ptr) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "target buffer is NULL");
  uint32_t value = 0;
  memcpy(&value, pattern, pattern_length);
  iree_hal_b200_device_t* d = command_buffer->device;
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(d->context), "cuCtxSetCurrent");
  const CUdeviceptr dst = reinterpret_cast<CUdeviceptr>(static_cast<uint8_t*>(target_device_ptr) + target_offset);
  const size_t count = length / pattern_length;
  if (command_buffer->recording) {
    if (!g_cu.cuGraphAddMemsetNode) return fail(IREE_B200_STATUS_UNAVAILABLE, "this CUDA driver has no cuGraphAddMemsetNode");
    CUDA_MEMSET_NODE_PARAMS mp;
    memset(&mp, 0, sizeof mp);
    mp.dst = dst;
    mp.elementSize = static_cast<unsigned>(pattern_length);
    mp.value = value;
    mp.width = count;
    mp.height = 1;
    CUgraphNode node = nullptr;
    CU_RETURN_IF_ERROR(g_cu.cuGraphAddMemsetNode(&node, command_buffer->recording,
                                                 command_buffer->last_node ? &command_buffer->last_node : nullptr,
                                                 command_buffer->last_node ? 1 : 0, &mp, d->context),
                       "cuGraphAddMemsetNode");
    return chain_node(command_buffer, node);
  }
  command_buffer->barrier_pending = true;
  if (pattern_length == 1) {
    CU_RETURN_IF_ERROR(g_cu.cuMemsetD8Async(dst, static_cast<unsigned char>(value), count, d->stream), "cuMemsetD8Async");
  } else if (pattern_length == 2) {
    if (!g_cu.cuMemsetD16Async) return fail(IREE_B200_STATUS_UNAVAILABLE, "this CUDA driver has no cuMemsetD16Async");
    CU_RETURN_IF_ERROR(g_cu.cuMemsetD16Async(dst, static_cast<unsigned short>(value), count, d->stream), "cuMemsetD16Async");
  } else {
    if (!g_cu.cuMemsetD32Async) return fail(IREE_B200_STATUS_UNAVAILABLE, "this CUDA driver has no cuMemsetD32Async");
    CU_RETURN_IF_ERROR(g_cu.cuMemsetD32Async(dst, value, count, d->stream), "cuMemsetD32Async");
  }
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_command_buffer_copy_buffer(iree_hal_b200_command_buffer_t* command_buffer,
                                                            const void* source_device_ptr, size_t source_offset,
                                                            void* target_device_ptr, size_t target_offset, size_t length) {
  if (!command_buffer) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "command_buffer is NULL");
  if (!length) return IREE_B200_STATUS_OK;
  if (!source_device_ptr || !target_device_ptr) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "buffer pointer is NULL");
  const uint8_t* src = static_cast<const uint8_t*>(source_device_ptr) + source_offset;
  uint8_t* dst = static_cast<uint8_t*>(target_device_ptr) + target_offset;
  if (src < dst + length && dst < src + length)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "source and target ranges of a copy must not overlap");
  iree_hal_b200_device_t* d = command_buffer->device;
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(d->context), "cuCtxSetCurrent");
  if (command_buffer->recording) {
    if (!g_cu.cuGraphAddMemcpyNode) return fail(IREE_B200_STATUS_UNAVAILABLE, "this CUDA driver has no cuGraphAddMemcpyNode");
    CUDA_MEMCPY3D cp;
    memset(&cp, 0, sizeof cp);
    cp.srcMemoryType = CU_MEMORYTYPE_DEVICE;
    cp.srcDevice = reinterpret_cast<CUdeviceptr>(src);
    cp.dstMemoryType = CU_MEMORYTYPE_DEVICE;
    cp.dstDevice = reinterpret_cast<CUdeviceptr>(dst);
    cp.WidthInBytes = length;
    cp.Height = 1;
    cp.Depth = 1;
    CUgraphNode node = nullptr;
    CU_RETURN_IF_ERROR(g_cu.cuGraphAddMemcpyNode(&node, command_buffer->recording,
                                                 command_buffer->last_node ? &command_buffer->last_node : nullptr,
                                                 command_buffer->last_node ? 1 : 0, &cp, d->context),
                       "cuGraphAddMemcpyNode");
    return chain_node(command_buffer, node);
  }
  if (!g_cu.cuMemcpyDtoDAsync) return fail(IREE_B200_STATUS_UNAVAILABLE, "this CUDA driver has no cuMemcpyDtoDAsync");
  command_buffer->barrier_pending = true;
  CU_RETURN_IF_ERROR(g_cu.cuMemcpyDtoDAsync(reinterpret_cast<CUdeviceptr>(dst), reinterpret_cast<CUdeviceptr>(src), length,
                                            d->stream),
                     "cuMemcpyDtoDAsync");
  return IREE_B200_STATUS_OK;
}

// ---- pipeline layouts ------------------------------------------------------------------------------
iree_b200_status_t iree_hal_b200_descriptor_set_layout_create(iree_hal_b200_device_t* device, uint32_t binding_count,
                                                              iree_hal_b200_descriptor_set_layout_t** out_layout) {
  if (!device || !out_layout) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  *out_layout = nullptr;
  if (binding_count > IREE_HAL_B200_MAX_DESCRIPTOR_SET_BINDING_COUNT)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "binding count %u over the limit of %d", binding_count,
                IREE_HAL_B200_MAX_DESCRIPTOR_SET_BINDING_COUNT);
  auto* l = new iree_hal_b200_descriptor_set_layout_t();
  l->binding_count = binding_count;
  *out_layout = l;
  return IREE_B200_STATUS_OK;
}
void iree_hal_b200_descriptor_set_layout_release(iree_hal_b200_descriptor_set_layout_t* layout) { delete layout; }

iree_b200_status_t iree_hal_b200_pipeline_layout_create(iree_hal_b200_device_t* device, uint32_t push_constant_count,
                                                        uint32_t set_layout_count,
                                                        iree_hal_b200_descriptor_set_layout_t* const* set_layouts,
                                                        iree_hal_b200_pipeline_layout_t** out_layout) {
  if (!device || !out_layout || (set_layout_count && !set_layouts)) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  *out_layout = nullptr;
  if (push_constant_count > IREE_HAL_B200_MAX_PUSH_CONSTANT_COUNT)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "push constant count %u over the limit of %d", push_constant_count,
                IREE_HAL_B200_MAX_PUSH_CONSTANT_COUNT);
  if (set_layout_count > IREE_HAL_B200_MAX_DESCRIPTOR_SET_COUNT)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "descriptor set count %u over the limit of %d", set_layout_count,
                IREE_HAL_B200_MAX_DESCRIPTOR_SET_COUNT);
  auto* l = new iree_hal_b200_pipeline_layout_t();
  l->push_constant_count = push_constant_count;
  for (uint32_t i = 0; i < set_layout_count; ++i) {
    if (!set_layouts[i]) {
      delete l;
      return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "descriptor set layout %u is NULL", i);
    }
    l->set_binding_counts.push_back(set_layouts[i]->binding_count);  // copied: the set layout may be released
  }
  *out_layout = l;
  return IREE_B200_STATUS_OK;
}
void iree_hal_b200_pipeline_layout_release(iree_hal_b200_pipeline_layout_t* layout) { delete layout; }

iree_b200_status_t iree_hal_b200_command_buffer_dispatch_with_layout(iree_hal_b200_command_buffer_t* command_buffer,
                                                                     iree_hal_b200_executable_t* executable,
                                                                     int32_t entry_point,
                                                                     const iree_hal_b200_pipeline_layout_t* layout,
                                                                     uint32_t workgroup_x, uint32_t workgroup_y,
                                                                     uint32_t workgroup_z) {
  if (!command_buffer || !layout) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  // Kernel parameters: the bindings of set 0, then of set 1, ... (each set's first parameter index is the
  // running sum of the binding counts before it), then the push constants. The sets are flattened into
  // the slots of set 0 for the launch and put back afterwards.
  void* saved[IREE_HAL_B200_MAX_DESCRIPTOR_SET_BINDING_COUNT];
  memcpy(saved, command_buffer->bindings[0], sizeof saved);
  uint32_t total = 0;
  void* flat[IREE_HAL_B200_MAX_DESCRIPTOR_SET_BINDING_COUNT];
  for (size_t set = 0; set < layout->set_binding_counts.size(); ++set) {
    for (uint32_t b = 0; b < layout->set_binding_counts[set]; ++b) {
      if (total >= IREE_HAL_B200_MAX_DESCRIPTOR_SET_BINDING_COUNT)
        return fail(IREE_B200_STATUS_OUT_OF_RANGE, "the layout's sets hold more than %d bindings",
                    IREE_HAL_B200_MAX_DESCRIPTOR_SET_BINDING_COUNT);
      flat[total++] = command_buffer->bindings[set][b];
    }
  }
  memcpy(command_buffer->bindings[0], flat, total * sizeof(void*));
  const iree_b200_status_t st = iree_hal_b200_command_buffer_dispatch(command_buffer, executable, entry_point, total,
                                                                      layout->push_constant_count, workgroup_x, workgroup_y,
                                                                      workgroup_z);
  memcpy(command_buffer->bindings[0], saved, sizeof saved);
  return st;
}

iree_b200_status_t iree_hal_b200_command_buffer_set_dispatch_overlap(iree_hal_b200_command_buffer_t* command_buffer,
                                                                     int32_t enable) {
  if (!command_buffer) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "command buffer is NULL");
  if (enable) {
    B200_RETURN_IF_ERROR(ensure_cuda());
    if (!g_cu.cuLaunchKernelEx || !g_cu.cuGraphAddDependencies_v2)
      return fail(IREE_B200_STATUS_UNAVAILABLE, "this CUDA driver has no programmatic dependent launch");
  }
  command_buffer->overlap = enable != 0;
  return IREE_B200_STATUS_OK;
}

uint64_t iree_hal_b200_command_buffer_launch_count(const iree_hal_b200_command_buffer_t* command_buffer) {
  return command_buffer ? command_buffer->launches : 0;
}

// ---- graph mode -----------------------------------------------------------------------------------
iree_b200_status_t iree_hal_b200_command_buffer_begin_graph(iree_hal_b200_command_buffer_t* command_buffer) {
  if (!command_buffer) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "command buffer is NULL");
  if (command_buffer->recording) return fail(IREE_B200_STATUS_FAILED_PRECONDITION, "a graph is already being recorded");
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(command_buffer->device->context), "cuCtxSetCurrent");
  CU_RETURN_IF_ERROR(g_cu.cuGraphCreate(&command_buffer->recording, 0), "cuGraphCreate");
  command_buffer->last_node = nullptr;
  command_buffer->recorded_nodes = 0;
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_command_buffer_end_graph(iree_hal_b200_command_buffer_t* command_buffer,
                                                          iree_hal_b200_graph_t** out_graph) {
  if (!command_buffer || !out_graph) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  *out_graph = nullptr;
  if (!command_buffer->recording) return fail(IREE_B200_STATUS_FAILED_PRECONDITION, "no graph is being recorded");
  auto* g = new iree_hal_b200_graph_t();
  g->device = command_buffer->device;
  g->graph = command_buffer->recording;
  g->kernel_nodes = command_buffer->recorded_nodes;
  command_buffer->recording = nullptr;
  command_buffer->last_node = nullptr;
  iree_b200_status_t st = cu_check(g_cu.cuGraphInstantiateWithFlags(&g->exec, g->graph, 0), "cuGraphInstantiate");
  if (st) {
    g_cu.cuGraphDestroy(g->graph);
    delete g;
    return st;
  }
  *out_graph = g;
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_graph_execute(iree_hal_b200_command_buffer_t* command_buffer,
                                               iree_hal_b200_graph_t* graph) {
  if (!command_buffer || !graph) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(graph->device->context), "cuCtxSetCurrent");
  CU_RETURN_IF_ERROR(g_cu.cuGraphLaunch(graph->exec, graph->device->stream), "cuGraphLaunch");
  command_buffer->launches += graph->kernel_nodes;
  return IREE_B200_STATUS_OK;
}

void iree_hal_b200_graph_release(iree_hal_b200_graph_t* graph) {
  if (!graph) return;
  g_cu.cuCtxSetCurrent(graph->device->context);
  if (graph->exec) g_cu.cuGraphExecDestroy(graph->exec);
  if (graph->graph) g_cu.cuGraphDestroy(graph->graph);
  delete graph;
}

// ---- semaphores and queue submission ------------------------------------------------------------------
iree_b200_status_t iree_hal_b200_semaphore_create(iree_hal_b200_device_t* device, uint64_t initial_value,
                                                  iree_hal_b200_semaphore_t** out_semaphore) {
  if (!device || !out_semaphore) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  auto* sem = new iree_hal_b200_semaphore_t();
  sem->device = device;
  sem->value = initial_value;
  *out_semaphore = sem;
  return IREE_B200_STATUS_OK;
}
void iree_hal_b200_semaphore_retain(iree_hal_b200_semaphore_t* semaphore) {
  if (semaphore) semaphore->references.fetch_add(1);
}
void iree_hal_b200_semaphore_release(iree_hal_b200_semaphore_t* semaphore) {
  if (!semaphore || semaphore->references.fetch_sub(1) != 1) return;
  g_cu.cuCtxSetCurrent(semaphore->device->context);
  for (auto& p : semaphore->pending) g_cu.cuEventDestroy(p.event);
  delete semaphore;
}

// Retires the pending device signals the device has passed; the caller holds the mutex.
static iree_b200_status_t semaphore_advance(iree_hal_b200_semaphore_t* sem) {
  if (sem->pending.empty()) return IREE_B200_STATUS_OK;
  if (!g_cu.cuEventQuery) return fail(IREE_B200_STATUS_UNAVAILABLE, "this CUDA driver has no cuEventQuery");
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(sem->device->context), "cuCtxSetCurrent");
  while (!sem->pending.empty()) {
    const CUresult r = g_cu.cuEventQuery(sem->pending.front().event);
    if (r == CUDA_ERROR_NOT_READY) break;
    CU_RETURN_IF_ERROR(r, "cuEventQuery");
    if (sem->pending.front().value > sem->value) sem->value = sem->pending.front().value;
    g_cu.cuEventDestroy(sem->pending.front().event);
    sem->pending.erase(sem->pending.begin());
  }
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_semaphore_query(iree_hal_b200_semaphore_t* semaphore, uint64_t* out_value) {
  if (!semaphore || !out_value) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  std::lock_guard<std::mutex> lock(semaphore->mutex);
  B200_RETURN_IF_ERROR(semaphore_advance(semaphore));
  *out_value = semaphore->value;
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_semaphore_signal(iree_hal_b200_semaphore_t* semaphore, uint64_t new_value) {
  if (!semaphore) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "semaphore is NULL");
  std::lock_guard<std::mutex> lock(semaphore->mutex);
  B200_RETURN_IF_ERROR(semaphore_advance(semaphore));
  if (new_value <= semaphore->value)
    return fail(IREE_B200_STATUS_OUT_OF_RANGE, "semaphore values must be monotonically increasing: %llu is not above %llu",
                static_cast<unsigned long long>(new_value), static_cast<unsigned long long>(semaphore->value));
  semaphore->value = new_value;
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_semaphore_wait(iree_hal_b200_semaphore_t* semaphore, uint64_t value, int64_t timeout_ms) {
  if (!semaphore) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "semaphore is NULL");
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms);
  while (true) {
    CUevent wait_on = nullptr;
    {
      std::lock_guard<std::mutex> lock(semaphore->mutex);
      B200_RETURN_IF_ERROR(semaphore_advance(semaphore));
      if (semaphore->value >= value) return IREE_B200_STATUS_OK;
      for (auto& p : semaphore->pending)
        if (p.value >= value) {
          wait_on = p.event;
          break;
        }
    }
    if (timeout_ms >= 0 && std::chrono::steady_clock::now() >= deadline)
      return fail(IREE_B200_STATUS_DEADLINE_EXCEEDED, "semaphore did not reach %llu in %lld ms",
                  static_cast<unsigned long long>(value), static_cast<long long>(timeout_ms));
    // A queued device signal will reach the value: sleep briefly between queries (the event is owned by the
    // semaphore and may be retired by another thread, so it is not waited on directly). Otherwise only a host
    // signal can: poll for it.
    (void)wait_on;
    std::this_thread::sleep_for(std::chrono::microseconds(wait_on ? 20 : 200));
  }
}

iree_b200_status_t iree_hal_b200_device_queue_execute(iree_hal_b200_device_t* device, size_t wait_count,
                                                      iree_hal_b200_semaphore_t* const* wait_semaphores,
                                                      const uint64_t* wait_values, size_t signal_count,
                                                      iree_hal_b200_semaphore_t* const* signal_semaphores,
                                                      const uint64_t* signal_values, size_t graph_count,
                                                      iree_hal_b200_graph_t* const* graphs) {
  if (!device) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "device is NULL");
  if ((wait_count && (!wait_semaphores || !wait_values)) || (signal_count && (!signal_semaphores || !signal_values)) ||
      (graph_count && !graphs))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL list");
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  // Waits: a value already reached needs nothing; one a queued device signal will reach is waited for by the
  // stream; one only the host can still signal holds this call (at most ten seconds).
  for (size_t i = 0; i < wait_count; ++i) {
    iree_hal_b200_semaphore_t* sem = wait_semaphores[i];
    if (!sem) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "wait semaphore %zu is NULL", i);
    bool satisfied = false;
    {
      std::lock_guard<std::mutex> lock(sem->mutex);
      B200_RETURN_IF_ERROR(semaphore_advance(sem));
      if (sem->value >= wait_values[i]) satisfied = true;
      for (auto& p : sem->pending)
        if (!satisfied && p.value >= wait_values[i]) {
          CU_RETURN_IF_ERROR(g_cu.cuStreamWaitEvent(device->stream, p.event, 0), "cuStreamWaitEvent");
          satisfied = true;
        }
    }
    if (!satisfied) B200_RETURN_IF_ERROR(iree_hal_b200_semaphore_wait(sem, wait_values[i], 10000));
  }
  for (size_t i = 0; i < graph_count; ++i) {
    if (!graphs[i]) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "command buffer %zu is NULL", i);
    CU_RETURN_IF_ERROR(g_cu.cuGraphLaunch(graphs[i]->exec, device->stream), "cuGraphLaunch");
  }
  for (size_t i = 0; i < signal_count; ++i) {
    iree_hal_b200_semaphore_t* sem = signal_semaphores[i];
    if (!sem) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "signal semaphore %zu is NULL", i);
    std::lock_guard<std::mutex> lock(sem->mutex);
    const uint64_t last = sem->pending.empty() ? sem->value : sem->pending.back().value;
    if (signal_values[i] <= last)
      return fail(IREE_B200_STATUS_OUT_OF_RANGE, "semaphore values must be monotonically increasing");
    CUevent ev = nullptr;
    CU_RETURN_IF_ERROR(g_cu.cuEventCreate(&ev, CU_EVENT_DISABLE_TIMING), "cuEventCreate");
    const CUresult r = g_cu.cuEventRecord(ev, device->stream);
    if (r != CUDA_SUCCESS) {
      g_cu.cuEventDestroy(ev);
      CU_RETURN_IF_ERROR(r, "cuEventRecord");
    }
    sem->pending.push_back({signal_values[i], ev});
  }
  return IREE_B200_STATUS_OK;
}

// ---- channel ------------------------------------------------------------------------------------------
iree_b200_status_t iree_hal_b200_channel_create_id(void* out_id, size_t id_capacity) {
  if (!out_id || id_capacity < IREE_HAL_B200_CHANNEL_ID_SIZE)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "channel id buffer must hold %d bytes", IREE_HAL_B200_CHANNEL_ID_SIZE);
  B200_RETURN_IF_ERROR(ensure_nccl());
  ncclUniqueId id;
  B200_RETURN_IF_ERROR(nccl_check(g_nccl.ncclGetUniqueId(&id), "ncclGetUniqueId"));
  memcpy(out_id, &id, sizeof id);
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_channel_create(iree_hal_b200_device_t* device, const void* id, size_t id_size,
                                                int32_t rank, int32_t count,
                                                iree_hal_b200_channel_t** out_channel) {
  if (!out_channel) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "out_channel is NULL");
  *out_channel = nullptr;
  if (!device) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "device is NULL");
  if (!id || id_size != IREE_HAL_B200_CHANNEL_ID_SIZE)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NCCL ID must be %d bytes matching the ncclUniqueId struct but caller provided %zu bytes",
                IREE_HAL_B200_CHANNEL_ID_SIZE, id_size);
  if (count < 1 || rank < 0 || rank >= count)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "rank %d out of range for a channel of %d participants", rank, count);
  B200_RETURN_IF_ERROR(ensure_nccl());
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  ncclUniqueId nid;
  memcpy(&nid, id, sizeof nid);
  auto* ch = new iree_hal_b200_channel_t();
  ch->device = device;
  ch->rank = rank;
  ch->count = count;
  iree_b200_status_t st = nccl_check(g_nccl.ncclCommInitRank(&ch->comm, count, nid, rank), "ncclCommInitRank");
  if (st) {
    delete ch;
    return st;
  }
  *out_channel = ch;
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_channel_split(iree_hal_b200_channel_t* base_channel, int32_t color, int32_t key,
                                               iree_hal_b200_channel_t** out_channel) {
  if (!out_channel) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "out_channel is NULL");
  *out_channel = nullptr;
  if (!base_channel) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "base_channel is NULL");
  B200_RETURN_IF_ERROR(ensure_nccl());
  if (!g_nccl.ncclCommSplit || !g_nccl.ncclCommCount || !g_nccl.ncclCommUserRank)
    return fail(IREE_B200_STATUS_UNAVAILABLE, "this NCCL has no ncclCommSplit");
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(base_channel->device->context), "cuCtxSetCurrent");
  ncclComm_t comm = nullptr;
  // a negative color is NCCL_SPLIT_NOCOLOR: the rank takes part in the call and gets no channel
  B200_RETURN_IF_ERROR(nccl_check(g_nccl.ncclCommSplit(base_channel->comm, color < 0 ? -1 : color, key, &comm, nullptr),
                                  "ncclCommSplit"));
  if (color < 0 || !comm) return IREE_B200_STATUS_OK;
  auto* ch = new iree_hal_b200_channel_t();
  ch->device = base_channel->device;
  ch->comm = comm;
  int count = 0, rank = 0;
  iree_b200_status_t st = nccl_check(g_nccl.ncclCommCount(comm, &count), "ncclCommCount");
  if (!st) st = nccl_check(g_nccl.ncclCommUserRank(comm, &rank), "ncclCommUserRank");
  if (st) {
    g_nccl.ncclCommDestroy(comm);
    delete ch;
    return st;
  }
  ch->count = count;
  ch->rank = rank;
  *out_channel = ch;
  return IREE_B200_STATUS_OK;
}

void iree_hal_b200_channel_retain(iree_hal_b200_channel_t* channel) {
  if (channel) channel->references.fetch_add(1);
}
void iree_hal_b200_channel_release(iree_hal_b200_channel_t* channel) {
  if (!channel || channel->references.fetch_sub(1) != 1) return;
  if (channel->comm) g_nccl.ncclCommDestroy(channel->comm);
  if (channel->barrier_word) iree_hal_b200_buffer_free(channel->device, channel->barrier_word);
  delete channel;
}
int32_t iree_hal_b200_channel_rank(const iree_hal_b200_channel_t* channel) { return channel ? channel->rank : 0; }
int32_t iree_hal_b200_channel_count(const iree_hal_b200_channel_t* channel) { return channel ? channel->count : 0; }

static iree_b200_status_t all_gather_on(iree_hal_b200_command_buffer_t* command_buffer, iree_hal_b200_channel_t* channel,
                                        int32_t element_type, const void* send_device_ptr, void* recv_device_ptr,
                                        size_t element_count, CUstream stream) {
  int nccl_type;  // ncclDataType_t values: int8 0, int32 2, float16 6, float32 7, bfloat16 9
  switch (element_type) {
    case IREE_HAL_B200_ELEMENT_TYPE_I8: nccl_type = 0; break;
    case IREE_HAL_B200_ELEMENT_TYPE_I32: nccl_type = 2; break;
    case IREE_HAL_B200_ELEMENT_TYPE_F16: nccl_type = 6; break;
    case IREE_HAL_B200_ELEMENT_TYPE_F32: nccl_type = 7; break;
    case IREE_HAL_B200_ELEMENT_TYPE_BF16: nccl_type = 9; break;
    default: return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "unsupported collective element type %d", element_type);
  }
  // One collective per flush, inside a group like iree_hal_cuda_nccl_submit_batch (nccl_channel.c:542-585).
  B200_RETURN_IF_ERROR(nccl_check(g_nccl.ncclGroupStart(), "ncclGroupStart"));
  iree_b200_status_t st = nccl_check(
      g_nccl.ncclAllGather(send_device_ptr, recv_device_ptr, element_count, nccl_type, channel->comm, stream),
      "ncclAllGather");
  iree_b200_status_t st2 = nccl_check(g_nccl.ncclGroupEnd(), "ncclGroupEnd");
  return st ? st : st2;
}

iree_b200_status_t iree_hal_b200_command_buffer_all_gather(iree_hal_b200_command_buffer_t* command_buffer,
                                                           iree_hal_b200_channel_t* channel, int32_t element_type,
                                                           const void* send_device_ptr, void* recv_device_ptr,
                                                           size_t element_count) {
  if (!command_buffer || !channel) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if (command_buffer->recording)
    return fail(IREE_B200_STATUS_UNIMPLEMENTED, "collectives cannot be recorded into a graph");
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(command_buffer->device->context), "cuCtxSetCurrent");
  return all_gather_on(command_buffer, channel, element_type, send_device_ptr, recv_device_ptr, element_count,
                       command_buffer->device->stream);
}

// iree_hal_command_buffer_collective for every kind the reference's NCCL channel submits
// (nccl_channel.c:327-500): one group per call, on the dispatch stream.
iree_b200_status_t iree_hal_b200_command_buffer_collective(iree_hal_b200_command_buffer_t* command_buffer,
                                                           iree_hal_b200_channel_t* channel, int32_t kind,
                                                           int32_t reduction, int32_t element_type, uint32_t param,
                                                           const void* send_device_ptr, void* recv_device_ptr,
                                                           size_t element_count) {
  if (!command_buffer || !channel) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if (command_buffer->recording)
    return fail(IREE_B200_STATUS_UNIMPLEMENTED, "collectives cannot be recorded into a graph");
  B200_RETURN_IF_ERROR(ensure_nccl());
  int type, elem_bytes;  // ncclDataType_t values: int8 0, int32 2, float16 6, float32 7, bfloat16 9
  switch (element_type) {
    case IREE_HAL_B200_ELEMENT_TYPE_I8: type = 0, elem_bytes = 1; break;
    case IREE_HAL_B200_ELEMENT_TYPE_I32: type = 2, elem_bytes = 4; break;
    case IREE_HAL_B200_ELEMENT_TYPE_F16: type = 6, elem_bytes = 2; break;
    case IREE_HAL_B200_ELEMENT_TYPE_F32: type = 7, elem_bytes = 4; break;
    case IREE_HAL_B200_ELEMENT_TYPE_BF16: type = 9, elem_bytes = 2; break;
    default: return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "unsupported collective element type %d", element_type);
  }
  const bool reduces = kind == IREE_HAL_B200_COLLECTIVE_ALL_REDUCE || kind == IREE_HAL_B200_COLLECTIVE_REDUCE ||
                       kind == IREE_HAL_B200_COLLECTIVE_REDUCE_SCATTER;
  int op = 0;  // ncclRedOp_t: sum 0, prod 1, max 2, min 3, avg 4
  if (reduces) {
    switch (reduction) {
      case IREE_HAL_B200_REDUCTION_SUM: op = 0; break;
      case IREE_HAL_B200_REDUCTION_PRODUCT: op = 1; break;
      case IREE_HAL_B200_REDUCTION_MINIMUM: op = 3; break;
      case IREE_HAL_B200_REDUCTION_MAXIMUM: op = 2; break;
      case IREE_HAL_B200_REDUCTION_AVERAGE: op = 4; break;
      default: return fail(IREE_B200_STATUS_UNIMPLEMENTED, "unhandled reduction type for collective op");
    }
  }
  const bool sends = kind != IREE_HAL_B200_COLLECTIVE_RECV, receives = kind != IREE_HAL_B200_COLLECTIVE_SEND;
  if ((sends && !send_device_ptr) || (receives && !recv_device_ptr))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "buffer pointer is NULL");
  iree_hal_b200_device_t* d = command_buffer->device;
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(d->context), "cuCtxSetCurrent");
  const int peer = static_cast<int>(param & 0xffff), peer2 = static_cast<int>(param >> 16);
  auto need = [&](bool have, const char* name) -> iree_b200_status_t {
    return have ? IREE_B200_STATUS_OK : fail(IREE_B200_STATUS_UNAVAILABLE, "this NCCL has no %s", name);
  };
  B200_RETURN_IF_ERROR(nccl_check(g_nccl.ncclGroupStart(), "ncclGroupStart"));
  iree_b200_status_t st = IREE_B200_STATUS_OK;
  switch (kind) {
    case IREE_HAL_B200_COLLECTIVE_ALL_GATHER:
      st = nccl_check(g_nccl.ncclAllGather(send_device_ptr, recv_device_ptr, element_count, type, channel->comm, d->stream),
                      "ncclAllGather");
      break;
    case IREE_HAL_B200_COLLECTIVE_ALL_REDUCE:
      st = need(g_nccl.ncclAllReduce, "ncclAllReduce");
      if (!st)
        st = nccl_check(g_nccl.ncclAllReduce(send_device_ptr, recv_device_ptr, element_count, type, op, channel->comm, d->stream),
                        "ncclAllReduce");
      break;
    case IREE_HAL_B200_COLLECTIVE_ALL_TO_ALL: {
      // element_count is the whole send buffer: count / ranks elements go to, and come from, every rank
      st = need(g_nccl.ncclSend && g_nccl.ncclRecv, "ncclSend / ncclRecv");
      const size_t per_rank = element_count / channel->count;
      for (int r = 0; r < channel->count && !st; ++r) {
        st = nccl_check(g_nccl.ncclSend(static_cast<const uint8_t*>(send_device_ptr) + r * per_rank * elem_bytes, per_rank, type,
                                        r, channel->comm, d->stream),
                        "ncclSend");
        if (!st)
          st = nccl_check(g_nccl.ncclRecv(static_cast<uint8_t*>(recv_device_ptr) + r * per_rank * elem_bytes, per_rank, type, r,
                                          channel->comm, d->stream),
                          "ncclRecv");
      }
      break;
    }
    case IREE_HAL_B200_COLLECTIVE_BROADCAST:
      st = need(g_nccl.ncclBroadcast, "ncclBroadcast");
      if (!st)
        st = nccl_check(g_nccl.ncclBroadcast(send_device_ptr, recv_device_ptr, element_count, type, peer, channel->comm, d->stream),
                        "ncclBroadcast");
      break;
    case IREE_HAL_B200_COLLECTIVE_REDUCE:
      st = need(g_nccl.ncclReduce, "ncclReduce");
      if (!st)
        st = nccl_check(g_nccl.ncclReduce(send_device_ptr, recv_device_ptr, element_count, type, op, peer, channel->comm, d->stream),
                        "ncclReduce");
      break;
    case IREE_HAL_B200_COLLECTIVE_REDUCE_SCATTER:
      // element_count is what every rank receives
      st = need(g_nccl.ncclReduceScatter, "ncclReduceScatter");
      if (!st)
        st = nccl_check(g_nccl.ncclReduceScatter(send_device_ptr, recv_device_ptr, element_count, type, op, channel->comm, d->stream),
                        "ncclReduceScatter");
      break;
    case IREE_HAL_B200_COLLECTIVE_SEND:
      st = need(g_nccl.ncclSend, "ncclSend");
      if (!st) st = nccl_check(g_nccl.ncclSend(send_device_ptr, element_count, type, peer, channel->comm, d->stream), "ncclSend");
      break;
    case IREE_HAL_B200_COLLECTIVE_RECV:
      st = need(g_nccl.ncclRecv, "ncclRecv");
      if (!st) st = nccl_check(g_nccl.ncclRecv(recv_device_ptr, element_count, type, peer, channel->comm, d->stream), "ncclRecv");
      break;
    case IREE_HAL_B200_COLLECTIVE_SEND_RECV:
      // param: low 16 bits the rank to send to, high 16 bits the rank to receive from
      st = need(g_nccl.ncclSend && g_nccl.ncclRecv, "ncclSend / ncclRecv");
      if (!st) st = nccl_check(g_nccl.ncclSend(send_device_ptr, element_count, type, peer, channel->comm, d->stream), "ncclSend");
      if (!st) st = nccl_check(g_nccl.ncclRecv(recv_device_ptr, element_count, type, peer2, channel->comm, d->stream), "ncclRecv");
      break;
    default:
      st = fail(IREE_B200_STATUS_INVALID_ARGUMENT, "unknown collective kind %d", kind);
  }
  const iree_b200_status_t end = nccl_check(g_nccl.ncclGroupEnd(), "ncclGroupEnd");
  if (st) return st;
  if (end) return end;
  command_buffer->barrier_pending = true;
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_command_buffer_all_gather_overlapped(iree_hal_b200_command_buffer_t* command_buffer,
                                                                      iree_hal_b200_channel_t* channel,
                                                                      int32_t element_type, const void* send_device_ptr,
                                                                      void* recv_device_ptr, size_t element_count) {
  if (!command_buffer || !channel) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if (command_buffer->recording)
    return fail(IREE_B200_STATUS_UNIMPLEMENTED, "collectives cannot be recorded into a graph");
  iree_hal_b200_device_t* d = command_buffer->device;
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(d->context), "cuCtxSetCurrent");
  if (!d->collective_stream) {
    CU_RETURN_IF_ERROR(g_cu.cuStreamCreate(&d->collective_stream, CU_STREAM_NON_BLOCKING), "cuStreamCreate");
    CU_RETURN_IF_ERROR(g_cu.cuEventCreate(&d->dispatch_done, CU_EVENT_DISABLE_TIMING), "cuEventCreate");
    CU_RETURN_IF_ERROR(g_cu.cuEventCreate(&d->collective_done, CU_EVENT_DISABLE_TIMING), "cuEventCreate");
  }
  // The collective starts once everything recorded so far has run; later dispatches do not wait for it.
  CU_RETURN_IF_ERROR(g_cu.cuEventRecord(d->dispatch_done, d->stream), "cuEventRecord");
  CU_RETURN_IF_ERROR(g_cu.cuStreamWaitEvent(d->collective_stream, d->dispatch_done, 0), "cuStreamWaitEvent");
  return all_gather_on(command_buffer, channel, element_type, send_device_ptr, recv_device_ptr, element_count,
                       d->collective_stream);
}

// ---- peer memory: buffers of other ranks (processes) on the same node -----------------------------------
iree_b200_status_t iree_hal_b200_buffer_export(iree_hal_b200_device_t* device, void* device_ptr, void* out_handle) {
  if (!device || !device_ptr || !out_handle) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if (!g_cu.cuIpcGetMemHandle) return fail(IREE_B200_STATUS_UNAVAILABLE, "this CUDA driver cannot share device memory");
  static_assert(sizeof(CUipcMemHandle) == IREE_HAL_B200_PEER_HANDLE_SIZE, "handle size");
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  CUipcMemHandle h;
  CU_RETURN_IF_ERROR(g_cu.cuIpcGetMemHandle(&h, reinterpret_cast<CUdeviceptr>(device_ptr)), "cuIpcGetMemHandle");
  memcpy(out_handle, &h, sizeof h);
  return IREE_B200_STATUS_OK;
}
iree_b200_status_t iree_hal_b200_buffer_import(iree_hal_b200_device_t* device, const void* handle, void** out_device_ptr) {
  if (!device || !handle || !out_device_ptr) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  *out_device_ptr = nullptr;
  if (!g_cu.cuIpcOpenMemHandle) return fail(IREE_B200_STATUS_UNAVAILABLE, "this CUDA driver cannot share device memory");
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  CUipcMemHandle h;
  memcpy(&h, handle, sizeof h);
  CUdeviceptr p = 0;
  CU_RETURN_IF_ERROR(g_cu.cuIpcOpenMemHandle(&p, h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS), "cuIpcOpenMemHandle");
  *out_device_ptr = reinterpret_cast<void*>(p);
  return IREE_B200_STATUS_OK;
}
iree_b200_status_t iree_hal_b200_buffer_unimport(iree_hal_b200_device_t* device, void* device_ptr) {
  if (!device || !device_ptr) return IREE_B200_STATUS_OK;
  if (!g_cu.cuIpcCloseMemHandle) return fail(IREE_B200_STATUS_UNAVAILABLE, "this CUDA driver cannot share device memory");
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(device->context), "cuCtxSetCurrent");
  CU_RETURN_IF_ERROR(g_cu.cuIpcCloseMemHandle(reinterpret_cast<CUdeviceptr>(device_ptr)), "cuIpcCloseMemHandle");
  return IREE_B200_STATUS_OK;
}

// All-gather by peer copies: this rank's block goes into slot `rank` of every rank's receive
// buffer through the copy engines (no SM is used, so it runs beside a persistent dispatch that
// fills them all), on the collective stream, after everything recorded on the dispatch stream so
// far. A channel barrier (a one-word all-reduce) follows on the same stream: when the collective
// stream of a rank has passed it, every rank has finished the copies it enqueued before its own
// barrier, i.e. that rank's receive buffer is complete.
iree_b200_status_t iree_hal_b200_command_buffer_all_gather_peer_copies(iree_hal_b200_command_buffer_t* command_buffer,
                                                                        iree_hal_b200_channel_t* channel,
                                                                        const void* send_device_ptr, size_t byte_count,
                                                                        void* const* recv_device_ptrs) {
  if (!command_buffer || !channel || !recv_device_ptrs || (byte_count && !send_device_ptr))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if (command_buffer->recording)
    return fail(IREE_B200_STATUS_UNIMPLEMENTED, "collectives cannot be recorded into a graph");
  if (!g_cu.cuMemcpyDtoDAsync || !g_nccl.ncclAllReduce)
    return fail(IREE_B200_STATUS_UNAVAILABLE, "peer copies need cuMemcpyDtoDAsync and ncclAllReduce");
  iree_hal_b200_device_t* d = command_buffer->device;
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(d->context), "cuCtxSetCurrent");
  if (!d->collective_stream) {
    CU_RETURN_IF_ERROR(g_cu.cuStreamCreate(&d->collective_stream, CU_STREAM_NON_BLOCKING), "cuStreamCreate");
    CU_RETURN_IF_ERROR(g_cu.cuEventCreate(&d->dispatch_done, CU_EVENT_DISABLE_TIMING), "cuEventCreate");
    CU_RETURN_IF_ERROR(g_cu.cuEventCreate(&d->collective_done, CU_EVENT_DISABLE_TIMING), "cuEventCreate");
  }
  if (!channel->barrier_word) {
    B200_RETURN_IF_ERROR(iree_hal_b200_buffer_allocate(d, 256, &channel->barrier_word));
    B200_RETURN_IF_ERROR(iree_hal_b200_fill_buffer(d, channel->barrier_word, 256, 0));
    B200_RETURN_IF_ERROR(iree_hal_b200_device_synchronize(d));
  }
  constexpr int kStreams = iree_hal_b200_device_t::kCopyStreams;
  if (!d->copies_go) {
    CU_RETURN_IF_ERROR(g_cu.cuEventCreate(&d->copies_go, CU_EVENT_DISABLE_TIMING), "cuEventCreate");
    for (int i = 0; i < kStreams; ++i) {
      CU_RETURN_IF_ERROR(g_cu.cuStreamCreate(&d->copy_streams[i], CU_STREAM_NON_BLOCKING), "cuStreamCreate");
      CU_RETURN_IF_ERROR(g_cu.cuEventCreate(&d->copy_done[i], CU_EVENT_DISABLE_TIMING), "cuEventCreate");
    }
  }
  CU_RETURN_IF_ERROR(g_cu.cuEventRecord(d->dispatch_done, d->stream), "cuEventRecord");
  CU_RETURN_IF_ERROR(g_cu.cuStreamWaitEvent(d->collective_stream, d->dispatch_done, 0), "cuStreamWaitEvent");
  // Barrier ahead of the copies: every rank's collective stream has waited for that rank's dispatch
  // stream, so once all ranks have passed it, whatever a peer recorded earlier that still reads its
  // receive buffer (from the buffer's previous use) has finished before anybody writes into it.
  B200_RETURN_IF_ERROR(nccl_check(g_nccl.ncclAllReduce(channel->barrier_word, channel->barrier_word, 1, 2, 0, channel->comm,
                                                       d->collective_stream),
                                  "ncclAllReduce"));
  CU_RETURN_IF_ERROR(g_cu.cuEventRecord(d->copies_go, d->collective_stream), "cuEventRecord");
  // One copy engine moves a fraction of what the links carry, so the copies to different peers
  // run side by side on streams of their own, and a block of 64 MiB or more goes as two pieces.
  // (More pieces cost more driver calls per step than they save: with 8 pieces of 4 MiB the
  // 133 us step of the 2-GPU f16 4096^3 workload became host-bound at 170 us.)
  const int32_t peers = channel->count > 1 ? channel->count - 1 : 1;
  size_t pieces = (byte_count >= (64u << 20) && 2 * peers <= kStreams) ? 2 : 1;
  const size_t piece_bytes = ((byte_count + pieces - 1) / pieces + 255) & ~static_cast<size_t>(255);
  int next_stream = 0, used = 0;
  for (int32_t i = 0; i < channel->count; ++i) {
    // start with the neighbour so that the ranks do not all write to the same peer at once
    const int32_t p = (channel->rank + 1 + i) % channel->count;
    if (!recv_device_ptrs[p]) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "receive buffer of rank %d is NULL", p);
    uint8_t* dst = static_cast<uint8_t*>(recv_device_ptrs[p]) + static_cast<size_t>(channel->rank) * byte_count;
    for (size_t off = 0; off < byte_count; off += piece_bytes) {
      const size_t n = byte_count - off < piece_bytes ? byte_count - off : piece_bytes;
      const int k = next_stream;
      next_stream = (next_stream + 1) % kStreams;
      if (used < kStreams) {
        CU_RETURN_IF_ERROR(g_cu.cuStreamWaitEvent(d->copy_streams[k], d->copies_go, 0), "cuStreamWaitEvent");
        ++used;
      }
      CU_RETURN_IF_ERROR(g_cu.cuMemcpyDtoDAsync(reinterpret_cast<CUdeviceptr>(dst + off),
                                                reinterpret_cast<CUdeviceptr>(static_cast<const uint8_t*>(send_device_ptr) + off),
                                                n, d->copy_streams[k]),
                         "cuMemcpyDtoDAsync");
    }
  }
  for (int k = 0; k < used; ++k) {
    CU_RETURN_IF_ERROR(g_cu.cuEventRecord(d->copy_done[k], d->copy_streams[k]), "cuEventRecord");
    CU_RETURN_IF_ERROR(g_cu.cuStreamWaitEvent(d->collective_stream, d->copy_done[k], 0), "cuStreamWaitEvent");
  }
  // ncclInt32 = 2, ncclSum = 0
  B200_RETURN_IF_ERROR(nccl_check(g_nccl.ncclAllReduce(channel->barrier_word, channel->barrier_word, 1, 2, 0, channel->comm,
                                                       d->collective_stream),
                                  "ncclAllReduce"));
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_hal_b200_command_buffer_join_collectives(iree_hal_b200_command_buffer_t* command_buffer) {
  if (!command_buffer) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "command buffer is NULL");
  iree_hal_b200_device_t* d = command_buffer->device;
  if (!d->collective_stream) return IREE_B200_STATUS_OK;
  CU_RETURN_IF_ERROR(g_cu.cuCtxSetCurrent(d->context), "cuCtxSetCurrent");
  CU_RETURN_IF_ERROR(g_cu.cuEventRecord(d->collective_done, d->collective_stream), "cuEventRecord");
  CU_RETURN_IF_ERROR(g_cu.cuStreamWaitEvent(d->stream, d->collective_done, 0), "cuStreamWaitEvent");
  return IREE_B200_STATUS_OK;
}

}  // extern "C"

// ==========================================================================================
// Operator level
// ==========================================================================================
namespace {

constexpr uint32_t kGemmThreads = 256;
constexpr uint32_t kGemmSmemBytes = 1024 + 4 * (128 * 128 + 256 * 128) + 2 * 128 * 128 /*epilogue staging*/ + 256;
constexpr uint32_t kMmt4dSmemBytes = 1024 + 4 * (128 * 128 + 256 * 128) + 256;
// weight ring (5 / 4 stages of 16 rows x 2048 B + 128 B), scale ring (4 KiB per stage), 3 slots of 16 per-warp
// chunk sums, the per-warp offsets, barriers (decode_smem_bytes in w4a16_decode.cuh)
constexpr uint32_t kDecodeSmemM8 = 5 * (16 * 2048 + 128) + 5 * 4096 + 3 * 16 * 32 * 16 * 1 + 16 * 1 * 2 * 32 * 8 + 256;
constexpr uint32_t kDecodeSmemM16 = 4 * (16 * 2048 + 128) + 4 * 4096 + 3 * 16 * 32 * 16 * 2 + 16 * 2 * 2 * 32 * 8 + 256;
// K per CTA of the decode kernels, and the scratch they need beyond one slice: a counter per 16-row
// tile (padded to 256 bytes), then one 1 KiB partial tile per tile and slice (DecodeScratchLayout).
constexpr int kDecodeSliceK = 4096, kDecodeMaxSlices = 4;
size_t decode_counter_bytes(int64_t N) { return (static_cast<size_t>(N / 16) * 4 + 255) & ~static_cast<size_t>(255); }
size_t decode_scratch_bytes(int64_t N, int slices) {
  return decode_counter_bytes(N) + static_cast<size_t>(N / 16) * slices * 1024;
}
constexpr uint32_t kW4SmemBytes = 1024 + 224 * 1024 + 256;  // operand stages + raw stages of either variant
// b200_w4a16_gemm_wt: 4 activation stages of 32 KiB, 6 raw stages of 8 KiB, 2 staging tiles of 16 KiB, barriers
constexpr uint32_t kW4WtSmemBytes = 1024 + 4 * 32768 + 6 * 8192 + 2 * 16384 + 512;
constexpr int kWtMaxDestinations = 8;
// staging region of the pack / unpack kernels: 64 rows of at most 512 bytes, 16 bytes of padding per row
constexpr uint32_t kTilingStageBytes = 64 * (2 * 256 + 16);

struct EntryDecl {
  const char* name;
  uint32_t block[3];
  uint32_t smem;
};
// Every export of the contraction cubin with the launch configuration the plugin records on
// its hal.executable.export (workgroup_size, workgroup_local_memory).
const EntryDecl kEntries[] = {
    {"b200_matmul_f16_f16", {kGemmThreads, 1, 1}, kGemmSmemBytes},
    {"b200_matmul_f16_f32", {kGemmThreads, 1, 1}, kGemmSmemBytes},
    {"b200_matmul_bf16_bf16", {kGemmThreads, 1, 1}, kGemmSmemBytes},
    {"b200_matmul_bf16_f32", {kGemmThreads, 1, 1}, kGemmSmemBytes},
    {"b200_matmul_i8_i32", {kGemmThreads, 1, 1}, kGemmSmemBytes},
    {"b200_matmul_i8_requant_f16", {kGemmThreads, 1, 1}, kGemmSmemBytes},
    {"b200_matmul_pair_f16_f16", {kGemmThreads, 1, 1}, kGemmSmemBytes},
    {"b200_matmul_pair_f16_f32", {kGemmThreads, 1, 1}, kGemmSmemBytes},
    {"b200_matmul_pair_bf16_bf16", {kGemmThreads, 1, 1}, kGemmSmemBytes},
    {"b200_matmul_pair_bf16_f32", {kGemmThreads, 1, 1}, kGemmSmemBytes},
    {"b200_matmul_pair_i8_i32", {kGemmThreads, 1, 1}, kGemmSmemBytes},
    {"b200_matmul_pair_i8_requant_f16", {kGemmThreads, 1, 1}, kGemmSmemBytes},
    {"b200_encode_tensormaps", {32, 1, 1}, 0},
    {"b200_encode_tensormap", {32, 1, 1}, 0},
    {"b200_selftest_wait_timeout", {32, 1, 1}, 0},
    {"b200_matmul_generic_f16_f16", {16, 16, 1}, 0},
    {"b200_matmul_generic_f16_f32", {16, 16, 1}, 0},
    {"b200_matmul_generic_bf16_bf16", {16, 16, 1}, 0},
    {"b200_matmul_generic_bf16_f32", {16, 16, 1}, 0},
    {"b200_matmul_generic_i8_i32", {16, 16, 1}, 0},
    {"b200_matmul_generic_i8_requant_f16", {16, 16, 1}, 0},
    {"b200_w4a16_decode_m8", {512, 1, 1}, kDecodeSmemM8},
    {"b200_w4a16_decode_m16", {512, 1, 1}, kDecodeSmemM16},
    {"b200_w4a16_decode_tc", {b200::kTcThreads, 1, 1}, b200::kTcSmemBytes},
    {"b200_w4a16_gemm", {512, 1, 1}, kW4SmemBytes},
    {"b200_w4a16_gemm_wt", {512, 1, 1}, kW4WtSmemBytes},
    {"b200_wait_arrivals", {32, 1, 1}, 0},
    {"b200_w4a16_generic", {256, 1, 1}, 0},
    {"b200_mmt4d_s8s8s32", {512, 1, 1}, kMmt4dSmemBytes},
    {"b200_mmt4d_f16f16f32", {512, 1, 1}, kMmt4dSmemBytes},
    {"b200_mmt4d_f16f16f16", {512, 1, 1}, kMmt4dSmemBytes},
    {"b200_mmt4d_bf16bf16f32", {512, 1, 1}, kMmt4dSmemBytes},
    {"b200_mmt4d_bf16bf16bf16", {512, 1, 1}, kMmt4dSmemBytes},
    {"b200_mmt4d_generic", {256, 1, 1}, 0},
    {"b200_tiling_tma", {32, 1, 1}, 1024 + 8 * 16384 + 128},
    {"b200_pack_i8_rhs_16x2", {288, 1, 1}, 1024 + 4 * 16384 + 2 * 8 * (64 * 32 + 32) + 128},
    {"b200_pack_lhs_16x2b", {288, 1, 1}, 1024 + 4 * 16384 + 2 * 8 * (64 * 32 + 32) + 128},
    {"b200_pack_b8", {256, 1, 1}, kTilingStageBytes},
    {"b200_pack_b16", {256, 1, 1}, kTilingStageBytes},
    {"b200_pack_b32", {256, 1, 1}, kTilingStageBytes},
    {"b200_unpack_b8", {256, 1, 1}, kTilingStageBytes},
    {"b200_unpack_b16", {256, 1, 1}, kTilingStageBytes},
    {"b200_unpack_b32", {256, 1, 1}, kTilingStageBytes},
};
constexpr int kEntryCount = sizeof kEntries / sizeof kEntries[0];

}  // namespace

struct iree_b200_context_t {
  iree_hal_b200_device_t* device = nullptr;
  iree_hal_b200_executable_t* executable = nullptr;
  iree_hal_b200_command_buffer_t* command_buffer = nullptr;
  void* templates = nullptr;  // device copy of two template tensor maps per element size: [f16 A, f16 B, bf16.., i8..]
  // pack / unpack by TMA: three rank-4 template maps (1-, 2-, 4-byte elements) in the first 4 KiB, then 256 bytes
  // per CTA in which the kernel builds its own two maps
  void* tiling_scratch = nullptr;
  // Grow-only device staging area for the host-buffer entry points, so that repeated calls do
  // not pay for cuMemAlloc / cuMemFree.
  void* arena = nullptr;
  size_t arena_size = 0;
  bool dispatch_overlap = false;
  // SMs the operator entry points leave free (for collectives that run beside the dispatches)
  int reserved_sms = 0;
};

namespace {
// SMs the persistent kernels of this context may fill: all of them, less the reserved ones, even.
int usable_sms(const iree_b200_context_t* ctx) {
  int sms = ctx->device->sm_count > 0 ? ctx->device->sm_count : 148;
  sms -= ctx->reserved_sms;
  if (sms < 2) sms = 2;
  return sms & ~1;
}
}  // namespace

namespace {

int elem_bytes_of(int kind) { return kind == IREE_B200_KIND_I8 ? 1 : 2; }

const char* pair_export_name(int kind, int epilogue) {
  if (kind == IREE_B200_KIND_F16 && epilogue == IREE_B200_EPILOGUE_CAST) return "b200_matmul_pair_f16_f16";
  if (kind == IREE_B200_KIND_F16 && epilogue == IREE_B200_EPILOGUE_ACCUMULATOR) return "b200_matmul_pair_f16_f32";
  if (kind == IREE_B200_KIND_BF16 && epilogue == IREE_B200_EPILOGUE_CAST) return "b200_matmul_pair_bf16_bf16";
  if (kind == IREE_B200_KIND_BF16 && epilogue == IREE_B200_EPILOGUE_ACCUMULATOR) return "b200_matmul_pair_bf16_f32";
  if (kind == IREE_B200_KIND_I8 && epilogue == IREE_B200_EPILOGUE_ACCUMULATOR) return "b200_matmul_pair_i8_i32";
  if (kind == IREE_B200_KIND_I8 && epilogue == IREE_B200_EPILOGUE_REQUANT_F16) return "b200_matmul_pair_i8_requant_f16";
  return nullptr;
}

// CTA pairs (256 x tile_n tiles) pay off when there are enough 256-row tiles to fill the SM pairs.
bool use_pairs(const iree_b200_context_t* ctx, const iree_b200_matmul_params_t* p);

const char* export_name(int kind, int epilogue, bool generic) {
  if (kind == IREE_B200_KIND_F16 && epilogue == IREE_B200_EPILOGUE_CAST)
    return generic ? "b200_matmul_generic_f16_f16" : "b200_matmul_f16_f16";
  if (kind == IREE_B200_KIND_F16 && epilogue == IREE_B200_EPILOGUE_ACCUMULATOR)
    return generic ? "b200_matmul_generic_f16_f32" : "b200_matmul_f16_f32";
  if (kind == IREE_B200_KIND_BF16 && epilogue == IREE_B200_EPILOGUE_CAST)
    return generic ? "b200_matmul_generic_bf16_bf16" : "b200_matmul_bf16_bf16";
  if (kind == IREE_B200_KIND_BF16 && epilogue == IREE_B200_EPILOGUE_ACCUMULATOR)
    return generic ? "b200_matmul_generic_bf16_f32" : "b200_matmul_bf16_f32";
  if (kind == IREE_B200_KIND_I8 && epilogue == IREE_B200_EPILOGUE_ACCUMULATOR)
    return generic ? "b200_matmul_generic_i8_i32" : "b200_matmul_i8_i32";
  if (kind == IREE_B200_KIND_I8 && epilogue == IREE_B200_EPILOGUE_REQUANT_F16)
    return generic ? "b200_matmul_generic_i8_requant_f16" : "b200_matmul_i8_requant_f16";
  return nullptr;
}

iree_b200_status_t validate(const iree_b200_matmul_params_t* p) {
  if (!p) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "params is NULL");
  if (p->M < 0 || p->N < 0 || p->K < 0 || p->batch < 0)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "negative dimension");
  if (p->rhs_layout != IREE_B200_RHS_KN && p->rhs_layout != IREE_B200_RHS_NK)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "unknown rhs layout %d", p->rhs_layout);
  if (!export_name(p->kind, p->epilogue, false))
    return fail(IREE_B200_STATUS_UNIMPLEMENTED, "no kernel for kind %d with epilogue %d", p->kind, p->epilogue);
  return IREE_B200_STATUS_OK;
}

// The TMA path needs 16-byte aligned bases and row pitches.
bool tma_eligible(const iree_b200_matmul_params_t* p, const void* lhs, const void* rhs) {
  const int es = elem_bytes_of(p->kind);
  if (p->flags & IREE_B200_FLAG_FORCE_GENERIC) return false;
  if ((reinterpret_cast<uintptr_t>(lhs) % 16) || (reinterpret_cast<uintptr_t>(rhs) % 16)) return false;
  if ((static_cast<int64_t>(p->K) * es) % 16) return false;
  if (p->rhs_layout == IREE_B200_RHS_KN && (static_cast<int64_t>(p->N) * es) % 16) return false;
  return true;
}

// Tile width: the widest tile that still gives every SM work, weighing wave quantisation
// against the lower efficiency of narrow tiles.
bool use_pairs(const iree_b200_context_t* ctx, const iree_b200_matmul_params_t* p) {
  if (p->flags & IREE_B200_FLAG_SINGLE_CTA) return false;
  if (p->flags & IREE_B200_FLAG_PAIR_CTAS) return true;
  const int sms = usable_sms(ctx);
  const int64_t tiles = static_cast<int64_t>((p->M + 255) / 256) * ((p->N + 255) / 256) * p->batch;
  return p->M >= 256 && tiles >= sms / 2 && p->K >= 512;
}

int choose_tile_n(const iree_b200_context_t* ctx, const iree_b200_matmul_params_t* p) {
  const int es = elem_bytes_of(p->kind);
  const bool pairs = use_pairs(ctx, p);
  // In pair mode each CTA holds half a tile: the half must be whole 128-byte column chunks.
  const int chunk = (p->rhs_layout == IREE_B200_RHS_KN) ? (pairs ? 2 : 1) * 128 / es : (pairs ? 64 : 32);
  const int sms = usable_sms(ctx) / (pairs ? 2 : 1);
  const int64_t tiles_m = (p->M + (pairs ? 255 : 127)) / (pairs ? 256 : 128);
  int best = 0;
  double best_score = -1;
  for (int bn = 256; bn >= 32; bn -= 32) {
    if (bn % chunk) continue;
    if (p->tile_n && bn != p->tile_n) continue;
    // Few rows: the product only streams the right-hand side; tiles of at most 128 columns select
    // the kernels' deep-ring variant (32-row A box, nine stages in flight).
    if (!p->tile_n && p->M <= 32 && bn > 128 && chunk <= 128) continue;
    const int64_t tiles = tiles_m * ((p->N + bn - 1) / bn) * p->batch;
    const int64_t waves = (tiles + sms - 1) / sms;
    // Time model fitted on 4096^3 f16 (wave time 25.0 / 22.3 / 20.3 us at tile widths 256 / 192 / 128):
    // a wave costs (400 + bn) units, i.e. narrow tiles are far from proportionally cheaper because the
    // A tile is re-fetched per tile and the operand traffic per flop grows.
    const double cost = static_cast<double>(waves) * (400.0 + bn);
    const double score = 1.0 / cost;
    if (score > best_score * 1.0001) {
      best_score = score;
      best = bn;
    }
  }
  return best;
}

// Few-rows products (the kernels' deep-ring variant) leave most SMs idle when N / tile_n is small
// against the SM count; every tile's K range can be cut into `splits` work items that are dealt to
// the CTAs.
constexpr int kFewRows = 32, kMaxSplits = 16;
constexpr size_t kSplitCountersOffset = 512;
size_t split_partials_offset(int64_t tiles) { return kSplitCountersOffset + ((static_cast<size_t>(tiles) * 4 + 127) / 128) * 128; }
int choose_splits(const iree_b200_context_t* ctx, const iree_b200_matmul_params_t* p, int bn) {
  if (!(p->flags & IREE_B200_FLAG_SPLIT_K) || p->M > kFewRows || bn > 128 || use_pairs(ctx, p)) return 1;
  const int es = elem_bytes_of(p->kind);
  const int num_kb = (p->K + 128 / es - 1) / (128 / es);
  const int64_t tiles = static_cast<int64_t>((p->N + bn - 1) / bn) * p->batch;
  // Measured on C3 (M = 1 and 16, N = 11008, K = 4096, three splits): 28 us against 17.6 us unsplit. The
  // meeting of the partial accumulators (a fence and a counter per item, under a saturated memory
  // system) costs more than the idle SMs do, so a split is only made on request (bits 8..11).
  (void)tiles;
  const int forced = (p->flags >> 8) & 0xf;
  if (!forced) return 1;
  return forced <= num_kb ? forced : num_kb;
}

}  // namespace

extern "C" {

size_t iree_b200_matmul_workspace_bytes(iree_b200_context_t* context, const iree_b200_matmul_params_t* params) {
  if (!context || !params || validate(params) != IREE_B200_STATUS_OK || !params->M || !params->N || !params->K || !params->batch)
    return IREE_B200_WORKSPACE_BYTES;
  const int bn = choose_tile_n(context, params);
  const int splits = bn ? choose_splits(context, params, bn) : 1;
  if (splits <= 1) return IREE_B200_WORKSPACE_BYTES;
  const int64_t tiles = static_cast<int64_t>((params->N + bn - 1) / bn) * params->batch;
  return split_partials_offset(tiles) + static_cast<size_t>(tiles) * splits * kFewRows * bn * 4;
}

iree_b200_status_t iree_b200_contraction_executable_def(const char* cubin_path, void* out_data, size_t out_capacity,
                                                        size_t* out_size) {
  if (!cubin_path || !out_size) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  FILE* f = fopen(cubin_path, "rb");
  if (!f) return fail(IREE_B200_STATUS_NOT_FOUND, "cannot open cubin '%s'", cubin_path);
  std::vector<uint8_t> image;
  uint8_t chunk[65536];
  size_t n;
  while ((n = fread(chunk, 1, sizeof chunk, f)) > 0) image.insert(image.end(), chunk, chunk + n);
  fclose(f);
  // Wrap the cubin the way the compiler's CUDA target does for an external object.
  const char* names[kEntryCount];
  uint32_t blocks[3 * kEntryCount], smem[kEntryCount];
  for (int i = 0; i < kEntryCount; ++i) {
    names[i] = kEntries[i].name;
    memcpy(&blocks[3 * i], kEntries[i].block, 12);
    smem[i] = kEntries[i].smem;
  }
  return iree_b200_executable_def_build(kEntryCount, names, blocks, smem, image.data(), image.size(), out_data,
                                        out_capacity, out_size);
}

iree_b200_status_t iree_b200_context_create(int32_t device_ordinal, const char* cubin_path,
                                            iree_b200_context_t** out_context) {
  if (!out_context || !cubin_path) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  *out_context = nullptr;
  size_t fb_size = 0;
  B200_RETURN_IF_ERROR(iree_b200_contraction_executable_def(cubin_path, nullptr, 0, &fb_size));
  std::vector<uint8_t> fb(fb_size);
  B200_RETURN_IF_ERROR(iree_b200_contraction_executable_def(cubin_path, fb.data(), fb.size(), &fb_size));
  auto* ctx = new iree_b200_context_t();
  iree_b200_status_t st = iree_hal_b200_device_create(device_ordinal, &ctx->device);
  if (!st) st = iree_hal_b200_executable_create(ctx->device, "PTXE", fb.data(), fb.size(), &ctx->executable);
  if (!st) st = iree_hal_b200_command_buffer_create(ctx->device, &ctx->command_buffer);
  if (st) {
    iree_b200_context_release(ctx);
    return st;
  }
  *out_context = ctx;
  return IREE_B200_STATUS_OK;
}

void iree_b200_context_release(iree_b200_context_t* context) {
  if (!context) return;
  if (context->device) iree_hal_b200_device_synchronize(context->device);
  if (context->templates) iree_hal_b200_buffer_free(context->device, context->templates);
  if (context->tiling_scratch) iree_hal_b200_buffer_free(context->device, context->tiling_scratch);
  if (context->arena) iree_hal_b200_buffer_free(context->device, context->arena);
  iree_hal_b200_command_buffer_release(context->command_buffer);
  iree_hal_b200_executable_release(context->executable);
  iree_hal_b200_device_release(context->device);
  delete context;
}
iree_b200_status_t iree_b200_context_set_dispatch_overlap(iree_b200_context_t* context, int32_t enable) {
  if (!context) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "context is NULL");
  // probes the driver; the command buffer's own switch is only raised around eligible dispatches
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_set_dispatch_overlap(context->command_buffer, enable));
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_set_dispatch_overlap(context->command_buffer, 0));
  context->dispatch_overlap = enable != 0;
  return IREE_B200_STATUS_OK;
}
iree_b200_status_t iree_b200_context_set_reserved_sms(iree_b200_context_t* context, int32_t count) {
  if (!context) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "context is NULL");
  const int sms = context->device->sm_count > 0 ? context->device->sm_count : 148;
  if (count < 0 || count > sms - 2) return fail(IREE_B200_STATUS_OUT_OF_RANGE, "cannot reserve %d of %d SMs", count, sms);
  context->reserved_sms = count;
  return IREE_B200_STATUS_OK;
}
iree_hal_b200_device_t* iree_b200_context_device(iree_b200_context_t* c) { return c ? c->device : nullptr; }
iree_hal_b200_executable_t* iree_b200_context_executable(iree_b200_context_t* c) { return c ? c->executable : nullptr; }
iree_hal_b200_command_buffer_t* iree_b200_context_command_buffer(iree_b200_context_t* c) {
  return c ? c->command_buffer : nullptr;
}

// Rank-3 row-major tensor [dim2, dim1, dim0]; the box is box0 x box1 x 1 elements.
static iree_b200_status_t encode_map(CUtensorMapDataType dt, int elem_bytes, CUtensorMapSwizzle swizzle,
                                     uint32_t swizzle_bytes, const void* device_ptr, uint32_t dim0, uint32_t dim1,
                                     uint32_t dim2, uint32_t box0, uint32_t box1, void* out_map, uint32_t box2 = 1) {
  B200_RETURN_IF_ERROR(ensure_cuda());
  if (box0 * elem_bytes != swizzle_bytes || box1 == 0 || box1 > 256)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "box must be %u bytes wide and 1..256 rows", swizzle_bytes);
  if ((reinterpret_cast<uintptr_t>(device_ptr) % 16) || (static_cast<uint64_t>(dim0) * elem_bytes) % 16)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "tensor base and row pitch must be multiples of 16 bytes");
  CUtensorMap map;
  const cuuint64_t dims[3] = {dim0, dim1, dim2};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(dim0) * elem_bytes,
                                 static_cast<cuuint64_t>(dim0) * dim1 * elem_bytes};
  const cuuint32_t box[3] = {box0, box1, box2};
  const cuuint32_t estrides[3] = {1, 1, 1};
  CU_RETURN_IF_ERROR(g_cu.cuTensorMapEncodeTiled(&map, dt, 3, const_cast<void*>(device_ptr), dims, strides, box,
                                                 estrides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
                     "cuTensorMapEncodeTiled");
  memcpy(out_map, &map, 128);
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_b200_encode_tensor_map(iree_b200_context_t* context, int32_t elem_bytes, int32_t is_bf16,
                                               const void* device_ptr, uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                               uint32_t box0, uint32_t box1, void* out_map) {
  if (!context || !out_map) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if (elem_bytes != 1 && elem_bytes != 2) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "element size must be 1 or 2");
  const CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : is_bf16       ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return encode_map(dt, elem_bytes, CU_TENSOR_MAP_SWIZZLE_128B, 128, device_ptr, dim0, dim1, dim2, box0, box1, out_map);
}

iree_b200_status_t iree_b200_tensormap_templates(iree_b200_context_t* context, void* out_templates) {
  if (!context || !out_templates) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  B200_RETURN_IF_ERROR(ensure_cuda());
  // Any valid, 16-byte aligned device address will do for the tensor the templates describe: every
  // field that depends on it is replaced on the device.
  void* dummy = nullptr;
  B200_RETURN_IF_ERROR(iree_hal_b200_buffer_allocate(context->device, 4096, &dummy));
  struct FreeDummy {
    iree_hal_b200_device_t* device;
    void* p;
    ~FreeDummy() { iree_hal_b200_buffer_free(device, p); }
  } free_dummy{context->device, dummy};
  uint8_t* out = static_cast<uint8_t*>(out_templates);
  struct Kind {
    CUtensorMapDataType type;
    int elem_bytes;
    CUtensorMapSwizzle swizzle;
    uint32_t inner_bytes;
    int rank;
  };
  const Kind kinds[IREE_B200_TEMPLATE_COUNT] = {
      {CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, CU_TENSOR_MAP_SWIZZLE_128B, 128, 3},
      {CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, CU_TENSOR_MAP_SWIZZLE_128B, 128, 3},
      {CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, CU_TENSOR_MAP_SWIZZLE_128B, 128, 3},
      {CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, CU_TENSOR_MAP_SWIZZLE_64B, 64, 3},
      {CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, CU_TENSOR_MAP_SWIZZLE_NONE, 256, 2},
      {CU_TENSOR_MAP_DATA_TYPE_UINT64, 8, CU_TENSOR_MAP_SWIZZLE_NONE, 2048, 2},
  };
  for (int i = 0; i < IREE_B200_TEMPLATE_COUNT; ++i) {
    const Kind& k = kinds[i];
    CUtensorMap map;
    const cuuint32_t box0 = k.inner_bytes / k.elem_bytes;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(box0) * 4, 256, 1};
    const cuuint64_t strides[2] = {dims[0] * k.elem_bytes, dims[0] * k.elem_bytes * 256};
    const cuuint32_t box[3] = {box0, 8, 1};
    const cuuint32_t estrides[3] = {1, 1, 1};
    const CUtensorMapL2promotion promo = i == IREE_B200_TEMPLATE_F16_PLAIN_RANK2 ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                                                                                 : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
    CU_RETURN_IF_ERROR(g_cu.cuTensorMapEncodeTiled(&map, k.type, k.rank, dummy, dims, strides, box, estrides,
                                                   CU_TENSOR_MAP_INTERLEAVE_NONE, k.swizzle, promo,
                                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
                       "cuTensorMapEncodeTiled(template)");
    memcpy(out + 128 * i, &map, 128);
  }
  return IREE_B200_STATUS_OK;
}

// The 512-byte workspace header of a TMA-eligible product, encoded on the host: tensor maps of
// both operands (for the tile width `bn`), status words zero.
static iree_b200_status_t encode_workspace_header(iree_b200_context_t* context, const iree_b200_matmul_params_t* params,
                                                  const void* lhs, const void* rhs, int bn, uint8_t* host) {
  memset(host, 0, IREE_B200_WORKSPACE_BYTES);
  const int es = elem_bytes_of(params->kind);
  const uint32_t bk = 128 / es;
  const uint32_t M = params->M, N = params->N, K = params->K, B = params->batch;
  const int bf = params->kind == IREE_B200_KIND_BF16;
  // A box: 128 rows, or 32 in the few-rows variant (the same rule as in the kernels)
  const uint32_t a_rows = (params->M <= 32 && bn <= 128) ? 32 : 128;
  B200_RETURN_IF_ERROR(iree_b200_encode_tensor_map(context, es, bf, lhs, K, M, B, bk, a_rows, host));
  if (params->rhs_layout == IREE_B200_RHS_NK)
    return iree_b200_encode_tensor_map(context, es, bf, rhs, K, N, B, bk, use_pairs(context, params) ? bn / 2 : bn,
                                       host + 128);
  return iree_b200_encode_tensor_map(context, es, bf, rhs, N, K, B, bk, bk, host + 128);
}

iree_b200_status_t iree_b200_matmul_prepare(iree_b200_context_t* context, const iree_b200_matmul_params_t* params,
                                            const void* lhs, const void* rhs, void* workspace, int32_t* out_tile_n) {
  if (!context) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "context is NULL");
  B200_RETURN_IF_ERROR(validate(params));
  if (out_tile_n) *out_tile_n = 0;
  if (!params->M || !params->N || !params->batch) return IREE_B200_STATUS_OK;
  if (!tma_eligible(params, lhs, rhs) || !params->K) return IREE_B200_STATUS_OK;  // generic kernel: nothing to prepare
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) % 128))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "workspace must be a 128-byte aligned device buffer");
  const int es = elem_bytes_of(params->kind);
  const int bn = choose_tile_n(context, params);
  if (!bn) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "tile_n %d is not usable for this layout", params->tile_n);
  const int splits = choose_splits(context, params, bn);
  if (out_tile_n) *out_tile_n = bn | ((splits - 1) << 16);
  if (splits > 1) {  // the tile counters behind the header start at zero
    const int64_t tiles = static_cast<int64_t>((params->N + bn - 1) / bn) * params->batch;
    B200_RETURN_IF_ERROR(iree_hal_b200_fill_buffer(context->device, static_cast<uint8_t*>(workspace) + kSplitCountersOffset,
                                                   split_partials_offset(tiles) - kSplitCountersOffset, 0));
  }
  const uint32_t bk = 128 / es;
  const uint32_t M = params->M, N = params->N, K = params->K, B = params->batch;
  if (params->flags & IREE_B200_FLAG_DEVICE_TENSORMAPS) {
    // Templates: maps encoded once for a dummy tensor of the right element type.
    if (!context->templates) {
      uint8_t host[6 * 128];
      B200_RETURN_IF_ERROR(iree_hal_b200_buffer_allocate(context->device, sizeof host, &context->templates));
      for (int t = 0; t < 3; ++t) {
        const int tes = t == 2 ? 1 : 2;
        for (int i = 0; i < 2; ++i)
          B200_RETURN_IF_ERROR(iree_b200_encode_tensor_map(context, tes, t == 1, context->templates, 128 / tes * 4, 256,
                                                           1, 128 / tes, 64, host + (2 * t + i) * 128));
      }
      B200_RETURN_IF_ERROR(iree_hal_b200_transfer_h2d(context->device, host, context->templates, sizeof host));
    }
    const int t = params->kind == IREE_B200_KIND_I8 ? 2 : params->kind == IREE_B200_KIND_BF16 ? 1 : 0;
    iree_hal_b200_descriptor_set_binding_t bindings[4] = {
        {0, const_cast<void*>(lhs)},
        {1, const_cast<void*>(rhs)},
        {2, static_cast<uint8_t*>(context->templates) + 2 * t * 128},
        {3, workspace}};
    const int32_t constants[7] = {params->M, params->N, params->K, params->batch, params->rhs_layout,
                                  use_pairs(context, params) ? bn / 2 : bn, es};
    auto* cb = context->command_buffer;
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 4, bindings));
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, constants, sizeof constants));
    const int32_t ord = iree_hal_b200_executable_lookup(context->executable, "b200_encode_tensormaps");
    return iree_hal_b200_command_buffer_dispatch(cb, context->executable, ord, 4, 7, 1, 1, 1);
  }
  uint8_t host[IREE_B200_WORKSPACE_BYTES];
  B200_RETURN_IF_ERROR(encode_workspace_header(context, params, lhs, rhs, bn, host));
  // The source is pageable, so the driver has consumed it when this returns.
  return iree_hal_b200_transfer_h2d(context->device, host, workspace, sizeof host);
}

// A dispatch of an export that orders itself on the device (it waits there for the dispatch ahead
// before it touches global memory): launched early when the context allows dispatch overlap.
static iree_b200_status_t dispatch_self_ordering(iree_b200_context_t* context, int32_t ordinal, uint32_t binding_count,
                                                 uint32_t constant_count, uint32_t grid_x, uint32_t grid_y = 1) {
  auto* cb = context->command_buffer;
  const bool saved_overlap = cb->overlap;  // what the caller set on the command buffer itself survives
  cb->overlap = saved_overlap || context->dispatch_overlap;
  const iree_b200_status_t st = iree_hal_b200_command_buffer_dispatch(cb, context->executable, ordinal, binding_count,
                                                                      constant_count, grid_x, grid_y, 1);
  cb->overlap = saved_overlap;
  return st;
}

iree_b200_status_t iree_b200_matmul_run(iree_b200_context_t* context, const iree_b200_matmul_params_t* params,
                                        const void* lhs, const void* rhs, void* out, const float* row_scale,
                                        const float* col_scale, void* workspace, int32_t tile_n) {
  if (!context) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "context is NULL");
  B200_RETURN_IF_ERROR(validate(params));
  if (!params->M || !params->N || !params->batch) return IREE_B200_STATUS_OK;  // empty result
  if (!lhs || !rhs || !out) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "operand pointer is NULL");
  const bool requant = params->epilogue == IREE_B200_EPILOGUE_REQUANT_F16;
  if (requant && (!row_scale || !col_scale))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "the requant epilogue needs row and column scales");
  auto* cb = context->command_buffer;
  const bool generic = !tma_eligible(params, lhs, rhs) || !params->K;
  const bool pairs = !generic && use_pairs(context, params);
  const int32_t ord = iree_hal_b200_executable_lookup(
      context->executable, pairs ? pair_export_name(params->kind, params->epilogue)
                                 : export_name(params->kind, params->epilogue, generic));
  if (ord < 0) return fail(IREE_B200_STATUS_NOT_FOUND, "export missing from the executable");
  if (generic) {
    iree_hal_b200_descriptor_set_binding_t bindings[5] = {{0, const_cast<void*>(lhs)},
                                                          {1, const_cast<void*>(rhs)},
                                                          {2, out},
                                                          {3, const_cast<float*>(row_scale)},
                                                          {4, const_cast<float*>(col_scale)}};
    const int32_t constants[4] = {params->M, params->N, params->K, params->rhs_layout};
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, requant ? 5 : 3, bindings));
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, constants, sizeof constants));
    return iree_hal_b200_command_buffer_dispatch(cb, context->executable, ord, requant ? 5 : 3, 4,
                                                 (params->N + 15) / 16, (params->M + 15) / 16, params->batch);
  }
  if (!workspace) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "workspace is NULL");
  if (tile_n <= 0) return fail(IREE_B200_STATUS_FAILED_PRECONDITION, "run() needs the tile_n that prepare() returned");
  const int sms = usable_sms(context);
  const int width = tile_n & 0xffff, splits = (tile_n >> 16) + 1;
  if (splits > 1 && (pairs || params->M > kFewRows || width > 128 || splits > kMaxSplits))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "tile_n %#x asks for a K split this product cannot take", tile_n);
  uint32_t grid;
  if (pairs) {
    const int64_t tiles =
        static_cast<int64_t>((params->M + 255) / 256) * ((params->N + width - 1) / width) * params->batch;
    grid = 2u * static_cast<uint32_t>(tiles < sms / 2 ? tiles : sms / 2);  // whole pairs only
  } else {
    const int64_t items =
        static_cast<int64_t>((params->M + 127) / 128) * ((params->N + width - 1) / width) * params->batch * splits;
    grid = static_cast<uint32_t>(items < sms ? items : sms);
  }
  const int32_t constants[6] = {params->M, params->N, params->K, params->batch, params->rhs_layout, tile_n};
  if (requant) {
    iree_hal_b200_descriptor_set_binding_t bindings[4] = {
        {0, out}, {1, const_cast<float*>(row_scale)}, {2, const_cast<float*>(col_scale)}, {3, workspace}};
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 4, bindings));
  } else {
    iree_hal_b200_descriptor_set_binding_t bindings[2] = {{0, out}, {1, workspace}};
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 2, bindings));
  }
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, constants, sizeof constants));
  // These exports set up their barriers and tensor memory before they wait, on the device, for the
  // dispatch ahead of them: like the decode exports they may be launched early.
  return dispatch_self_ordering(context, ord, requant ? 4 : 2, 6, grid);
}

iree_b200_status_t iree_b200_matmul(iree_b200_context_t* context, const iree_b200_matmul_params_t* params,
                                    const void* lhs, const void* rhs, void* out, const float* row_scale,
                                    const float* col_scale, void* workspace) {
  int32_t tile_n = 0;
  B200_RETURN_IF_ERROR(iree_b200_matmul_prepare(context, params, lhs, rhs, workspace, &tile_n));
  return iree_b200_matmul_run(context, params, lhs, rhs, out, row_scale, col_scale, workspace, tile_n);
}

iree_b200_status_t iree_b200_workspace_status(iree_b200_context_t* context, const void* workspace) {
  if (!context || !workspace) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  uint32_t status[19] = {0};
  B200_RETURN_IF_ERROR(iree_hal_b200_transfer_d2h(context->device, static_cast<const uint8_t*>(workspace) + 384,
                                                  status, sizeof status));
  B200_RETURN_IF_ERROR(iree_hal_b200_device_synchronize(context->device));
  if (status[0] == 0) return IREE_B200_STATUS_OK;
  if (status[0] == 5) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "kernel rejected its arguments (shape / alignment)");
  if (status[16] == b200::kTcNoteMagic) {
    // A tensor-core decode dispatch that gave up may have left tile counters behind (status word 17
    // is its N): clear them and the status words, so the workspace is usable again.
    uint8_t* ws = static_cast<uint8_t*>(const_cast<void*>(workspace));
    B200_RETURN_IF_ERROR(iree_hal_b200_fill_buffer(context->device, ws + b200::kTcCountersOffset,
                                                   b200::tc_partials_offset(status[17]) - b200::kTcCountersOffset, 0));
    B200_RETURN_IF_ERROR(iree_hal_b200_fill_buffer(context->device, ws + 384, 64, 0));
    B200_RETURN_IF_ERROR(iree_hal_b200_device_synchronize(context->device));
    return fail(IREE_B200_STATUS_DEADLINE_EXCEEDED, "kernel wait %u ran out at iteration %u", status[0], status[1]);
  }
  if (status[0] >= 16 && status[2] > 0) {
    // A decode dispatch that gave up may have left tile counters of its slice reduction behind
    // (status word 2 is its N): clear them and the status words, so the workspace is usable again.
    uint8_t* ws = static_cast<uint8_t*>(const_cast<void*>(workspace));
    B200_RETURN_IF_ERROR(iree_hal_b200_fill_buffer(context->device, ws + IREE_B200_WORKSPACE_BYTES,
                                                   decode_counter_bytes(status[2]), 0));
    B200_RETURN_IF_ERROR(iree_hal_b200_fill_buffer(context->device, ws + 384, 64, 0));  // words 16.. keep the map's note
    B200_RETURN_IF_ERROR(iree_hal_b200_device_synchronize(context->device));
  }
  return fail(IREE_B200_STATUS_DEADLINE_EXCEEDED, "kernel wait %u ran out at iteration %u", status[0], status[1]);
}

}  // extern "C"

namespace {

// Device -> host copy of `bytes` on the readback stream, ordered after everything recorded on the
// dispatch stream so far.
iree_b200_status_t readback_after_dispatch(iree_hal_b200_device_t* d, const void* src, void* dst, size_t bytes) {
  if (!d->readback_stream) {
    CU_RETURN_IF_ERROR(g_cu.cuStreamCreate(&d->readback_stream, CU_STREAM_NON_BLOCKING), "cuStreamCreate");
    CU_RETURN_IF_ERROR(g_cu.cuEventCreate(&d->readback_ready, CU_EVENT_DISABLE_TIMING), "cuEventCreate");
  }
  CU_RETURN_IF_ERROR(g_cu.cuEventRecord(d->readback_ready, d->stream), "cuEventRecord");
  CU_RETURN_IF_ERROR(g_cu.cuStreamWaitEvent(d->readback_stream, d->readback_ready, 0), "cuStreamWaitEvent");
  CU_RETURN_IF_ERROR(g_cu.cuMemcpyDtoHAsync(dst, reinterpret_cast<CUdeviceptr>(src), bytes, d->readback_stream),
                     "cuMemcpyDtoHAsync");
  return IREE_B200_STATUS_OK;
}

}  // namespace

extern "C" {

iree_b200_status_t iree_b200_matmul_host(iree_b200_context_t* context, const iree_b200_matmul_params_t* params,
                                         const void* lhs, const void* rhs, void* out, const float* row_scale,
                                         const float* col_scale) {
  if (!context) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "context is NULL");
  // The host-buffer calls copy on the streams themselves and wait: they cannot become nodes of a graph.
  if (context->command_buffer->recording)
    return fail(IREE_B200_STATUS_FAILED_PRECONDITION, "a host-buffer call cannot be recorded into a graph");
  B200_RETURN_IF_ERROR(validate(params));
  const size_t es = elem_bytes_of(params->kind);
  const size_t os = params->epilogue == IREE_B200_EPILOGUE_ACCUMULATOR ? 4 : 2;
  const size_t a_bytes = static_cast<size_t>(params->batch) * params->M * params->K * es;
  const size_t b_bytes = static_cast<size_t>(params->batch) * params->K * params->N * es;
  const size_t c_bytes = static_cast<size_t>(params->batch) * params->M * params->N * os;
  if (!c_bytes) return IREE_B200_STATUS_OK;
  const bool requant = params->epilogue == IREE_B200_EPILOGUE_REQUANT_F16;
  if (requant && (!row_scale || !col_scale))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "the requant epilogue needs row and column scales");
  auto* d = context->device;
  auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
  // A product whose operands and result are many megabytes spends its time on the bus, not in
  // the kernel. It is then run as row blocks of the left-hand side: the block's rows go up, its
  // dispatch runs, and its result comes back on a second stream while the next block goes up, so
  // the two directions of the link work at the same time.
  constexpr int kMaxBlocks = 8;
  int blocks = 1;
  if (params->batch == 1 && params->M >= 1024 && a_bytes + c_bytes >= (static_cast<size_t>(16) << 20)) {
    blocks = params->M / 512;
    if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  }
  const int block_rows = blocks > 1 ? ((params->M + blocks - 1) / blocks + 255) / 256 * 256 : params->M;
  if (blocks > 1) blocks = (params->M + block_rows - 1) / block_rows;
  const size_t rs_bytes = requant ? sizeof(float) * params->M : 0, cs_bytes = requant ? sizeof(float) * params->N : 0;
  const size_t need = up(static_cast<size_t>(blocks) * IREE_B200_WORKSPACE_BYTES) + up(a_bytes) + up(b_bytes) + up(c_bytes) +
                      up(rs_bytes) + up(cs_bytes);
  if (need > context->arena_size) {
    B200_RETURN_IF_ERROR(iree_hal_b200_device_synchronize(d));
    if (context->arena) B200_RETURN_IF_ERROR(iree_hal_b200_buffer_free(d, context->arena));
    context->arena = nullptr;
    context->arena_size = 0;
    B200_RETURN_IF_ERROR(iree_hal_b200_buffer_allocate(d, need, &context->arena));
    context->arena_size = need;
  }
  uint8_t* base = static_cast<uint8_t*>(context->arena);
  uint8_t* ws = base;
  uint8_t* da = base + up(static_cast<size_t>(blocks) * IREE_B200_WORKSPACE_BYTES);
  uint8_t* db = da + up(a_bytes);
  uint8_t* dc = db + up(b_bytes);
  float* drs = reinterpret_cast<float*>(dc + up(c_bytes));
  float* dcs = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(drs) + up(rs_bytes));
  if (blocks == 1) B200_RETURN_IF_ERROR(iree_hal_b200_fill_buffer(d, ws, IREE_B200_WORKSPACE_BYTES, 0));
  B200_RETURN_IF_ERROR(iree_hal_b200_transfer_h2d(d, rhs, db, b_bytes));
  if (requant) {
    B200_RETURN_IF_ERROR(iree_hal_b200_transfer_h2d(d, row_scale, drs, rs_bytes));
    B200_RETURN_IF_ERROR(iree_hal_b200_transfer_h2d(d, col_scale, dcs, cs_bytes));
  }
  if (blocks == 1) {
    B200_RETURN_IF_ERROR(iree_hal_b200_transfer_h2d(d, lhs, da, a_bytes));
    B200_RETURN_IF_ERROR(iree_b200_matmul(context, params, da, db, dc, requant ? drs : nullptr, requant ? dcs : nullptr, ws));
    B200_RETURN_IF_ERROR(iree_hal_b200_transfer_d2h(d, dc, out, c_bytes));
    // Reads the status words back and waits for the stream: the result is in `out` on return.
    return iree_b200_workspace_status(context, ws);
  }
  // Every block's workspace header (tensor maps) is encoded first and uploaded in one copy, so
  // that no small host copy sits between the large ones.
  uint8_t headers[kMaxBlocks * IREE_B200_WORKSPACE_BYTES];
  int32_t block_tile_n[kMaxBlocks] = {0};
  memset(headers, 0, sizeof headers);
  for (int b = 0; b < blocks; ++b) {
    const int row0 = b * block_rows;
    iree_b200_matmul_params_t bp = *params;
    bp.M = params->M - row0 < block_rows ? params->M - row0 : block_rows;
    const uint8_t* a_block = da + static_cast<size_t>(row0) * params->K * es;
    if (tma_eligible(&bp, a_block, db) && bp.K) {
      block_tile_n[b] = choose_tile_n(context, &bp);
      if (!block_tile_n[b]) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "tile_n %d is not usable for this layout", bp.tile_n);
      B200_RETURN_IF_ERROR(encode_workspace_header(context, &bp, a_block, db, block_tile_n[b],
                                                   headers + static_cast<size_t>(b) * IREE_B200_WORKSPACE_BYTES));
    }
  }
  B200_RETURN_IF_ERROR(iree_hal_b200_transfer_h2d(d, headers, ws, static_cast<size_t>(blocks) * IREE_B200_WORKSPACE_BYTES));
  for (int b = 0; b < blocks; ++b) {
    const int row0 = b * block_rows;
    iree_b200_matmul_params_t bp = *params;
    bp.M = params->M - row0 < block_rows ? params->M - row0 : block_rows;
    const size_t a_off = static_cast<size_t>(row0) * params->K * es, c_off = static_cast<size_t>(row0) * params->N * os;
    B200_RETURN_IF_ERROR(iree_hal_b200_transfer_h2d(d, static_cast<const uint8_t*>(lhs) + a_off, da + a_off,
                                                    static_cast<size_t>(bp.M) * params->K * es));
    B200_RETURN_IF_ERROR(iree_b200_matmul_run(context, &bp, da + a_off, db, dc + c_off, requant ? drs + row0 : nullptr,
                                              requant ? dcs : nullptr, ws + static_cast<size_t>(b) * IREE_B200_WORKSPACE_BYTES,
                                              block_tile_n[b]));
    B200_RETURN_IF_ERROR(readback_after_dispatch(d, dc + c_off, static_cast<uint8_t*>(out) + c_off,
                                                 static_cast<size_t>(bp.M) * params->N * os));
  }
  // one read of every block's status words, then wait for both streams
  B200_RETURN_IF_ERROR(iree_hal_b200_transfer_d2h(d, ws, headers, static_cast<size_t>(blocks) * IREE_B200_WORKSPACE_BYTES));
  B200_RETURN_IF_ERROR(iree_hal_b200_device_synchronize(d));
  CU_RETURN_IF_ERROR(g_cu.cuStreamSynchronize(d->readback_stream), "cuStreamSynchronize");
  for (int b = 0; b < blocks; ++b) {
    uint32_t status[2];
    memcpy(status, headers + static_cast<size_t>(b) * IREE_B200_WORKSPACE_BYTES + 384, sizeof status);
    if (status[0] == 5) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "kernel rejected its arguments (shape / alignment)");
    if (status[0]) return fail(IREE_B200_STATUS_DEADLINE_EXCEEDED, "kernel wait %u ran out at iteration %u", status[0], status[1]);
  }
  return IREE_B200_STATUS_OK;
}

}  // extern "C"

extern "C" {

// ---- fused int4 dequant + matmul ---------------------------------------------------------------------
static int w4_variant(const iree_b200_context_t* ctx, const iree_b200_w4a16_params_t* p, const void* a, const void* wq,
                      const void* scales, const void* out) {
  if (p->variant != IREE_B200_W4A16_AUTO) return p->variant;
  const bool aligned = !(reinterpret_cast<uintptr_t>(a) % 16) && !(reinterpret_cast<uintptr_t>(wq) % 16) &&
                       !(reinterpret_cast<uintptr_t>(scales) % 2) && !(reinterpret_cast<uintptr_t>(out) % 2);
  // The decode kernel fetches scale rows with bulk copies: they need a 16-byte aligned base as well.
  const bool scales16 = !(reinterpret_cast<uintptr_t>(scales) % 16);
  if (p->group_size == 128 && aligned && scales16 && p->M <= 16 && p->N % 16 == 0 && p->K % 256 == 0 && p->K <= 16384)
    return IREE_B200_W4A16_DECODE;
  if (p->group_size == 128 && aligned && p->K % 128 == 0) {
    // The kernel with the weights as the tensor-memory operand (activation tiles of 128 rows up to
    // M = 128, of 256 above); it leaves its results by TMA stores, which need the result on 16-byte
    // boundaries. Otherwise the kernel with the expanded weights as a shared-memory operand.
    const bool out16 = !(reinterpret_cast<uintptr_t>(out) % 16) && (static_cast<int64_t>(p->ldo) * 2) % 16 == 0 &&
                       p->n_offset % 8 == 0;
    return out16 ? IREE_B200_W4A16_GEMM_WT : IREE_B200_W4A16_GEMM;
  }
  return IREE_B200_W4A16_GENERIC;
}

static iree_b200_status_t w4_validate(const iree_b200_w4a16_params_t* p) {
  if (!p) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "params is NULL");
  if (p->M < 0 || p->N < 0 || p->K < 0) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "negative dimension");
  if (p->group_size <= 0 || (p->group_size & 1) || p->K % p->group_size)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "K (%d) must be a multiple of an even group size (%d)", p->K,
                p->group_size);
  if (p->n_offset < 0 || static_cast<int64_t>(p->ldo) < static_cast<int64_t>(p->n_offset) + p->N)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "output pitch %d cannot hold columns [%d, %lld)", p->ldo, p->n_offset,
                static_cast<long long>(p->n_offset) + p->N);
  return IREE_B200_STATUS_OK;
}

size_t iree_b200_w4a16_workspace_bytes(int32_t N) {
  const int64_t n = N > 0 ? N : 0;
  // the decode kernels' slice-reduction scratch, and at least the output maps and arrival-word pointers
  // that the many-rows kernel keeps behind the 512-byte header
  size_t behind_header = decode_scratch_bytes(n, kDecodeMaxSlices);
  if (behind_header < static_cast<size_t>(kWtMaxDestinations) * (128 + 8)) behind_header = kWtMaxDestinations * (128 + 8);
  // the tensor-core decode kernel: tile counters and two partial sums per CTA
  if (behind_header < b200::tc_workspace_bytes(n) - IREE_B200_WORKSPACE_BYTES)
    behind_header = b200::tc_workspace_bytes(n) - IREE_B200_WORKSPACE_BYTES;
  return (IREE_B200_WORKSPACE_BYTES + behind_header + 255) & ~static_cast<size_t>(255);
}

static int w4_choose_tile_n(const iree_b200_context_t* ctx, const iree_b200_w4a16_params_t* p) {
  const int sms = usable_sms(ctx);
  // Tiles are a multiple of 16 and at most 128 columns wide. M >= 256 runs the kernel's 256-row
  // variant, which expands every weight half as often per flop; below that the 128-row variant
  // streams the weights once and the narrowest one-wave tile wins.
  const bool tall = p->M >= 256;
  const int64_t tiles_m = tall ? (p->M + 255) / 256 : (p->M + 127) / 128;
  int best = 0;
  double best_cost = 0;
  for (int bn = 128; bn >= 16; bn -= 16) {
    if (p->tile_n && bn != p->tile_n) continue;
    const int64_t tiles = tiles_m * ((p->N + bn - 1) / bn);
    const int64_t waves = (tiles + sms - 1) / sms;
    const double cost = static_cast<double>(waves) * (400.0 + (tall ? 2 * bn : bn));
    if (!best || cost < best_cost * 0.9999) {
      best = bn;
      best_cost = cost;
    }
  }
  return best;
}

// The decode kernels' view of the weights when K spans several 4096-wide slices: [N, K / 16] 8-byte
// elements, box 256 x 8 (eight rows of one slice, 16 KiB), no swizzle.
static iree_b200_status_t encode_decode_weight_map(const void* wq, int32_t N, int32_t K, void* out_map) {
  B200_RETURN_IF_ERROR(ensure_cuda());
  if ((reinterpret_cast<uintptr_t>(wq) % 16) || (K % 256))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "weights must start on a 16-byte boundary and K must be a multiple of 256");
  CUtensorMap map;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K) / 16, static_cast<cuuint64_t>(N)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) / 2};
  const cuuint32_t box[2] = {256, 8};
  const cuuint32_t estrides[2] = {1, 1};
  CU_RETURN_IF_ERROR(g_cu.cuTensorMapEncodeTiled(&map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(wq), dims, strides,
                                                 box, estrides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
                     "cuTensorMapEncodeTiled(weights)");
  memcpy(out_map, &map, 128);
  return IREE_B200_STATUS_OK;
}

// Rank-2 row-major f16 tensor [rows, cols] with row pitch `pitch_bytes`, no swizzle: the output maps of
// b200_w4a16_gemm_wt (box: 128 columns x 64 rows).
static iree_b200_status_t encode_output_map(const void* device_ptr, uint32_t cols, uint32_t rows, uint64_t pitch_bytes,
                                            void* out_map) {
  B200_RETURN_IF_ERROR(ensure_cuda());
  if ((reinterpret_cast<uintptr_t>(device_ptr) % 16) || pitch_bytes % 16)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "result base and row pitch must be multiples of 16 bytes");
  CUtensorMap map;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {128, 64};
  const cuuint32_t estrides[2] = {1, 1};
  CU_RETURN_IF_ERROR(g_cu.cuTensorMapEncodeTiled(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(device_ptr), dims,
                                                 strides, box, estrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                 CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
                     "cuTensorMapEncodeTiled(result)");
  memcpy(out_map, &map, 128);
  return IREE_B200_STATUS_OK;
}

// Workspace of b200_w4a16_gemm_wt: operand maps, zeroed status words, one output map per destination and
// (several ranks) the pointers to every rank's arrival words. 512 + 1024 + 64 bytes.
constexpr size_t kWtWorkspaceBytes = 512 + kWtMaxDestinations * 128 + kWtMaxDestinations * 8;
static iree_b200_status_t w4_encode_wt(const iree_b200_w4a16_params_t* params, const void* a, const void* wq,
                                       void* const* results, void* const* flags, int32_t world,
                                       uint8_t host[kWtWorkspaceBytes]) {
  if (world < 1 || world > kWtMaxDestinations)
    return fail(IREE_B200_STATUS_OUT_OF_RANGE, "1 to %d destinations", kWtMaxDestinations);
  if (params->n_offset % 8)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "n_offset must be a multiple of 8 (TMA stores start on 16-byte boundaries)");
  memset(host, 0, kWtWorkspaceBytes);
  B200_RETURN_IF_ERROR(encode_map(CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, CU_TENSOR_MAP_SWIZZLE_128B, 128, a, params->K,
                                  params->M, 1, 64, 128, host));
  B200_RETURN_IF_ERROR(encode_map(CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, CU_TENSOR_MAP_SWIZZLE_64B, 64, wq, params->K / 2,
                                  params->N, 1, 64, 128, host + 128));
  for (int32_t p = 0; p < world; ++p) {
    if (!results[p]) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "result buffer of rank %d is NULL", p);
    // columns beyond this rank's block are outside the map, so a ragged last tile cannot touch them
    B200_RETURN_IF_ERROR(encode_output_map(results[p], static_cast<uint32_t>(params->n_offset + params->N),
                                           static_cast<uint32_t>(params->M), static_cast<uint64_t>(params->ldo) * 2,
                                           host + 512 + 128 * p));
    if (flags) {
      const uint64_t f = reinterpret_cast<uint64_t>(flags[p]);
      memcpy(host + 512 + kWtMaxDestinations * 128 + 8 * p, &f, 8);
    }
  }
  return IREE_B200_STATUS_OK;
}
static iree_b200_status_t w4_prepare_wt(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                        const void* a, const void* wq, void* const* results, void* const* flags,
                                        int32_t world, void* workspace) {
  uint8_t host[kWtWorkspaceBytes];
  B200_RETURN_IF_ERROR(w4_encode_wt(params, a, wq, results, flags, world, host));
  return iree_hal_b200_transfer_h2d(context->device, host, workspace, sizeof host);
}

static iree_b200_status_t w4_check_decode_tc(const iree_b200_w4a16_params_t* params, const void* a, const void* wq,
                                             const void* scales) {
  if (params->group_size != 128 || params->M > b200::kTcARows || params->K % 256)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "the tensor-core decode kernel needs M <= 16, K %% 256 == 0, group 128");
  // TMA over activations and weights (16-byte bases and pitches), 4-byte copies of scale pairs
  if ((reinterpret_cast<uintptr_t>(a) % 16) || (reinterpret_cast<uintptr_t>(wq) % 16) ||
      (reinterpret_cast<uintptr_t>(scales) % 4))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT,
                "the tensor-core decode kernel needs activations and weights on 16-byte, scales on 4-byte boundaries");
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_b200_w4a16_prepare(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                           const void* a, const void* wq, const void* scales, const void* out,
                                           void* workspace, int32_t* out_variant, int32_t* out_tile_n) {
  if (!context) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "context is NULL");
  B200_RETURN_IF_ERROR(w4_validate(params));
  const int variant = w4_variant(context, params, a, wq, scales, out);
  if (out_variant) *out_variant = variant;
  if (out_tile_n) *out_tile_n = 0;
  if (variant == IREE_B200_W4A16_DECODE && params->K > kDecodeSliceK && params->N) {
    // K beyond one slice: the kernel fetches its weight tiles through a tensor map at the start of the workspace
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) % 128))
      return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "workspace must be a 128-byte aligned device buffer");
    uint8_t map[128];
    B200_RETURN_IF_ERROR(encode_decode_weight_map(wq, params->N, params->K, map));
    B200_RETURN_IF_ERROR(iree_hal_b200_transfer_h2d(context->device, map, workspace, sizeof map));
    // what the map was built for (status words 16..19): the kernel refuses a workspace without this note
    const uint64_t address = reinterpret_cast<uint64_t>(wq);
    const uint32_t note[4] = {static_cast<uint32_t>(address), static_cast<uint32_t>(address >> 32),
                              static_cast<uint32_t>(params->N), static_cast<uint32_t>(params->K)};
    return iree_hal_b200_transfer_h2d(context->device, note, static_cast<uint8_t*>(workspace) + 384 + 64, sizeof note);
  }
  if (variant == IREE_B200_W4A16_DECODE_TC && params->M && params->N) {
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) % 128))
      return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "workspace must be a 128-byte aligned device buffer");
    B200_RETURN_IF_ERROR(w4_check_decode_tc(params, a, wq, scales));
    // header: maps over the activations (boxes of 64 K x 16 rows) and the weights (seen as [N][K / 256][128
    // bytes], boxes of 128 rows x 2 x 128 bytes), status words with the note the kernel checks; behind it
    // the tile counters, zeroed
    std::vector<uint8_t> host(b200::tc_partials_offset(params->N), 0);
    B200_RETURN_IF_ERROR(encode_map(CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, CU_TENSOR_MAP_SWIZZLE_128B, 128, a, params->K,
                                    params->M, 1, 64, b200::kTcARows, host.data()));
    B200_RETURN_IF_ERROR(encode_map(CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, CU_TENSOR_MAP_SWIZZLE_128B, 128, wq, 128,
                                    params->K / 256, params->N, 128, b200::kTcUnitK / 256, host.data() + 128,
                                    b200::kTcWRows));
    const uint32_t note[3] = {b200::kTcNoteMagic, static_cast<uint32_t>(params->N), static_cast<uint32_t>(params->K)};
    memcpy(host.data() + 384 + 64, note, sizeof note);
    return iree_hal_b200_transfer_h2d(context->device, host.data(), workspace, host.size());
  }
  if ((variant != IREE_B200_W4A16_GEMM && variant != IREE_B200_W4A16_GEMM_WT) || !params->M || !params->N)
    return IREE_B200_STATUS_OK;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) % 128))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "workspace must be a 128-byte aligned device buffer");
  if (params->group_size != 128 || params->K % 128)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "the tensor-core kernel needs group size 128 and K %% 128 == 0");
  if (variant == IREE_B200_W4A16_GEMM_WT) {
    if (out_tile_n) *out_tile_n = 128;
    void* results[1] = {const_cast<void*>(out)};
    return w4_prepare_wt(context, params, a, wq, results, nullptr, 1, workspace);
  }
  const int bn = w4_choose_tile_n(context, params);
  if (!bn) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "tile_n %d is not usable", params->tile_n);
  if (out_tile_n) *out_tile_n = bn;
  uint8_t host[IREE_B200_WORKSPACE_BYTES];
  memset(host, 0, sizeof host);
  B200_RETURN_IF_ERROR(encode_map(CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, CU_TENSOR_MAP_SWIZZLE_128B, 128, a, params->K,
                                  params->M, 1, 64, 128, host));
  B200_RETURN_IF_ERROR(encode_map(CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, CU_TENSOR_MAP_SWIZZLE_64B, 64, wq, params->K / 2,
                                  params->N, 1, 64, bn, host + 128));
  return iree_hal_b200_transfer_h2d(context->device, host, workspace, sizeof host);
}

static iree_b200_status_t w4_run_wt(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                    const void* scales, void* out, void* workspace, int32_t world, int32_t rank,
                                    int32_t epoch) {
  if (!workspace) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "workspace is NULL");
  if (params->group_size != 128 || params->K % 128 || params->n_offset % 8)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "this kernel needs group size 128, K %% 128 == 0 and n_offset %% 8 == 0");
  auto* cb = context->command_buffer;
  iree_hal_b200_descriptor_set_binding_t bindings[3] = {{0, const_cast<void*>(scales)}, {1, out}, {2, workspace}};
  const int32_t constants[7] = {params->M, params->N, params->K, params->ldo, params->n_offset, (world << 8) | rank, epoch};
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 3, bindings));
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, constants, sizeof constants));
  const int sms = usable_sms(context);
  const int64_t tiles = static_cast<int64_t>((params->M + 255) / 256) * ((params->N + 127) / 128);
  const int32_t ord = iree_hal_b200_executable_lookup(context->executable, "b200_w4a16_gemm_wt");
  if (ord < 0) return fail(IREE_B200_STATUS_NOT_FOUND, "export b200_w4a16_gemm_wt missing from the executable");
  return dispatch_self_ordering(context, ord, 3, 7, static_cast<uint32_t>(tiles < sms ? tiles : sms));
}

iree_b200_status_t iree_b200_w4a16_prepare_push(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                                const void* a, const void* wq, const void* scales,
                                                void* const* results, void* const* flags, int32_t world,
                                                int32_t rank, void* workspace) {
  if (!context || !results || !flags) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  B200_RETURN_IF_ERROR(w4_validate(params));
  if (rank < 0 || rank >= world) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "rank %d is not in a channel of %d", rank, world);
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) % 128))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "workspace must be a 128-byte aligned device buffer");
  if (params->group_size != 128 || params->K % 128 || params->M < 256 || (reinterpret_cast<uintptr_t>(a) % 16) ||
      (reinterpret_cast<uintptr_t>(wq) % 16) || (reinterpret_cast<uintptr_t>(scales) % 2))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT,
                "the pushing dispatch needs M >= 256, group size 128, K %% 128 == 0 and 16-byte aligned operands");
  for (int32_t p = 0; p < world; ++p)
    if (!flags[p]) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "arrival words of rank %d are NULL", p);
  return w4_prepare_wt(context, params, a, wq, results, flags, world, workspace);
}

iree_b200_status_t iree_b200_w4a16_run_push(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                            const void* scales, void* result, void* workspace, int32_t world,
                                            int32_t rank, int32_t epoch) {
  if (!context) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "context is NULL");
  B200_RETURN_IF_ERROR(w4_validate(params));
  if (world < 1 || world > kWtMaxDestinations || rank < 0 || rank >= world)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "rank %d is not in a channel of %d (at most %d)", rank, world, kWtMaxDestinations);
  if (!scales || !result) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "operand pointer is NULL");
  return w4_run_wt(context, params, scales, result, workspace, world, rank, epoch);
}

iree_b200_status_t iree_b200_w4a16_wait_arrivals(iree_b200_context_t* context, const void* own_flags, void* workspace,
                                                 int32_t world, int32_t epoch) {
  if (!context || !own_flags || !workspace) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if (world < 1 || world > kWtMaxDestinations) return fail(IREE_B200_STATUS_OUT_OF_RANGE, "1 to %d ranks", kWtMaxDestinations);
  auto* cb = context->command_buffer;
  iree_hal_b200_descriptor_set_binding_t bindings[2] = {{0, const_cast<void*>(own_flags)}, {1, workspace}};
  const int32_t constants[2] = {world, epoch};
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 2, bindings));
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, constants, sizeof constants));
  const int32_t ord = iree_hal_b200_executable_lookup(context->executable, "b200_wait_arrivals");
  if (ord < 0) return fail(IREE_B200_STATUS_NOT_FOUND, "export b200_wait_arrivals missing from the executable");
  return iree_hal_b200_command_buffer_dispatch(cb, context->executable, ord, 2, 2, 1, 1, 1);
}

iree_b200_status_t iree_b200_w4a16_run(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                       const void* a, const void* wq, const void* scales, void* out, void* workspace,
                                       int32_t variant, int32_t tile_n) {
  if (!context) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "context is NULL");
  B200_RETURN_IF_ERROR(w4_validate(params));
  if (!params->M || !params->N) return IREE_B200_STATUS_OK;
  if (!a || !wq || !scales || !out) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "operand pointer is NULL");
  auto* cb = context->command_buffer;
  auto* exe = context->executable;
  const int sms = usable_sms(context);
  if (variant == IREE_B200_W4A16_DECODE) {
    if (params->group_size != 128 || params->M > 16 || params->N % 16 || params->K % 256 || params->K > 16384)
      return fail(IREE_B200_STATUS_INVALID_ARGUMENT,
                  "the decode kernel needs M <= 16, N %% 16 == 0, K %% 256 == 0, K <= 16384, group 128");
    // Bulk copies (weights, scales) and 16-byte loads (activations): a misaligned base would fault on the device.
    if ((reinterpret_cast<uintptr_t>(a) % 16) || (reinterpret_cast<uintptr_t>(wq) % 16) ||
        (reinterpret_cast<uintptr_t>(scales) % 16))
      return fail(IREE_B200_STATUS_INVALID_ARGUMENT,
                  "the decode kernel needs activations, weights and scales on 16-byte boundaries");
    if (!workspace) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "workspace is NULL");
    iree_hal_b200_descriptor_set_binding_t bindings[5] = {{0, const_cast<void*>(a)},
                                                          {1, const_cast<void*>(wq)},
                                                          {2, const_cast<void*>(scales)},
                                                          {3, out},
                                                          {4, workspace}};
    const int32_t constants[5] = {params->M, params->N, params->K, params->ldo, params->n_offset};
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 5, bindings));
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, constants, sizeof constants));
    const int32_t ord = iree_hal_b200_executable_lookup(exe, params->M <= 8 ? "b200_w4a16_decode_m8" : "b200_w4a16_decode_m16");
    // One CTA per SM; the CTAs that hold the K slices of the same tiles sit next to each other.
    const int tiles = params->N / 16;
    const int slices = (params->K + kDecodeSliceK - 1) / kDecodeSliceK;
    int walkers = sms / slices;
    if (walkers < 1) walkers = 1;
    if (walkers > tiles) walkers = tiles;
    const int gx = walkers * slices;
    // The decode exports order themselves on the device, so they may overlap the dispatch ahead.
    const bool saved_overlap = cb->overlap;  // what the caller set on the command buffer itself survives
    cb->overlap = saved_overlap || context->dispatch_overlap;
    const iree_b200_status_t st = iree_hal_b200_command_buffer_dispatch(cb, exe, ord, 5, 5, gx, 1, 1);
    cb->overlap = saved_overlap;
    return st;
  }
  if (variant == IREE_B200_W4A16_DECODE_TC) {
    B200_RETURN_IF_ERROR(w4_check_decode_tc(params, a, wq, scales));
    if (!workspace) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "workspace is NULL");
    iree_hal_b200_descriptor_set_binding_t bindings[3] = {{0, const_cast<void*>(scales)}, {1, out}, {2, workspace}};
    const int32_t constants[5] = {params->M, params->N, params->K, params->ldo, params->n_offset};
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 3, bindings));
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, constants, sizeof constants));
    const int32_t ord = iree_hal_b200_executable_lookup(exe, "b200_w4a16_decode_tc");
    // equal contiguous ranges of (128 rows x 512 K) units, one CTA per SM
    const int64_t units = static_cast<int64_t>((params->N + b200::kTcWRows - 1) / b200::kTcWRows) *
                          ((params->K + b200::kTcUnitK - 1) / b200::kTcUnitK);
    int64_t gx = sms < b200::kTcMaxCtas ? sms : b200::kTcMaxCtas;
    if (gx > units) gx = units;
    const bool saved_overlap = cb->overlap;
    cb->overlap = saved_overlap || context->dispatch_overlap;
    const iree_b200_status_t st = iree_hal_b200_command_buffer_dispatch(cb, exe, ord, 3, 5, static_cast<uint32_t>(gx), 1, 1);
    cb->overlap = saved_overlap;
    return st;
  }
  if (variant == IREE_B200_W4A16_GEMM) {
    if (!workspace) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "workspace is NULL");
    if (tile_n <= 0) return fail(IREE_B200_STATUS_FAILED_PRECONDITION, "run() needs the tile_n that prepare() returned");
    iree_hal_b200_descriptor_set_binding_t bindings[3] = {{0, const_cast<void*>(scales)}, {1, out}, {2, workspace}};
    const int32_t constants[6] = {params->M, params->N, params->K, params->ldo, params->n_offset, tile_n};
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 3, bindings));
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, constants, sizeof constants));
    const int tile_rows = params->M >= 256 ? 256 : 128;  // the kernel's 256-row variant
    const int64_t tiles = static_cast<int64_t>((params->M + tile_rows - 1) / tile_rows) * ((params->N + tile_n - 1) / tile_n);
    const int32_t ord = iree_hal_b200_executable_lookup(exe, "b200_w4a16_gemm");
    return dispatch_self_ordering(context, ord, 3, 6, static_cast<uint32_t>(tiles < sms ? tiles : sms));
  }
  if (variant == IREE_B200_W4A16_GEMM_WT) return w4_run_wt(context, params, scales, out, workspace, 1, 0, 0);
  if (variant == IREE_B200_W4A16_GENERIC) {
    iree_hal_b200_descriptor_set_binding_t bindings[4] = {
        {0, const_cast<void*>(a)}, {1, const_cast<void*>(wq)}, {2, const_cast<void*>(scales)}, {3, out}};
    const int32_t constants[6] = {params->M, params->N, params->K, params->group_size, params->ldo, params->n_offset};
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 4, bindings));
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, constants, sizeof constants));
    const int32_t ord = iree_hal_b200_executable_lookup(exe, "b200_w4a16_generic");
    return iree_hal_b200_command_buffer_dispatch(cb, exe, ord, 4, 6, (params->N + 255) / 256, params->M, 1);
  }
  return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "unknown W4A16 variant %d", variant);
}

iree_b200_status_t iree_b200_w4a16(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                   const void* a, const void* wq, const void* scales, void* out, void* workspace) {
  int32_t variant = 0, tile_n = 0;
  B200_RETURN_IF_ERROR(iree_b200_w4a16_prepare(context, params, a, wq, scales, out, workspace, &variant, &tile_n));
  return iree_b200_w4a16_run(context, params, a, wq, scales, out, workspace, variant, tile_n);
}

// A many-rows product whose operands and result are tens of megabytes spends its time on the bus. It is
// cut into units that follow the operands' arrival: blocks of activation rows and blocks of weight rows go
// up in turn (by bytes), and every new block is multiplied at once with all the blocks of the other operand
// that are on the device - a rectangle of the result per unit - so results start to leave after a few
// percent of the operands have arrived and the rectangles grow as fast as the link allows. Uploads run on a
// stream of their own, each unit's dispatch waits for its upload, and its rectangle returns by a pitched
// copy on the readback stream: both directions of the link are busy for most of the call. (Letting the
// kernel's TMA stores write page-locked host memory directly was measured too: 42-48 GB/s against the copy
// engine's 55, and it slowed the uploads.)
// Block counts from a sweep on the 70B shape (weight-row blocks x activation-row blocks: 8 x 4 6.03 ms, 16 x 8 6.42,
// 4 x 4 6.21, 8 x 2 6.33): fewer, larger copies move faster beside the kernels than many small ones.
constexpr int kHostMaxColBlocks = 8, kHostMaxRowBlocks = 4, kHostMaxUnits = kHostMaxColBlocks + kHostMaxRowBlocks;
constexpr size_t kHostUnitWorkspace = (kWtWorkspaceBytes + 255) & ~static_cast<size_t>(255);
static bool w4_host_in_units(const iree_b200_w4a16_params_t* p, size_t w_bytes, size_t c_bytes) {
  return p->variant == IREE_B200_W4A16_AUTO && p->group_size == 128 && p->K % 128 == 0 &&
         p->M >= 256 && p->N >= 2048 && p->N % 8 == 0 && p->ldo == p->N && p->n_offset == 0 &&
         w_bytes + c_bytes >= (static_cast<size_t>(32) << 20);  // N % 8: the result rows are TMA-stored (16-byte pitch)
}
// A unit: the rectangle [row0, row0 + rows) x [col0, col0 + cols) of the result, computed after the upload
// of one block of weight rows (new_cols), of activation rows (new_rows), or - the first - of both.
struct HostUnit {
  int64_t row0, rows, col0, cols;
  bool new_rows, new_cols;
};
// At most 4 blocks of activation rows (multiples of 256 rows) and 8 of weight rows (multiples of 256);
// the operand that has fewer bytes on the device so far gets the next block.
static int w4_plan_units(const iree_b200_w4a16_params_t* params, HostUnit* units) {
  const int64_t M = params->M, N = params->N, K = params->K;
  int col_blocks = static_cast<int>(N / 1024 < kHostMaxColBlocks ? N / 1024 : kHostMaxColBlocks);
  if (col_blocks < 1) col_blocks = 1;
  const int64_t block_cols = ((N + col_blocks - 1) / col_blocks + 255) / 256 * 256;
  col_blocks = static_cast<int>((N + block_cols - 1) / block_cols);
  int row_blocks = static_cast<int>(M / 512 < kHostMaxRowBlocks ? M / 512 : kHostMaxRowBlocks);
  if (row_blocks < 1) row_blocks = 1;
  const int64_t block_rows = ((M + row_blocks - 1) / row_blocks + 255) / 256 * 256;
  row_blocks = static_cast<int>((M + block_rows - 1) / block_rows);
  const size_t w_pitch = static_cast<size_t>(K / 2), s_pitch = static_cast<size_t>(K / 128) * 2, a_pitch = static_cast<size_t>(K) * 2;
  int count = 0, rows_up = 1, cols_up = 1;
  auto rows_to = [&](int blocks) { return blocks * block_rows < M ? blocks * block_rows : M; };
  auto cols_to = [&](int blocks) { return blocks * block_cols < N ? blocks * block_cols : N; };
  units[count++] = {0, rows_to(1), 0, cols_to(1), true, true};
  while (rows_up < row_blocks || cols_up < col_blocks) {
    const bool weights_next = cols_up < col_blocks && (rows_up == row_blocks || cols_to(cols_up) * (w_pitch + s_pitch) <= rows_to(rows_up) * a_pitch);
    if (weights_next) {
      units[count++] = {0, rows_to(rows_up), cols_to(cols_up), cols_to(cols_up + 1) - cols_to(cols_up), false, true};
      ++cols_up;
    } else {
      units[count++] = {rows_to(rows_up), rows_to(rows_up + 1) - rows_to(rows_up), 0, cols_to(cols_up), true, false};
      ++rows_up;
    }
  }
  return count;
}
static iree_b200_status_t w4_host_units(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                        const uint8_t* a, const uint8_t* wq, const uint8_t* scales, uint8_t* out,
                                        uint8_t* ws, uint8_t* da, uint8_t* dw, uint8_t* ds, uint8_t* dc) {
  if (!a || !wq || !scales || !out) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "operand pointer is NULL");
  auto* d = context->device;
  if (!d->readback_stream) {
    CU_RETURN_IF_ERROR(g_cu.cuStreamCreate(&d->readback_stream, CU_STREAM_NON_BLOCKING), "cuStreamCreate");
    CU_RETURN_IF_ERROR(g_cu.cuEventCreate(&d->readback_ready, CU_EVENT_DISABLE_TIMING), "cuEventCreate");
  }
  if (!d->upload_stream) {
    CU_RETURN_IF_ERROR(g_cu.cuStreamCreate(&d->upload_stream, CU_STREAM_NON_BLOCKING), "cuStreamCreate");
    CU_RETURN_IF_ERROR(g_cu.cuEventCreate(&d->upload_ready, CU_EVENT_DISABLE_TIMING), "cuEventCreate");
  }
  const int64_t N = params->N, K = params->K;
  const size_t w_pitch = static_cast<size_t>(K / 2), s_pitch = static_cast<size_t>(K / 128) * 2, a_pitch = static_cast<size_t>(K) * 2;
  HostUnit units[kHostMaxUnits];
  const int count = w4_plan_units(params, units);
  // every unit's header (operand and result maps) is encoded first and uploaded in one copy
  std::vector<uint8_t> headers(static_cast<size_t>(count) * kHostUnitWorkspace, 0);
  iree_b200_w4a16_params_t up[kHostMaxUnits];
  for (int u = 0; u < count; ++u) {
    up[u] = *params;
    up[u].variant = IREE_B200_W4A16_GEMM_WT;
    up[u].M = static_cast<int32_t>(units[u].rows);
    up[u].N = static_cast<int32_t>(units[u].cols);
    up[u].n_offset = static_cast<int32_t>(units[u].col0);
    void* results[1] = {dc + static_cast<size_t>(units[u].row0) * N * 2};
    B200_RETURN_IF_ERROR(w4_encode_wt(&up[u], da + static_cast<size_t>(units[u].row0) * a_pitch,
                                      dw + static_cast<size_t>(units[u].col0) * w_pitch, results, nullptr, 1,
                                      headers.data() + static_cast<size_t>(u) * kHostUnitWorkspace));
  }
  B200_RETURN_IF_ERROR(iree_hal_b200_transfer_h2d(d, headers.data(), ws, headers.size()));
  // uploads start after whatever the dispatch stream still runs on the arena
  CU_RETURN_IF_ERROR(g_cu.cuEventRecord(d->upload_ready, d->stream), "cuEventRecord");
  CU_RETURN_IF_ERROR(g_cu.cuStreamWaitEvent(d->upload_stream, d->upload_ready, 0), "cuStreamWaitEvent");
  auto upload = [&](const uint8_t* src, uint8_t* dst, size_t bytes) -> iree_b200_status_t {
    CU_RETURN_IF_ERROR(g_cu.cuMemcpyHtoDAsync(reinterpret_cast<CUdeviceptr>(dst), src, bytes, d->upload_stream),
                       "cuMemcpyHtoDAsync");
    return IREE_B200_STATUS_OK;
  };
  for (int u = 0; u < count; ++u) {
    const HostUnit& t = units[u];
    if (t.new_cols) {  // a block of weight rows with its scales
      B200_RETURN_IF_ERROR(upload(wq + static_cast<size_t>(t.col0) * w_pitch, dw + static_cast<size_t>(t.col0) * w_pitch,
                                  static_cast<size_t>(t.cols) * w_pitch));
      B200_RETURN_IF_ERROR(upload(scales + static_cast<size_t>(t.col0) * s_pitch, ds + static_cast<size_t>(t.col0) * s_pitch,
                                  static_cast<size_t>(t.cols) * s_pitch));
    }
    if (t.new_rows)  // a block of activation rows
      B200_RETURN_IF_ERROR(upload(a + static_cast<size_t>(t.row0) * a_pitch, da + static_cast<size_t>(t.row0) * a_pitch,
                                  static_cast<size_t>(t.rows) * a_pitch));
    CU_RETURN_IF_ERROR(g_cu.cuEventRecord(d->upload_ready, d->upload_stream), "cuEventRecord");
    CU_RETURN_IF_ERROR(g_cu.cuStreamWaitEvent(d->stream, d->upload_ready, 0), "cuStreamWaitEvent");
    uint8_t* unit_out = dc + static_cast<size_t>(t.row0) * N * 2;
    B200_RETURN_IF_ERROR(w4_run_wt(context, &up[u], ds + static_cast<size_t>(t.col0) * s_pitch, unit_out,
                                   ws + static_cast<size_t>(u) * kHostUnitWorkspace, 1, 0, 0));
    CU_RETURN_IF_ERROR(g_cu.cuEventRecord(d->readback_ready, d->stream), "cuEventRecord");
    CU_RETURN_IF_ERROR(g_cu.cuStreamWaitEvent(d->readback_stream, d->readback_ready, 0), "cuStreamWaitEvent");
    CUDA_MEMCPY2D copy;
    memset(&copy, 0, sizeof copy);
    copy.srcMemoryType = CU_MEMORYTYPE_DEVICE;
    copy.srcDevice = reinterpret_cast<CUdeviceptr>(unit_out + static_cast<size_t>(t.col0) * 2);
    copy.srcPitch = static_cast<size_t>(N) * 2;
    copy.dstMemoryType = CU_MEMORYTYPE_HOST;
    copy.dstHost = out + (static_cast<size_t>(t.row0) * N + static_cast<size_t>(t.col0)) * 2;
    copy.dstPitch = static_cast<size_t>(N) * 2;
    copy.WidthInBytes = static_cast<size_t>(t.cols) * 2;
    copy.Height = static_cast<size_t>(t.rows);
    CU_RETURN_IF_ERROR(g_cu.cuMemcpy2DAsync(&copy, d->readback_stream), "cuMemcpy2DAsync");
  }
  // one read of every unit's status words, then wait for the dispatch and readback streams
  uint32_t status[kHostMaxUnits][2];
  CUDA_MEMCPY2D words;
  memset(&words, 0, sizeof words);
  words.srcMemoryType = CU_MEMORYTYPE_DEVICE;
  words.srcDevice = reinterpret_cast<CUdeviceptr>(ws + 384);
  words.srcPitch = kHostUnitWorkspace;
  words.dstMemoryType = CU_MEMORYTYPE_HOST;
  words.dstHost = status;
  words.dstPitch = sizeof status[0];
  words.WidthInBytes = sizeof status[0];
  words.Height = static_cast<size_t>(count);
  CU_RETURN_IF_ERROR(g_cu.cuMemcpy2DAsync(&words, d->stream), "cuMemcpy2DAsync");
  B200_RETURN_IF_ERROR(iree_hal_b200_device_synchronize(d));
  CU_RETURN_IF_ERROR(g_cu.cuStreamSynchronize(d->readback_stream), "cuStreamSynchronize");
  for (int u = 0; u < count; ++u) {
    if (status[u][0] == 5) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "kernel rejected its arguments (shape / alignment)");
    if (status[u][0]) return fail(IREE_B200_STATUS_DEADLINE_EXCEEDED, "kernel wait %u ran out at iteration %u", status[u][0], status[u][1]);
  }
  return IREE_B200_STATUS_OK;
}

int32_t iree_b200_w4a16_host_plan(const iree_b200_w4a16_params_t* params, int32_t* out_units, int32_t capacity) {
  if (!params || w4_validate(params) != IREE_B200_STATUS_OK) return -1;
  const size_t w_bytes = static_cast<size_t>(params->N) * (params->K / 2);
  const size_t c_bytes = static_cast<size_t>(params->M) * params->ldo * 2;
  if (!params->M || !params->N || !w4_host_in_units(params, w_bytes, c_bytes)) return 0;
  HostUnit units[kHostMaxUnits];
  const int count = w4_plan_units(params, units);
  for (int u = 0; u < count && u < capacity && out_units; ++u) {
    int32_t* o = out_units + 6 * u;
    o[0] = static_cast<int32_t>(units[u].row0), o[1] = static_cast<int32_t>(units[u].rows);
    o[2] = static_cast<int32_t>(units[u].col0), o[3] = static_cast<int32_t>(units[u].cols);
    o[4] = units[u].new_rows, o[5] = units[u].new_cols;
  }
  return count;
}

iree_b200_status_t iree_b200_w4a16_host(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                        const void* a, const void* wq, const void* scales, void* out) {
  if (!context) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "context is NULL");
  if (context->command_buffer->recording)
    return fail(IREE_B200_STATUS_FAILED_PRECONDITION, "a host-buffer call cannot be recorded into a graph");
  B200_RETURN_IF_ERROR(w4_validate(params));
  const size_t a_bytes = static_cast<size_t>(params->M) * params->K * 2;
  const size_t w_bytes = static_cast<size_t>(params->N) * (params->K / 2);
  const size_t s_bytes = static_cast<size_t>(params->N) * (params->K / params->group_size) * 2;
  const size_t c_bytes = static_cast<size_t>(params->M) * params->ldo * 2;
  if (!params->M || !params->N) return IREE_B200_STATUS_OK;
  auto* d = context->device;
  auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
  const bool in_units = g_cu.cuMemcpy2DAsync && w4_host_in_units(params, w_bytes, c_bytes);
  const size_t ws_bytes = in_units ? kHostMaxUnits * kHostUnitWorkspace : iree_b200_w4a16_workspace_bytes(params->N);
  const size_t need = up(ws_bytes) + up(a_bytes) + up(w_bytes) + up(s_bytes) + up(c_bytes);
  if (need > context->arena_size) {
    B200_RETURN_IF_ERROR(iree_hal_b200_device_synchronize(d));
    if (context->arena) B200_RETURN_IF_ERROR(iree_hal_b200_buffer_free(d, context->arena));
    context->arena = nullptr;
    context->arena_size = 0;
    B200_RETURN_IF_ERROR(iree_hal_b200_buffer_allocate(d, need, &context->arena));
    context->arena_size = need;
  }
  uint8_t* base = static_cast<uint8_t*>(context->arena);
  void* ws = base;
  void* da = base + up(ws_bytes);
  void* dw = static_cast<uint8_t*>(da) + up(a_bytes);
  void* ds = static_cast<uint8_t*>(dw) + up(w_bytes);
  void* dc = static_cast<uint8_t*>(ds) + up(s_bytes);
  if (in_units)
    return w4_host_units(context, params, static_cast<const uint8_t*>(a), static_cast<const uint8_t*>(wq),
                         static_cast<const uint8_t*>(scales), static_cast<uint8_t*>(out), base, static_cast<uint8_t*>(da),
                         static_cast<uint8_t*>(dw), static_cast<uint8_t*>(ds), static_cast<uint8_t*>(dc));
  // The decode scratch (K > 4096) must start at zero; the kernel leaves it zero afterwards, but the arena
  // is shared with other entry points, so it is cleared on every call here (a few hundred KiB).
  B200_RETURN_IF_ERROR(iree_hal_b200_fill_buffer(d, ws, ws_bytes, 0));
  B200_RETURN_IF_ERROR(iree_hal_b200_transfer_h2d(d, a, da, a_bytes));
  B200_RETURN_IF_ERROR(iree_hal_b200_transfer_h2d(d, wq, dw, w_bytes));
  B200_RETURN_IF_ERROR(iree_hal_b200_transfer_h2d(d, scales, ds, s_bytes));
  if (params->ldo != params->N) B200_RETURN_IF_ERROR(iree_hal_b200_transfer_h2d(d, out, dc, c_bytes));
  B200_RETURN_IF_ERROR(iree_b200_w4a16(context, params, da, dw, ds, dc, ws));
  B200_RETURN_IF_ERROR(iree_hal_b200_transfer_d2h(d, dc, out, c_bytes));
  return iree_b200_workspace_status(context, ws);
}

// ---- command sequences -------------------------------------------------------------------------------
// A recorded run of `count` dispatches over rotating operand sets, issued from C in one call:
// what replaying a command buffer that holds `count` dispatches does in the reference
// (runtime/src/iree/hal/drivers/cuda/pending_queue_actions.c:729-742). Step i uses operand set
// (first + i) % set_count.
iree_b200_status_t iree_b200_matmul_run_sequence(iree_b200_context_t* context, const iree_b200_matmul_params_t* params,
                                                 int32_t set_count, const void* const* lhs, const void* const* rhs,
                                                 void* const* out, const float* const* row_scale,
                                                 const float* const* col_scale, void* const* workspace,
                                                 int32_t tile_n, int32_t first, int32_t count) {
  if (set_count < 1 || !lhs || !rhs || !out || !workspace) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  for (int32_t i = 0; i < count; ++i) {
    const int32_t s = (first + i) % set_count;
    B200_RETURN_IF_ERROR(iree_b200_matmul_run(context, params, lhs[s], rhs[s], out[s], row_scale ? row_scale[s] : nullptr,
                                              col_scale ? col_scale[s] : nullptr, workspace[s], tile_n));
  }
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_b200_w4a16_run_sequence(iree_b200_context_t* context, const iree_b200_w4a16_params_t* params,
                                                int32_t set_count, const void* const* a, const void* const* wq,
                                                const void* const* scales, void* const* out, void* const* workspace,
                                                int32_t variant, int32_t tile_n, int32_t first, int32_t count) {
  if (set_count < 1 || !a || !wq || !scales || !out || !workspace)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  for (int32_t i = 0; i < count; ++i) {
    const int32_t s = (first + i) % set_count;
    B200_RETURN_IF_ERROR(iree_b200_w4a16_run(context, params, a[s], wq[s], scales[s], out[s], workspace[s], variant, tile_n));
  }
  return IREE_B200_STATUS_OK;
}

}  // extern "C"

// ---- pack / unpack / mmt4d ----------------------------------------------------------------------------

namespace {

constexpr uint32_t kUkTransposeInner = 0x100, kUkTransposeOuter = 0x200;
constexpr uint32_t kTilingAccumulateI32 = 0x10000, kTilingAccumulateF32 = 0x20000;

int pack_elem_bytes(uint32_t flags) {
  switch (flags & IREE_B200_UK_FLAG_PACK_TYPE_MASK) {
    case IREE_B200_UK_FLAG_PACK_TYPE_F32F32:
    case IREE_B200_UK_FLAG_PACK_TYPE_I32I32: return 4;
    case IREE_B200_UK_FLAG_PACK_TYPE_I8I8: return 1;
    case IREE_B200_UK_FLAG_PACK_TYPE_F16F16:
    case IREE_B200_UK_FLAG_PACK_TYPE_BF16BF16: return 2;
    default: return 0;
  }
}

bool fits_i32(int64_t v) { return v >= 0 && v <= INT32_MAX; }

// Grid of the tiling kernels: one CTA per staged region (at most 64 rows by 256 bytes of whole
// tiles), or a bounded grid-stride launch when a tile is too large to stage.
uint32_t tiling_grid(int64_t o0, int64_t o1, int64_t o2, int64_t o3, uint32_t flags, int es, int sms) {
  const bool ti = flags & kUkTransposeInner, to = flags & kUkTransposeOuter;
  const int64_t tile0 = ti ? o3 : o2, tile1 = ti ? o2 : o3, outer0 = to ? o1 : o0, outer1 = to ? o0 : o1;
  if (tile0 > 0 && tile1 > 0 && tile0 <= 64 && tile1 * es <= 512) {
    const int64_t nr = 64 / tile0;
    int64_t nc = (256 / es) / tile1;
    if (nc == 0) nc = 1;
    return static_cast<uint32_t>(((outer0 + nr - 1) / nr) * ((outer1 + nc - 1) / nc));
  }
  const int64_t blocks = (o0 * o1 * o2 * o3 + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sms) * 8;
  return static_cast<uint32_t>(blocks < cap ? blocks : cap);
}

// Three rank-4 template maps (1-, 2-, 4-byte elements, no swizzle) and 256 bytes per CTA for the maps the
// TMA tiling kernels build on the device.
constexpr int kTilingScratchSlots = 1024;
constexpr size_t kTilingStatusOffset = 3072;  // a status word; the per-CTA slots follow 1024 bytes later
iree_b200_status_t ensure_tiling_scratch(iree_b200_context_t* ctx) {
  if (ctx->tiling_scratch) return IREE_B200_STATUS_OK;
  uint8_t host[3 * 128];
  void* scratch = nullptr;
  B200_RETURN_IF_ERROR(iree_hal_b200_buffer_allocate(ctx->device, 4096 + kTilingScratchSlots * 256, &scratch));
  const CUtensorMapDataType types[3] = {CU_TENSOR_MAP_DATA_TYPE_UINT8, CU_TENSOR_MAP_DATA_TYPE_UINT16,
                                        CU_TENSOR_MAP_DATA_TYPE_UINT32};
  for (int i = 0; i < 3; ++i) {
    // any valid rank-4 tensor will do: address, extents, pitches and box are replaced on the device
    const cuuint64_t e = 1ull << i;
    const cuuint64_t dims[4] = {64, 4, 4, 4};
    const cuuint64_t strides[3] = {64 * e, 256 * e, 1024 * e};
    const cuuint32_t box[4] = {static_cast<cuuint32_t>(16 / e), 1, 1, 1}, estrides[4] = {1, 1, 1, 1};
    CUtensorMap map;
    const CUresult r = g_cu.cuTensorMapEncodeTiled(&map, types[i], 4, scratch, dims, strides, box, estrides,
                                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      iree_hal_b200_buffer_free(ctx->device, scratch);
      return fail(IREE_B200_STATUS_INTERNAL, "cuTensorMapEncodeTiled(rank-4 template) failed: %d", static_cast<int>(r));
    }
    memcpy(host + 128 * i, &map, 128);
  }
  iree_b200_status_t st = iree_hal_b200_fill_buffer(ctx->device, scratch, 4096, 0);
  if (st == IREE_B200_STATUS_OK) st = iree_hal_b200_transfer_h2d(ctx->device, host, scratch, sizeof host);
  if (st != IREE_B200_STATUS_OK) {
    iree_hal_b200_buffer_free(ctx->device, scratch);
    return st;
  }
  ctx->tiling_scratch = scratch;
  return IREE_B200_STATUS_OK;
}

// The int8 right-hand side of the VNNI mmt4d ([K, N] -> [N1, K1, 16, 2], both transposes): TMA box in,
// byte interleave in shared memory, bulk copies out (pack_vnni_sm100.cu).
iree_b200_status_t pack_rhs_16x2(iree_b200_context_t* ctx, const void* in, void* out, int64_t K, int64_t N,
                                 int64_t rm_stride0, int64_t rm_stride1, int64_t t0, int64_t t1, int64_t t2, int64_t t3,
                                 int64_t t_stride0, uint32_t kernel_flags, uint64_t padding, bool* dispatched) {
  *dispatched = false;
  if (!(kernel_flags & kUkTransposeInner) || !(kernel_flags & kUkTransposeOuter) || t2 != 16 || t3 != 2) return IREE_B200_STATUS_OK;
  if ((kernel_flags & (kTilingAccumulateI32 | kTilingAccumulateF32)) || rm_stride1 != 1) return IREE_B200_STATUS_OK;
  const bool ragged = t1 * 2 != K || t0 * 16 != N;
  if (ragged && (padding & 0xff)) return IREE_B200_STATUS_OK;  // the TMA unit fills with zero
  if (t1 * 2 < K || t0 * 16 < N || rm_stride0 < N || t_stride0 < t1 * 32) return IREE_B200_STATUS_OK;
  if ((rm_stride0 & 15) || (t_stride0 & 15) || ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15))
    return IREE_B200_STATUS_OK;
  const int ctas = 2 * usable_sms(ctx);  // two CTAs per SM: eight 16 KiB loads in flight on each SM
  if (ctas > kTilingScratchSlots) return IREE_B200_STATUS_OK;
  B200_RETURN_IF_ERROR(ensure_tiling_scratch(ctx));
  const int32_t ord = iree_hal_b200_executable_lookup(ctx->executable, "b200_pack_i8_rhs_16x2");
  if (ord < 0) return fail(IREE_B200_STATUS_NOT_FOUND, "export b200_pack_i8_rhs_16x2 missing from the executable");
  const int64_t regions = ((t0 + 7) / 8) * ((t1 + 63) / 64);
  uint8_t* scratch = static_cast<uint8_t*>(ctx->tiling_scratch);
  iree_hal_b200_descriptor_set_binding_t bindings[4] = {{0, const_cast<void*>(in)}, {1, out}, {2, scratch}, {3, scratch + kTilingStatusOffset}};
  const int32_t c[6] = {(int32_t)K, (int32_t)N, (int32_t)rm_stride0, (int32_t)t0, (int32_t)t1, (int32_t)t_stride0};
  auto* cb = ctx->command_buffer;
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 4, bindings));
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, c, sizeof c));
  *dispatched = true;
  return dispatch_self_ordering(ctx, ord, 4, 6, static_cast<uint32_t>(regions < ctas ? regions : ctas));
}

// The left-hand side of the same family: tiles of sixteen rows x two bytes without transposes (int8 16 x 2,
// f16 / bf16 16 x 1), same kernel file, two-byte pieces of sixteen rows gathered into a tile.
iree_b200_status_t pack_lhs_16x2b(iree_b200_context_t* ctx, int es, const void* in, void* out, int64_t rows, int64_t cols,
                                  int64_t rm_stride0, int64_t rm_stride1, int64_t t0, int64_t t1, int64_t t2, int64_t t3,
                                  int64_t t_stride0, uint32_t kernel_flags, uint64_t padding, bool* dispatched) {
  *dispatched = false;
  if ((kernel_flags & (kUkTransposeInner | kUkTransposeOuter | kTilingAccumulateI32 | kTilingAccumulateF32)) || rm_stride1 != 1)
    return IREE_B200_STATUS_OK;
  if (t2 != 16 || t3 * es != 2) return IREE_B200_STATUS_OK;
  const bool ragged = t0 * 16 != rows || t1 * t3 != cols;
  const uint64_t pad_mask = es == 1 ? 0xffull : 0xffffull;
  if (ragged && (padding & pad_mask)) return IREE_B200_STATUS_OK;  // the TMA unit fills with zero
  if (t0 * 16 < rows || t1 * t3 < cols || rm_stride0 < cols || t_stride0 < t1 * 16 * t3) return IREE_B200_STATUS_OK;
  const int64_t in_pitch = rm_stride0 * es, out_pitch = t_stride0 * es, row_bytes = cols * es;
  if ((in_pitch & 15) || (out_pitch & 15) || !fits_i32(in_pitch) || !fits_i32(out_pitch) || !fits_i32(row_bytes) ||
      ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15))
    return IREE_B200_STATUS_OK;
  const int ctas = 2 * usable_sms(ctx);
  if (ctas > kTilingScratchSlots) return IREE_B200_STATUS_OK;
  B200_RETURN_IF_ERROR(ensure_tiling_scratch(ctx));
  const int32_t ord = iree_hal_b200_executable_lookup(ctx->executable, "b200_pack_lhs_16x2b");
  if (ord < 0) return fail(IREE_B200_STATUS_NOT_FOUND, "export b200_pack_lhs_16x2b missing from the executable");
  const int64_t regions = ((t0 + 7) / 8) * ((t1 + 63) / 64);
  uint8_t* scratch = static_cast<uint8_t*>(ctx->tiling_scratch);
  iree_hal_b200_descriptor_set_binding_t bindings[4] = {
      {0, const_cast<void*>(in)}, {1, out}, {2, scratch}, {3, scratch + kTilingStatusOffset}};
  const int32_t c[6] = {(int32_t)rows, (int32_t)row_bytes, (int32_t)in_pitch, (int32_t)t0, (int32_t)t1, (int32_t)out_pitch};
  auto* cb = ctx->command_buffer;
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 4, bindings));
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, c, sizeof c));
  *dispatched = true;
  return dispatch_self_ordering(ctx, ord, 4, 6, static_cast<uint32_t>(regions < ctas ? regions : ctas));
}

// pack / unpack as a pure TMA copy (tiling_tma_sm100.cu), for the shapes it takes: tiles not transposed
// inside, tile rows of whole 16-byte pieces, a matrix the tiles cover exactly, 16-byte aligned addresses
// and pitches, no accumulation. Everything else goes to the staging kernels.
constexpr uint32_t kTilingNoTma = IREE_B200_UK_FLAG_PACK_NO_TMA;  // take the staging kernel whatever the shape
iree_b200_status_t tiling_by_tma(iree_b200_context_t* ctx, bool pack, int es, const void* in, void* out, int64_t rm_size0,
                                 int64_t rm_size1, int64_t rm_stride0, int64_t rm_stride1, int64_t t0, int64_t t1,
                                 int64_t t2, int64_t t3, int64_t t_stride0, uint32_t kernel_flags, bool* dispatched) {
  *dispatched = false;
  bool ti = kernel_flags & kUkTransposeInner;
  const bool to = kernel_flags & kUkTransposeOuter;
  if (ti && t3 == 1) {  // a transposed tile one row high is that row: [t2][1] in memory = [1][t2] not transposed
    t3 = t2;
    t2 = 1;
    ti = false;
  }
  if (ti || (kernel_flags & (kTilingAccumulateI32 | kTilingAccumulateF32)) || rm_stride1 != 1) return IREE_B200_STATUS_OK;
  const int64_t outer0 = to ? t1 : t0, outer1 = to ? t0 : t1;  // tiles along matrix rows / columns
  if (outer0 * t2 != rm_size0 || outer1 * t3 != rm_size1) return IREE_B200_STATUS_OK;
  if ((t3 * es) % 16 || t3 > 256 || t2 > 256 || t2 * t3 * es > 16384) return IREE_B200_STATUS_OK;
  if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) return IREE_B200_STATUS_OK;
  // Pitches in bytes of (tile row, o1 step, o0 step) on both sides.
  const uint64_t tiled[3] = {static_cast<uint64_t>(t3) * es, static_cast<uint64_t>(t2) * t3 * es,
                             static_cast<uint64_t>(t_stride0) * es};
  const uint64_t row_pitch = static_cast<uint64_t>(rm_stride0) * es;
  const uint64_t along_rows = static_cast<uint64_t>(t2) * row_pitch, along_cols = static_cast<uint64_t>(t3) * es;
  const uint64_t matrix[3] = {row_pitch, to ? along_rows : along_cols, to ? along_cols : along_rows};
  for (int i = 0; i < 3; ++i)
    if ((tiled[i] & 15) || (matrix[i] & 15) || !tiled[i] || !matrix[i] || tiled[i] >= (1ull << 40) || matrix[i] >= (1ull << 40))
      return IREE_B200_STATUS_OK;
  const int sms = usable_sms(ctx);
  B200_RETURN_IF_ERROR(ensure_tiling_scratch(ctx));
  if (sms > kTilingScratchSlots) return IREE_B200_STATUS_OK;
  // tiles per box: as many as fit 16 KiB, at most 256 and at most what one o0 index holds
  int64_t box2 = 16384 / (t2 * t3 * es);
  if (box2 > 256) box2 = 256;
  if (box2 > t1) box2 = t1;
  const int64_t regions = ((t1 + box2 - 1) / box2) * t0;
  const int32_t ord = iree_hal_b200_executable_lookup(ctx->executable, "b200_tiling_tma");
  if (ord < 0) return fail(IREE_B200_STATUS_NOT_FOUND, "export b200_tiling_tma missing from the executable");
  const uint64_t* sp = pack ? matrix : tiled;
  const uint64_t* dp = pack ? tiled : matrix;
  uint8_t* scratch = static_cast<uint8_t*>(ctx->tiling_scratch);
  iree_hal_b200_descriptor_set_binding_t bindings[4] = {
      {0, const_cast<void*>(in)}, {1, out}, {2, scratch + 128 * (es == 1 ? 0 : es == 2 ? 1 : 2)}, {3, scratch + kTilingStatusOffset}};
  const int32_t c[18] = {(int32_t)t3, (int32_t)t2, (int32_t)t1, (int32_t)t0, (int32_t)box2, es,
                         (int32_t)(uint32_t)sp[0], (int32_t)(sp[0] >> 32), (int32_t)(uint32_t)sp[1], (int32_t)(sp[1] >> 32),
                         (int32_t)(uint32_t)sp[2], (int32_t)(sp[2] >> 32), (int32_t)(uint32_t)dp[0], (int32_t)(dp[0] >> 32),
                         (int32_t)(uint32_t)dp[1], (int32_t)(dp[1] >> 32), (int32_t)(uint32_t)dp[2], (int32_t)(dp[2] >> 32)};
  auto* cb = ctx->command_buffer;
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 4, bindings));
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, c, sizeof c));
  *dispatched = true;
  return dispatch_self_ordering(ctx, ord, 4, 18, static_cast<uint32_t>(regions < sms ? regions : sms));
}

// Shared by pack (row-major -> tiled) and unpack; `rm_*` describe the row-major side.
iree_b200_status_t tiling_dispatch(iree_b200_context_t* ctx, bool pack, int es, const void* in, void* out,
                                   int64_t rm_size0, int64_t rm_size1, int64_t rm_stride0, int64_t rm_stride1,
                                   int64_t t0, int64_t t1, int64_t t2, int64_t t3, int64_t t_stride0,
                                   uint32_t kernel_flags, uint64_t padding) {
  if (!fits_i32(rm_size0) || !fits_i32(rm_size1) || !fits_i32(rm_stride0) || !fits_i32(rm_stride1) || !fits_i32(t0) ||
      !fits_i32(t1) || !fits_i32(t2) || !fits_i32(t3) || !fits_i32(t_stride0))
    return fail(IREE_B200_STATUS_OUT_OF_RANGE, "sizes and strides must be non-negative 32-bit values");
  if (t0 == 0 || t1 == 0 || t2 == 0 || t3 == 0) return IREE_B200_STATUS_OK;  // early return, pack.c:106-109
  const bool ti = kernel_flags & kUkTransposeInner, to = kernel_flags & kUkTransposeOuter;
  const int64_t tile0 = ti ? t3 : t2, tile1 = ti ? t2 : t3, outer0 = to ? t1 : t0, outer1 = to ? t0 : t1;
  if (outer0 * tile0 < rm_size0 || outer1 * tile1 < rm_size1)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "the tiled shape does not cover the %lldx%lld matrix",
                static_cast<long long>(rm_size0), static_cast<long long>(rm_size1));
  if (!in || !out) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "buffer pointer is NULL");
  if (!(kernel_flags & kTilingNoTma)) {
    bool dispatched = false;
    if (pack && es == 1) {
      B200_RETURN_IF_ERROR(pack_rhs_16x2(ctx, in, out, rm_size0, rm_size1, rm_stride0, rm_stride1, t0, t1, t2, t3, t_stride0,
                                         kernel_flags, padding, &dispatched));
      if (dispatched) return IREE_B200_STATUS_OK;
    }
    if (pack && es <= 2) {
      B200_RETURN_IF_ERROR(pack_lhs_16x2b(ctx, es, in, out, rm_size0, rm_size1, rm_stride0, rm_stride1, t0, t1, t2, t3,
                                          t_stride0, kernel_flags, padding, &dispatched));
      if (dispatched) return IREE_B200_STATUS_OK;
    }
    B200_RETURN_IF_ERROR(tiling_by_tma(ctx, pack, es, in, out, rm_size0, rm_size1, rm_stride0, rm_stride1, t0, t1, t2, t3,
                                       t_stride0, kernel_flags, &dispatched));
    if (dispatched) return IREE_B200_STATUS_OK;
  }
  kernel_flags &= ~kTilingNoTma;
  const char* name = pack ? (es == 1 ? "b200_pack_b8" : es == 2 ? "b200_pack_b16" : "b200_pack_b32")
                          : (es == 1 ? "b200_unpack_b8" : es == 2 ? "b200_unpack_b16" : "b200_unpack_b32");
  const int32_t ord = iree_hal_b200_executable_lookup(ctx->executable, name);
  if (ord < 0) return fail(IREE_B200_STATUS_NOT_FOUND, "export %s missing from the executable", name);
  const int sms = usable_sms(ctx);
  const uint32_t grid = tiling_grid(t0, t1, t2, t3, kernel_flags, es, sms);
  auto* cb = ctx->command_buffer;
  iree_hal_b200_descriptor_set_binding_t bindings[2] = {{0, const_cast<void*>(in)}, {1, out}};
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 2, bindings));
  if (pack) {
    const int32_t c[13] = {(int32_t)rm_size0, (int32_t)rm_size1, (int32_t)rm_stride0, (int32_t)rm_stride1,
                           (int32_t)t0,       (int32_t)t1,       (int32_t)t2,         (int32_t)t3,
                           (int32_t)t_stride0, (int32_t)kernel_flags, (int32_t)(uint32_t)padding, 0, 0};
    B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, c, sizeof c));
    return iree_hal_b200_command_buffer_dispatch(cb, ctx->executable, ord, 2, 13, grid, 1, 1);
  }
  const int32_t c[12] = {(int32_t)t0,       (int32_t)t1,         (int32_t)t2,         (int32_t)t3, (int32_t)t_stride0,
                         (int32_t)rm_size0, (int32_t)rm_size1,   (int32_t)rm_stride0, (int32_t)rm_stride1,
                         (int32_t)kernel_flags, 0, 0};
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, c, sizeof c));
  return iree_hal_b200_command_buffer_dispatch(cb, ctx->executable, ord, 2, 12, grid, 1, 1);
}

struct Mmt4dTypes {
  int kind, epilogue, elem_bytes, out_bytes;
};
bool mmt4d_types(uint32_t flags, Mmt4dTypes* t) {
  switch (flags & IREE_B200_UK_FLAG_MMT4D_TYPE_MASK) {
    case IREE_B200_UK_FLAG_MMT4D_TYPE_S8S8S32: *t = {IREE_B200_KIND_I8, IREE_B200_EPILOGUE_ACCUMULATOR, 1, 4}; return true;
    case IREE_B200_UK_FLAG_MMT4D_TYPE_F16F16F32: *t = {IREE_B200_KIND_F16, IREE_B200_EPILOGUE_ACCUMULATOR, 2, 4}; return true;
    case IREE_B200_UK_FLAG_MMT4D_TYPE_BF16BF16F32: *t = {IREE_B200_KIND_BF16, IREE_B200_EPILOGUE_ACCUMULATOR, 2, 4}; return true;
    case IREE_B200_UK_FLAG_MMT4D_TYPE_F16F16F16: *t = {IREE_B200_KIND_F16, IREE_B200_EPILOGUE_CAST, 2, 2}; return true;
    case IREE_B200_UK_FLAG_MMT4D_TYPE_BF16BF16BF16: *t = {IREE_B200_KIND_BF16, IREE_B200_EPILOGUE_CAST, 2, 2}; return true;
    default: return false;
  }
}
size_t up256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

}  // namespace

extern "C" {

iree_b200_status_t iree_b200_uk_status(iree_b200_context_t* context) {
  if (!context) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "context is NULL");
  if (!context->tiling_scratch) return IREE_B200_STATUS_OK;  // no TMA pack / unpack was ever dispatched
  uint32_t status = 0;
  uint8_t* word = static_cast<uint8_t*>(context->tiling_scratch) + kTilingStatusOffset;
  B200_RETURN_IF_ERROR(iree_hal_b200_transfer_d2h(context->device, word, &status, sizeof status));
  B200_RETURN_IF_ERROR(iree_hal_b200_device_synchronize(context->device));
  if (status == 0) return IREE_B200_STATUS_OK;
  B200_RETURN_IF_ERROR(iree_hal_b200_fill_buffer(context->device, word, 4, 0));
  if (status == 5) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "a pack / unpack kernel rejected its arguments (shape / alignment)");
  return fail(IREE_B200_STATUS_DEADLINE_EXCEEDED, "a pack / unpack kernel gave up waiting for one of its copies (wait id %u)", status);
}

iree_b200_status_t iree_b200_uk_pack(iree_b200_context_t* context, const void* in_buffer, int64_t in_offset,
                                     int64_t in_stride0, int64_t in_stride1, void* out_buffer, int64_t out_offset,
                                     int64_t out_stride0, int64_t out_stride1, int64_t in_size0, int64_t in_size1,
                                     int64_t out_size0, int64_t out_size1, int64_t out_size2, int64_t out_size3,
                                     uint64_t padding_value, uint32_t flags) {
  if (!context) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "context is NULL");
  const int es = pack_elem_bytes(flags);
  if (!es) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "unknown pack type 0x%x", flags & 0xFF);
  if (flags & ~(IREE_B200_UK_FLAG_PACK_TYPE_MASK | kUkTransposeInner | kUkTransposeOuter | IREE_B200_UK_FLAG_PACK_NO_TMA))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "unknown pack flags 0x%x", flags);
  if (out_stride1 != out_size2 * out_size3)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "out_stride1 must equal out_size2 * out_size3");
  return tiling_dispatch(context, true, es, static_cast<const uint8_t*>(in_buffer) + in_offset * es,
                         static_cast<uint8_t*>(out_buffer) + out_offset * es, in_size0, in_size1, in_stride0, in_stride1,
                         out_size0, out_size1, out_size2, out_size3, out_stride0,
                         flags & (kUkTransposeInner | kUkTransposeOuter | kTilingNoTma), padding_value);
}

iree_b200_status_t iree_b200_uk_unpack(iree_b200_context_t* context, const void* in_buffer, int64_t in_offset,
                                       int64_t in_stride0, int64_t in_stride1, void* out_buffer, int64_t out_offset,
                                       int64_t out_stride0, int64_t out_stride1, int64_t in_size0, int64_t in_size1,
                                       int64_t in_size2, int64_t in_size3, int64_t out_size0, int64_t out_size1,
                                       uint32_t flags) {
  if (!context) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "context is NULL");
  const int es = pack_elem_bytes(flags);
  if (!es) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "unknown unpack type 0x%x", flags & 0xFF);
  if (flags & ~(IREE_B200_UK_FLAG_PACK_TYPE_MASK | kUkTransposeInner | kUkTransposeOuter | IREE_B200_UK_FLAG_PACK_NO_TMA))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "unknown unpack flags 0x%x", flags);
  if (in_stride1 != in_size2 * in_size3)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "in_stride1 must equal in_size2 * in_size3");
  return tiling_dispatch(context, false, es, static_cast<const uint8_t*>(in_buffer) + in_offset * es,
                         static_cast<uint8_t*>(out_buffer) + out_offset * es, out_size0, out_size1, out_stride0,
                         out_stride1, in_size0, in_size1, in_size2, in_size3, in_stride0,
                         flags & (kUkTransposeInner | kUkTransposeOuter | kTilingNoTma), 0);
}

// The element types without a tensor-core kernel (f32f32f32, s16s16s32, s16u4s32, s16s8s32, s8s4s32):
// one thread per output element, the reference's generic reduction order (mmt4d_generic_sm100.cu).
// Offsets and strides are in elements of each operand's type; a 4-bit element is half a byte
// (mmt4d.c:67-86).
static iree_b200_status_t mmt4d_other_types(iree_b200_context_t* context, const void* lhs_buffer, int64_t lhs_offset,
                                            int64_t lhs_stride0, const void* rhs_buffer, int64_t rhs_offset,
                                            int64_t rhs_stride0, void* out_buffer, int64_t out_offset, int64_t out_stride0,
                                            int64_t M, int64_t N, int64_t K, int32_t M0, int32_t N0, int32_t K0,
                                            uint32_t flags) {
  const uint32_t type = flags & IREE_B200_UK_FLAG_MMT4D_TYPE_MASK;
  int lhs_bits, rhs_bits;
  switch (type) {
    case 0x01: lhs_bits = 32, rhs_bits = 32; break;  // F32F32F32
    case 0x07: lhs_bits = 16, rhs_bits = 16; break;  // S16S16S32
    case 0x08: lhs_bits = 16, rhs_bits = 4; break;   // S16U4S32
    case 0x09: lhs_bits = 16, rhs_bits = 8; break;   // S16S8S32
    case 0x0A: lhs_bits = 8, rhs_bits = 4; break;    // S8S4S32
    default: return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "unknown mmt4d type 0x%x", type);
  }
  if (flags & ~(IREE_B200_UK_FLAG_MMT4D_TYPE_MASK | IREE_B200_UK_FLAG_MMT4D_ACCUMULATE | 0x200u | 0x400u |
                IREE_B200_UK_FLAG_MMT4D_UNTILE))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "unknown mmt4d flags 0x%x", flags);
  const bool accumulate = flags & IREE_B200_UK_FLAG_MMT4D_ACCUMULATE;
  if (M < 0 || N < 0 || K < 0 || M0 < 0 || N0 < 0 || K0 < 0) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "negative dimension");
  if (M == 0 || N == 0 || M0 == 0 || N0 == 0) return IREE_B200_STATUS_OK;  // nothing to write
  if (K == 0 && accumulate) return IREE_B200_STATUS_OK;
  if (rhs_bits == 4 && ((K0 & 1) || (rhs_offset & 1) || (rhs_stride0 & 1)))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "4-bit right-hand sides need an even K0, offset and stride");
  if (!lhs_buffer || !rhs_buffer || !out_buffer) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "buffer pointer is NULL");
  const int64_t lhs_pitch = lhs_stride0 * lhs_bits / 8, rhs_pitch = rhs_stride0 * rhs_bits / 8;
  if (!fits_i32(M) || !fits_i32(N) || !fits_i32(K) || !fits_i32(lhs_pitch) || !fits_i32(rhs_pitch) || !fits_i32(out_stride0))
    return fail(IREE_B200_STATUS_OUT_OF_RANGE, "dimension or pitch above 2^31");
  const uint8_t* lhs = static_cast<const uint8_t*>(lhs_buffer) + lhs_offset * lhs_bits / 8;
  const uint8_t* rhs = static_cast<const uint8_t*>(rhs_buffer) + rhs_offset * rhs_bits / 8;
  uint8_t* out = static_cast<uint8_t*>(out_buffer) + out_offset * 4;
  const int32_t ord = iree_hal_b200_executable_lookup(context->executable, "b200_mmt4d_generic");
  if (ord < 0) return fail(IREE_B200_STATUS_NOT_FOUND, "export b200_mmt4d_generic missing from the executable");
  const int64_t total = M * N * M0 * N0;
  const int64_t cap = static_cast<int64_t>(usable_sms(context)) * 16;
  const int64_t blocks = (total + 255) / 256;
  iree_hal_b200_descriptor_set_binding_t bindings[3] = {{0, const_cast<uint8_t*>(lhs)}, {1, const_cast<uint8_t*>(rhs)}, {2, out}};
  const int32_t c[11] = {(int32_t)M, (int32_t)N, (int32_t)K, M0, N0, K0, (int32_t)lhs_pitch, (int32_t)rhs_pitch,
                         (int32_t)out_stride0, (int32_t)type, accumulate ? 1 : 0};
  auto* cb = context->command_buffer;
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 3, bindings));
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, c, sizeof c));
  return iree_hal_b200_command_buffer_dispatch(cb, context->executable, ord, 3, 11, static_cast<uint32_t>(blocks < cap ? blocks : cap), 1, 1);
}

size_t iree_b200_uk_mmt4d_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t M0, int32_t N0, int32_t K0,
                                          uint32_t flags) {
  Mmt4dTypes t;
  if (!mmt4d_types(flags, &t) || M < 0 || N < 0 || K < 0 || M0 < 0 || N0 < 0 || K0 < 0) return 0;
  const size_t m = static_cast<size_t>(M) * M0, n = static_cast<size_t>(N) * N0, k = static_cast<size_t>(K) * K0;
  return up256(IREE_B200_WORKSPACE_BYTES) + up256(m * k * t.elem_bytes) + up256(n * k * t.elem_bytes) +
         up256(m * n * t.out_bytes);
}

// The kernel that multiplies tiled operands as they are (mmt4d_sm100.cu) takes tiles whose rows are 32
// bytes in both operands (i8 16x16x2, f16 / bf16 16x16x1) at 16-byte aligned addresses and pitches and
// 32-byte aligned results. True when it was dispatched; other shapes go through the un-tiling path.
static iree_b200_status_t mmt4d_direct(iree_b200_context_t* context, const Mmt4dTypes& t, const uint8_t* lhs,
                                       int64_t lhs_stride0, const uint8_t* rhs, int64_t rhs_stride0, uint8_t* out,
                                       int64_t out_stride0, int64_t M1, int64_t N1, int64_t K1, int32_t M0, int32_t N0,
                                       int32_t K0, bool accumulate, void* workspace, bool* dispatched) {
  *dispatched = false;
  const int es = t.elem_bytes;
  if (M0 != 16 || N0 != 16 || K0 != (es == 1 ? 2 : 1) || K1 <= 0) return IREE_B200_STATUS_OK;
  if ((reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs)) & 15) return IREE_B200_STATUS_OK;
  if (reinterpret_cast<uintptr_t>(out) & 31) return IREE_B200_STATUS_OK;
  if ((lhs_stride0 * es) % 16 || (rhs_stride0 * es) % 16 || (out_stride0 * t.out_bytes) % 32) return IREE_B200_STATUS_OK;
  if (lhs_stride0 <= 0 || rhs_stride0 <= 0 || !fits_i32(lhs_stride0) || !fits_i32(rhs_stride0) || !fits_i32(out_stride0))
    return IREE_B200_STATUS_OK;
  const int sms = usable_sms(context);
  const int run = 32 / es;                      // elements of one tile row; the product's row / column unit
  const int64_t rows = M1 * run, cols = N1 * run;  // extents of the product the tensor core computes
  const int64_t tiles_m = (rows + 127) / 128;
  int bn = 0;
  double best = 0;
  for (int w = 256; w >= 32; w -= 32) {
    const int64_t tiles = tiles_m * ((cols + w - 1) / w);
    const double cost = static_cast<double>((tiles + sms - 1) / sms) * (400.0 + w);  // the GEMM kernels' wave model
    if (!bn || cost < best * 0.9999) bn = w, best = cost;
  }
  const int64_t tiles = tiles_m * ((cols + bn - 1) / bn);
  const uint32_t grid = static_cast<uint32_t>(tiles < sms ? tiles : sms);
  const char* name = t.kind == IREE_B200_KIND_I8
                         ? "b200_mmt4d_s8s8s32"
                         : t.kind == IREE_B200_KIND_F16 ? (t.out_bytes == 4 ? "b200_mmt4d_f16f16f32" : "b200_mmt4d_f16f16f16")
                                                        : (t.out_bytes == 4 ? "b200_mmt4d_bf16bf16f32" : "b200_mmt4d_bf16bf16bf16");
  const int32_t ord = iree_hal_b200_executable_lookup(context->executable, name);
  if (ord < 0) return fail(IREE_B200_STATUS_NOT_FOUND, "export %s missing from the executable", name);
  iree_hal_b200_descriptor_set_binding_t bindings[4] = {
      {0, const_cast<uint8_t*>(lhs)}, {1, const_cast<uint8_t*>(rhs)}, {2, out}, {3, workspace}};
  const int32_t constants[7] = {(int32_t)M1,          (int32_t)N1,          (int32_t)K1, (int32_t)lhs_stride0,
                                (int32_t)rhs_stride0, (int32_t)out_stride0, bn | (accumulate ? 1 << 16 : 0)};
  auto* cb = context->command_buffer;
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_descriptor_set(cb, 0, 4, bindings));
  B200_RETURN_IF_ERROR(iree_hal_b200_command_buffer_push_constants(cb, 0, constants, sizeof constants));
  *dispatched = true;
  return dispatch_self_ordering(context, ord, 4, 7, grid);
}

iree_b200_status_t iree_b200_uk_mmt4d(iree_b200_context_t* context, const void* lhs_buffer, int64_t lhs_offset,
                                      int64_t lhs_stride0, const void* rhs_buffer, int64_t rhs_offset,
                                      int64_t rhs_stride0, void* out_buffer, int64_t out_offset, int64_t out_stride0,
                                      int64_t M, int64_t N, int64_t K, int32_t M0, int32_t N0, int32_t K0,
                                      uint32_t flags, void* workspace) {
  if (!context) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "context is NULL");
  Mmt4dTypes t;
  if (!mmt4d_types(flags, &t))
    return mmt4d_other_types(context, lhs_buffer, lhs_offset, lhs_stride0, rhs_buffer, rhs_offset, rhs_stride0, out_buffer,
                             out_offset, out_stride0, M, N, K, M0, N0, K0, flags);
  if (flags & ~(IREE_B200_UK_FLAG_MMT4D_TYPE_MASK | IREE_B200_UK_FLAG_MMT4D_ACCUMULATE | 0x200u | 0x400u |
                IREE_B200_UK_FLAG_MMT4D_UNTILE))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "unknown mmt4d flags 0x%x", flags);
  const bool accumulate = flags & IREE_B200_UK_FLAG_MMT4D_ACCUMULATE;
  if (accumulate && t.out_bytes != 4)
    return fail(IREE_B200_STATUS_UNIMPLEMENTED, "ACCUMULATE needs a 32-bit output type");
  if (M < 0 || N < 0 || K < 0 || M0 < 0 || N0 < 0 || K0 < 0)
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "negative dimension");
  const int64_t m = M * M0, n = N * N0, k = K * K0;
  if (!fits_i32(m) || !fits_i32(n) || !fits_i32(k)) return fail(IREE_B200_STATUS_OUT_OF_RANGE, "dimension above 2^31");
  if (m == 0 || n == 0) return IREE_B200_STATUS_OK;  // mmt4d.c early return: nothing to write
  if (k == 0 && accumulate) return IREE_B200_STATUS_OK;
  if (!lhs_buffer || !rhs_buffer || !out_buffer) return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "buffer pointer is NULL");
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) % 256))
    return fail(IREE_B200_STATUS_INVALID_ARGUMENT, "workspace must be a 256-byte aligned device buffer");
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint8_t* lhs_rm = ws + up256(IREE_B200_WORKSPACE_BYTES);
  uint8_t* rhs_rm = lhs_rm + up256(static_cast<size_t>(m) * k * t.elem_bytes);
  uint8_t* acc_rm = rhs_rm + up256(static_cast<size_t>(n) * k * t.elem_bytes);
  const uint8_t* lhs = static_cast<const uint8_t*>(lhs_buffer) + lhs_offset * t.elem_bytes;
  const uint8_t* rhs = static_cast<const uint8_t*>(rhs_buffer) + rhs_offset * t.elem_bytes;
  uint8_t* out = static_cast<uint8_t*>(out_buffer) + out_offset * t.out_bytes;
  if (!(flags & IREE_B200_UK_FLAG_MMT4D_UNTILE)) {
    bool dispatched = false;
    B200_RETURN_IF_ERROR(mmt4d_direct(context, t, lhs, lhs_stride0, rhs, rhs_stride0, out, out_stride0, M, N, K, M0, N0, K0,
                                      accumulate, workspace, &dispatched));
    if (dispatched) return IREE_B200_STATUS_OK;
  }
  if (k > 0) {
    B200_RETURN_IF_ERROR(tiling_dispatch(context, false, t.elem_bytes, lhs, lhs_rm, m, k, k, 1, M, K, M0, K0, lhs_stride0, 0, 0));
    B200_RETURN_IF_ERROR(tiling_dispatch(context, false, t.elem_bytes, rhs, rhs_rm, n, k, k, 1, N, K, N0, K0, rhs_stride0, 0, 0));
  }
  iree_b200_matmul_params_t p = {t.kind, t.epilogue, (int32_t)m, (int32_t)n, (int32_t)k, 1, IREE_B200_RHS_NK, 0, 0};
  B200_RETURN_IF_ERROR(iree_b200_matmul(context, &p, lhs_rm, rhs_rm, acc_rm, nullptr, nullptr, ws));
  uint32_t kf = 0;
  if (accumulate) kf = t.kind == IREE_B200_KIND_I8 ? kTilingAccumulateI32 : kTilingAccumulateF32;
  return tiling_dispatch(context, true, t.out_bytes, acc_rm, out, m, n, n, 1, M, N, M0, N0, out_stride0, kf, 0);
}

}  // extern "C"
