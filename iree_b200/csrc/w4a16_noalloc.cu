// iree_b200_w4a16_decode_noalloc: the W4A16 decode dispatch for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they run a dispatch: code
// running inside a CUDA stream capture (allocation is not a capturable operation), a serving
// loop that has handed every byte of device memory to its own pool, or a real-time path that is
// not allowed to take the driver's allocation lock. The regular entry point needs a
// caller-provided workspace for the scratch of K > 4096 (tile counters and f32 partial tiles of
// the K slices); this one brings its own, a fixed array that lives in the library's device
// image, so the caller passes nothing but inputs and outputs.
//
// The scratch is a file-scope `static __device__` array. In host code that name is only a
// handle for the symbol, not a device address, so the address is looked up once per device with
// cudaGetSymbolAddress while that device is current, and the looked-up pointer is what the
// kernel receives.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "../../include/iree_b200.h"
#include "hal_b200_internal.h"
#include "w4a16_decode.cuh"

namespace {

// Tile counters and one f32 partial tile per 16-row tile and K slice (b200::DecodeScratchLayout),
// for N up to the stated maximum at two slices (K <= 8192), or half / a quarter of it at three /
// four slices: N * slices <= 2 * kMaxN.
constexpr int kMaxN = IREE_B200_NOALLOC_MAX_N;
constexpr int kMaxSliceColumns = 2 * kMaxN;
constexpr size_t kScratchBytes = b200::DecodeScratchLayout::bytes(kMaxN, 2);

static __device__ __align__(256) unsigned char g_decode_scratch[kScratchBytes];
// What a kernel leaves here when one of its bounded waits ran out: [0] which wait, [1] tile, [2] N.
static __device__ __align__(16) uint32_t g_decode_status[4];

// The tensor map over the weights (used when K spans several slices) travels as a kernel parameter:
// it is encoded on the host for every call, which needs no device memory.
struct alignas(64) WeightMap {
  unsigned char bytes[128];
};

template <int MH>
__global__ void __launch_bounds__(b200::kDecodeThreads, 1)
    decode_noalloc_kernel(const __grid_constant__ WeightMap wmap, const __half* a, const uint8_t* wq, const __half* scales,
                          __half* out, void* scratch, uint32_t* status, int M, int N, int K, int ldo, int n_off) {
  b200::decode_body<MH>(a, wq, scales, out, scratch, status, &wmap, false, M, N, K, ldo, n_off);
}

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {nullptr};
void* g_status_ptr[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};

int32_t cuda_fail(cudaError_t e, const char* what) {
  char msg[512];
  snprintf(msg, sizeof msg, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  return iree_b200_internal_set_error(IREE_B200_STATUS_INTERNAL, msg);
}

}  // namespace

extern "C" iree_b200_status_t iree_b200_w4a16_decode_noalloc(const void* a, const void* wq, const void* scales,
                                                             void* out, int32_t M, int32_t N, int32_t K, int32_t ldo,
                                                             int32_t n_offset, void* stream) {
  if (!a || !wq || !scales || !out)
    return iree_b200_internal_set_error(IREE_B200_STATUS_INVALID_ARGUMENT, "operand pointer is NULL");
  if (M < 1 || M > 16 || N < 16 || (N % 16) || K < 256 || (K % 256) || K > 16384) {
    return iree_b200_internal_set_error(IREE_B200_STATUS_INVALID_ARGUMENT,
                                        "the no-allocation decode entry point needs 1 <= M <= 16, N a positive "
                                        "multiple of 16 and K a multiple of 256 up to 16384 (group size 128)");
  }
  const int slices = (K + b200::kDecodeSliceK - 1) / b200::kDecodeSliceK;
  if (N > kMaxN || static_cast<int64_t>(N) * slices > kMaxSliceColumns) {
    char msg[320];
    snprintf(msg, sizeof msg,
             "N = %d with K = %d exceeds the built-in scratch of the no-allocation entry point (at most %d columns, "
             "and at most %d columns x K slices of 4096)",
             N, K, kMaxN, kMaxSliceColumns);
    return iree_b200_internal_set_error(IREE_B200_STATUS_OUT_OF_RANGE, msg);
  }
  if (n_offset < 0 || static_cast<int64_t>(ldo) < static_cast<int64_t>(n_offset) + N)
    return iree_b200_internal_set_error(IREE_B200_STATUS_INVALID_ARGUMENT, "output pitch cannot hold the result columns");
  // The kernel reads activations with 16-byte loads and weights and scales with bulk copies; a base
  // that is not on a 16-byte boundary (say, a sub-allocation of the caller's pool at an odd offset)
  // would fault on the device, so it is refused here, before anything is launched.
  if ((reinterpret_cast<uintptr_t>(a) % 16) || (reinterpret_cast<uintptr_t>(wq) % 16) ||
      (reinterpret_cast<uintptr_t>(scales) % 16) || (reinterpret_cast<uintptr_t>(out) % 2))
    return iree_b200_internal_set_error(IREE_B200_STATUS_INVALID_ARGUMENT,
                                        "activations, weights and scales must start on 16-byte boundaries (the "
                                        "result on a 2-byte boundary)");

  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (device < 0 || device >= kMaxDevices)
    return iree_b200_internal_set_error(IREE_B200_STATUS_OUT_OF_RANGE, "device ordinal out of range");
  void* scratch = nullptr;
  uint32_t* status = nullptr;
  int sms = 0;
  {
    // Set-up, once per device, with that device current: resolve the symbol to a device address.
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ptr[device]) {
      void *p = nullptr, *ps = nullptr;
      e = cudaGetSymbolAddress(&p, g_decode_scratch);
      if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(scratch)");
      e = cudaGetSymbolAddress(&ps, g_decode_status);
      if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(status)");
      int n = 0;
      e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
      if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
      g_sm_count[device] = n > 0 ? n : 148;
      // Raising the dynamic shared-memory limit is a function attribute, not an allocation.
      e = cudaFuncSetAttribute(decode_noalloc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               b200::decode_smem_bytes(1));
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(decode_noalloc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 b200::decode_smem_bytes(2));
      if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
      g_status_ptr[device] = ps;
      g_scratch_ptr[device] = p;
    }
    scratch = g_scratch_ptr[device];
    status = static_cast<uint32_t*>(g_status_ptr[device]);
    sms = g_sm_count[device];
  }

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (slices > 1) {
    // Every call shares the array and it keeps what the last call left there. The kernel puts the
    // tile counters back to zero, but a call that was cut short would not have, so the counters
    // this call will use are cleared first (the partial tiles behind them need no initial value).
    e = cudaMemsetAsync(scratch, 0, b200::DecodeScratchLayout::counter_bytes(N), s);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(scratch)");
  }
  WeightMap wmap;
  memset(&wmap, 0, sizeof wmap);
  if (slices > 1) {
    const int32_t st = iree_b200_internal_encode_decode_weight_map(wq, N, K, wmap.bytes);
    if (st != IREE_B200_STATUS_OK) return st;
  }
  const int tiles = N / 16;
  int walkers = sms / slices;
  if (walkers < 1) walkers = 1;
  if (walkers > tiles) walkers = tiles;
  const dim3 grid(walkers * slices, 1, 1), block(b200::kDecodeThreads, 1, 1);
  if (M <= 8) {
    decode_noalloc_kernel<1><<<grid, block, b200::decode_smem_bytes(1), s>>>(
        wmap, static_cast<const __half*>(a), static_cast<const uint8_t*>(wq), static_cast<const __half*>(scales),
        static_cast<__half*>(out), scratch, status, M, N, K, ldo, n_offset);
  } else {
    decode_noalloc_kernel<2><<<grid, block, b200::decode_smem_bytes(2), s>>>(
        wmap, static_cast<const __half*>(a), static_cast<const uint8_t*>(wq), static_cast<const __half*>(scales),
        static_cast<__half*>(out), scratch, status, M, N, K, ldo, n_offset);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "decode kernel launch");
  return IREE_B200_STATUS_OK;
}

// Reads back (and clears) the status words the no-allocation kernels share on the current device.
// Synchronises the device's default stream path only through the copy itself: call it after the
// stream the dispatches ran on has been synchronised.
extern "C" iree_b200_status_t iree_b200_w4a16_decode_noalloc_status(void) {
  uint32_t words[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyFromSymbol(words, g_decode_status, sizeof words);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyFromSymbol(status)");
  if (words[0] == 0) return IREE_B200_STATUS_OK;
  const uint32_t zero[4] = {0, 0, 0, 0};
  e = cudaMemcpyToSymbol(g_decode_status, zero, sizeof zero);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyToSymbol(status)");
  char msg[160];
  snprintf(msg, sizeof msg, "a no-allocation decode dispatch gave up: wait %u ran out at tile %u", words[0], words[1]);
  return iree_b200_internal_set_error(IREE_B200_STATUS_DEADLINE_EXCEEDED, msg);
}
