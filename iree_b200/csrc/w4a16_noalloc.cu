// iree_b200_w4a16_decode_noalloc: the W4A16 decode dispatch for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they run a dispatch: code
// running inside a CUDA stream capture (allocation is not a capturable operation), a serving
// loop that has handed every byte of device memory to its own pool, or a real-time path that is
// not allowed to take the driver's allocation lock. The regular entry point needs a
// caller-provided workspace for the scratch of K > 4096; this one brings its own, a fixed array
// that lives in the library's device image, so the caller passes nothing but inputs and outputs.
//
// The scratch is a file-scope `static __device__` array. In host code that name is only a
// handle for the symbol, not a device address, so the address is looked up once per device with
// cudaGetSymbolAddress while that device is current, and the looked-up pointer is what the
// kernel receives.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "../../include/iree_b200.h"
#include "hal_b200_internal.h"
#include "w4a16_decode.cuh"

namespace {

// f32 partial sums [16][N] (+ one spare word per 16-row tile), for N up to the stated maximum.
constexpr int kMaxN = IREE_B200_NOALLOC_MAX_N;
constexpr size_t kScratchBytes = static_cast<size_t>(16) * kMaxN * 4 + static_cast<size_t>(kMaxN / 16) * 4;

static __device__ __align__(256) unsigned char g_decode_scratch[kScratchBytes];

template <int MH>
__global__ void __launch_bounds__(b200::kDecodeThreads, 1)
    decode_noalloc_kernel(const __half* a, const uint8_t* wq, const __half* scales, __half* out, float* scratch, int M,
                          int N, int K, int ldo, int n_off) {
  b200::decode_body<MH>(a, wq, scales, out, scratch, M, N, K, ldo, n_off);
}

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {nullptr};
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
  if (N > kMaxN) {
    char msg[256];
    snprintf(msg, sizeof msg, "N = %d exceeds the built-in scratch of the no-allocation entry point (at most %d columns)",
             N, kMaxN);
    return iree_b200_internal_set_error(IREE_B200_STATUS_OUT_OF_RANGE, msg);
  }
  if (ldo < n_offset + N || n_offset < 0)
    return iree_b200_internal_set_error(IREE_B200_STATUS_INVALID_ARGUMENT, "output pitch cannot hold the result columns");

  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (device < 0 || device >= kMaxDevices)
    return iree_b200_internal_set_error(IREE_B200_STATUS_OUT_OF_RANGE, "device ordinal out of range");
  void* scratch = nullptr;
  int sms = 0;
  {
    // Set-up, once per device, with that device current: resolve the symbol to a device address.
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ptr[device]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_decode_scratch);
      if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(scratch)");
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
      g_scratch_ptr[device] = p;
    }
    scratch = g_scratch_ptr[device];
    sms = g_sm_count[device];
  }

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int ksplit = 1;  // K beyond 4096 is covered by passes inside the kernel
  if (K > 4096) {
    // Every call shares the array and it keeps what the last call left there. The kernel zeroes
    // what it used, but a call that was cut short would not have, so the part this call will
    // use is cleared first: the partial sums [16][N] and the spare words that follow them.
    const size_t used = static_cast<size_t>(16) * N * 4 + static_cast<size_t>(N / 16) * 4;
    e = cudaMemsetAsync(scratch, 0, used, s);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(scratch)");
  }
  const int tiles = N / 16;
  int gx = sms / ksplit;
  if (gx < 1) gx = 1;
  if (gx > tiles) gx = tiles;
  const dim3 grid(gx, ksplit, 1), block(b200::kDecodeThreads, 1, 1);
  if (M <= 8) {
    decode_noalloc_kernel<1><<<grid, block, b200::decode_smem_bytes(1), s>>>(static_cast<const __half*>(a), static_cast<const uint8_t*>(wq),
                                                    static_cast<const __half*>(scales), static_cast<__half*>(out),
                                                    static_cast<float*>(scratch), M, N, K, ldo, n_offset);
  } else {
    decode_noalloc_kernel<2><<<grid, block, b200::decode_smem_bytes(2), s>>>(static_cast<const __half*>(a), static_cast<const uint8_t*>(wq),
                                                    static_cast<const __half*>(scales), static_cast<__half*>(out),
                                                    static_cast<float*>(scratch), M, N, K, ldo, n_offset);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "decode kernel launch");
  return IREE_B200_STATUS_OK;
}
