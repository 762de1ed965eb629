// Geometry of b200_w4a16_decode_tc shared by the kernel and the host code that sizes and prepares
// its workspace.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace b200 {

constexpr int kTcWRows = 128;    // weight rows per tile = lanes of tensor memory (MMA M)
constexpr int kTcARows = 16;     // activation rows the kernel takes (MMA N)
constexpr int kTcUnitK = 512;    // K per unit of work = per stage of the weight ring
constexpr int kTcThreads = 768;
constexpr int kTcSmemBytes = 1024 + 5 * (kTcWRows * (kTcUnitK / 2) + kTcWRows * 8) + 3 * ((kTcUnitK / 64) * kTcARows * 128) + 512;
constexpr int kTcMaxCtas = 148;  // CTAs of one dispatch at most: each owns two partial-sum slots
constexpr uint32_t kTcNoteMagic = 0x54433431u;  // status words 16..18 of a prepared workspace: magic, N, K

// Workspace: 512-byte header (maps, status words), then one counter per tile of 128 weight rows,
// then two f32 partial sums of [16][128] per CTA.
constexpr size_t kTcCountersOffset = 512;
#if defined(__CUDACC__)
__host__ __device__
#endif
constexpr size_t tc_partials_offset(int64_t N) {
  return kTcCountersOffset + ((static_cast<size_t>((N + kTcWRows - 1) / kTcWRows) * 4 + 127) / 128) * 128;
}
#if defined(__CUDACC__)
__host__ __device__
#endif
constexpr size_t tc_workspace_bytes(int64_t N) {
  return tc_partials_offset(N) + static_cast<size_t>(kTcMaxCtas) * 2 * kTcARows * kTcWRows * 4;
}

}  // namespace b200
