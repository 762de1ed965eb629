// Shared device code of the W4A16 kernels: int4 -> f16 unpacking helpers and the body of the
// decode (M <= 16) kernel, so that more than one translation unit can instantiate it.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace b200 {

// ---------------------------------------------------------------------------------------------
// int4 -> f16 helpers. A 32-bit word holds 8 weights; nibble j (bits 4j..4j+3) is weight j.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t v, uint32_t mask, uint32_t x) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(r) : "r"(v), "r"(mask), "r"(x));  // (v & mask) ^ x
  return r;
}
__device__ __forceinline__ __half2 as_half2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

// Exact signed values of weights in memory order: q[j] = (w(2j), w(2j+1)), j = 0..3 (byte j).
// 0x6400 | x is the f16 1024 + x and 0x5400 | (x << 4) is 64 + x; flipping the nibble's top bit
// turns two's complement into "value + 8", so the constants 1032 and 72 come off again exactly.
__device__ __forceinline__ void unpack8_ordered(uint32_t v, __half2 (&q)[4]) {
  const __half2 mul = __halves2half2(__float2half_rn(1.f), __float2half_rn(0.0625f));
  const __half2 add = __halves2half2(__float2half_rn(-1032.f), __float2half_rn(-72.f));
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t rep;
    asm("prmt.b32 %0, %1, %1, %2;" : "=r"(rep) : "r"(v), "r"(0x1111u * j));  // byte j in every byte
    // low half: 1024 + (n_lo ^ 8); high half: 1024 + 16 (n_hi ^ 8)
    q[j] = __hfma2(as_half2(lop3_and_xor(rep, 0x00f0000fu, 0x64806408u)), mul, add);
  }
}

__device__ __forceinline__ int sext4(uint32_t nib) { return static_cast<int>((nib ^ 8u) & 0xfu) - 8; }

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Shared-memory accesses by 32-bit shared-space address.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 r;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
  return r;
}
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
  float4 r;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "r"(addr));
  return r;
}
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
  float2 r;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(r.x), "=f"(r.y) : "r"(addr));
  return r;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t r;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r) : "r"(addr));
  return r;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts128f(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void sts64f(uint32_t addr, float a, float b) {
  asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
}
// Untiled bulk copy global -> shared, completion reported to an mbarrier as transaction bytes.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// =============================================================================================
// Decode kernel (M <= 16): HBM-bound streaming of the int4 weights.
//
// Work is cut along N into tiles of 16 weight rows and along K into slices of 4096. A CTA owns
// one K slice for its whole life and walks over every (grid / slices)-th tile; its 16 warps each
// own a 256-wide chunk of the slice and keep the activations of that chunk in registers, already
// in the order the MMAs want them. A tile travels global -> shared as two blocks of eight rows
// into a four-stage ring guarded by full / empty mbarriers: two bulk copies when the CTA's slice
// is the whole row (the blocks are contiguous in memory), else two TMA boxes from a tensor map in
// the workspace (issuing one copy per row would cost the issuing warp ~130 cycles each, more than
// the rows take to arrive). Even / odd fragment rows are taken from different blocks, and on the
// bulk-copy path the second block is staged 64 bytes off the first block's bank alignment, so that
// the two rows a quarter warp reads with one 16-byte load instruction fall into different banks
// (a TMA box must land on a 128-byte boundary: there the two rows share their banks).
//
// A warp turns its 16 x 128 bytes of a tile into f16 MMA operands with two logic operations per
// register: the nibbles become the biased halves 1032 + w (low nibbles, 0x6400 | n ^ 8) and
// 72 + w (high nibbles, 0x5400 | (n ^ 8) << 4), which go straight into mma.sync.m16n8k16 with
// the weights as the 16-row operand; the accumulator of each scale group starts at minus the
// constant part (1032 S_lo + 72 S_hi, with S the sums of the activations that meet low / high
// nibbles, computed once per kernel by an all-ones MMA), so what comes out is the exact group
// sum, which is multiplied by the group's scale in f32. The 16 chunk sums of a tile meet in a
// shared-memory slot; one warp per tile (in rotation, two tiles behind the main loop) adds them
// in chunk order and writes f16.
//
// K beyond one slice: every CTA leaves the f32 partial tiles of its slice in global scratch and,
// when it is done, bumps the counter of its tile walker; the CTA that bumps it last adds the
// slices of all the walker's tiles in slice order and writes the results, then resets the
// counter. Nobody waits for anybody.
// =============================================================================================
constexpr int kDecodeThreads = 512;
constexpr int kDecodeWarps = 16;
constexpr int kDecodeChunkK = 256;                           // K per warp
constexpr int kDecodeSliceK = kDecodeWarps * kDecodeChunkK;  // K per CTA: 4096
constexpr int kDecodeMaxSlices = 4;                          // K <= 16384
constexpr int kDecodeTileRows = 16;                          // weight rows per tile
// Weight tiles resident in shared memory. What the stream needs is bytes in flight: HBM delivers
// its peak to one CTA per SM only with about 128 KiB outstanding per SM. The 16-row variant has
// room for four stages, the 8-row variant for five.
__host__ __device__ constexpr int decode_stages(int mh) { return mh == 1 ? 5 : 4; }
constexpr int kDecodeSlots = 3;                              // tiles whose chunk sums are live at the same time
constexpr int kDecodeFinalizeLag = 2;                        // a tile is reduced this many tiles behind the main loop
constexpr int kDecodeHalfSkew = 64;                          // bulk-copy path: the second eight rows sit this far off the first block's banks
constexpr int kDecodeStageBytes = kDecodeTileRows * (kDecodeSliceK / 2) + 128;  // two blocks of 8 rows x <= 2048 B + skew
constexpr int kDecodeScaleStageBytes = 16 * 128 * 2;         // 16 rows x up to 128 groups of f16
constexpr int kDecodeBarrierBytes = 256;                     // up to 16 mbarriers + the abort word
static_assert(kDecodeSlots > kDecodeFinalizeLag, "a slot must be reduced before the main loop needs it again");

// Dynamic shared memory:
//   weight ring  [stage]{[8][pitch], 64 B, [8][pitch]}  the tile's rows of the CTA's K slice, pitch = slice bytes per row
//   scale ring   [stage][4096 B]                the tile's scale rows (whole rows: one contiguous copy)
//   chunk sums   [slot][warp][lane][MH] float4  MMA fragment order; doubles as the staging area of the prologue
//   offsets      [warp][MH][step][lane] float2  the constant part of each group sum, per output column
//   mbarriers    weights full / empty per stage, chunk sums full / empty per slot; abort word
__host__ __device__ constexpr int decode_smem_bytes(int mh) {
  return decode_stages(mh) * kDecodeStageBytes + decode_stages(mh) * kDecodeScaleStageBytes +
         kDecodeSlots * kDecodeWarps * 32 * 16 * mh + kDecodeWarps * mh * 2 * 32 * 8 + kDecodeBarrierBytes;
}

// Global scratch of a decode dispatch whose K spans more than one slice:
//   counters [N / 16] u32 (one per tile walker is used; zero between launches), padded to 256 bytes, then
//   partial tiles [tile][slice][lane][2] float4 (fragment order; contents need not be initialised).
struct DecodeScratchLayout {
  __host__ __device__ static constexpr size_t counter_bytes(int N) {
    return (static_cast<size_t>(N / 16) * 4 + 255) & ~size_t(255);
  }
  __host__ __device__ static constexpr size_t bytes(int N, int slices) {
    return counter_bytes(N) + static_cast<size_t>(N / 16) * slices * 32 * 2 * 16;
  }
};

// Status words a decode kernel writes when one of its bounded waits runs out (status[0] stays 0
// otherwise): [0] which wait, [1] tile index, [2] N (how much scratch the host has to clear).
enum : uint32_t {
  kStatusDecodeWeights = 16,   // a weight stage never filled
  kStatusDecodeStage = 17,     // a weight stage never drained
  kStatusDecodeSlotFull = 18,  // the chunk sums of a tile never all arrived
  kStatusDecodeSlotFree = 19,  // a chunk-sum slot was never released
};

__device__ __noinline__ bool decode_wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                              uint32_t* status, uint32_t code, uint32_t info, uint32_t n) {
  const uint64_t t0 = global_timer_ns();
  uint32_t polls = 0;
  while (true) {
    if (mbar_try_wait<false>(bar, parity)) return true;
    if ((++polls & 0xff) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > kDefaultWaitLimitNs) {
        *abort_flag = 1;
        if (status && atomicCAS(&status[0], 0u, code) == 0u) {
          status[1] = info;
          status[2] = n;
        }
        return false;
      }
    }
  }
}
// All lanes of a warp poll the same barrier, so they leave together; a phase that has completed
// stays completed until this warp arrives again, so they also agree on the outcome.
__device__ __forceinline__ bool decode_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                            uint32_t* status, uint32_t code, uint32_t info, uint32_t n) {
  if (mbar_try_wait<false>(bar, parity)) return true;
  return decode_wait_slow(bar, parity, abort_flag, status, code, info, n);
}

template <int MH>
__device__ __forceinline__ void decode_body(const __half* __restrict__ a, const uint8_t* __restrict__ wq,
                                            const __half* __restrict__ scales, __half* __restrict__ out,
                                            void* __restrict__ scratch, uint32_t* __restrict__ status,
                                            const void* __restrict__ wmap, bool wmap_in_workspace, int M, int N,
                                            int K, int ldo, int n_off) {
  extern __shared__ __align__(128) uint8_t decode_smem[];
  constexpr int kDecodeStages = decode_stages(MH);
  constexpr int kWRingBytes = kDecodeStages * kDecodeStageBytes;
  constexpr int kSRingBytes = kDecodeStages * kDecodeScaleStageBytes;
  constexpr int kSumBytes = kDecodeSlots * kDecodeWarps * 32 * 16 * MH;
  constexpr int kOffsetBytes = kDecodeWarps * MH * 2 * 32 * 8;
  const uint32_t smem0 = smem_u32(decode_smem);
  const uint32_t wring = smem0, sring = wring + kWRingBytes, sums = sring + kSRingBytes, offsets = sums + kSumBytes;
  const uint32_t bars = offsets + kOffsetBytes;
  auto wfull_bar = [&](int i) { return bars + 8u * i; };
  auto wempty_bar = [&](int i) { return bars + 8u * (kDecodeStages + i); };
  auto pfull_bar = [&](int i) { return bars + 8u * (2 * kDecodeStages + i); };
  auto pempty_bar = [&](int i) { return bars + 8u * (2 * kDecodeStages + kDecodeSlots + i); };
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(
      decode_smem + kWRingBytes + kSRingBytes + kSumBytes + kOffsetBytes + 8 * (2 * kDecodeStages + 2 * kDecodeSlots));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int groups_per_row = K >> 7;
  const int row_bytes = K >> 1;
  const int num_tiles = N / kDecodeTileRows;
  const int slices = (K + kDecodeSliceK - 1) / kDecodeSliceK;
  if (slices > 1 && wmap_in_workspace) {
    // The tensor map over the weights is written into the workspace by the host (or by a map-building
    // dispatch) together with a note of what it was built for: status words 16..19 = weights address
    // (low, high), N, K. A map that was never written, or written for other weights, must not reach
    // the copy engine: the whole grid refuses, reports, and leaves the result untouched.
    const uint64_t noted = static_cast<uint64_t>(__ldcg(&status[16])) | (static_cast<uint64_t>(__ldcg(&status[17])) << 32);
    if (noted != reinterpret_cast<uint64_t>(wq) || __ldcg(&status[18]) != static_cast<uint32_t>(N) ||
        __ldcg(&status[19]) != static_cast<uint32_t>(K)) {
      if (threadIdx.x == 0 && atomicCAS(&status[0], 0u, static_cast<uint32_t>(kStatusBadArgument)) == 0u) status[1] = 16;
      return;
    }
  }
  // CTA c holds slice c % slices of the tiles c / slices, c / slices + walkers, ...
  const int slice = blockIdx.x % slices;
  const int walker = blockIdx.x / slices, walkers = gridDim.x / slices;
  const int my_tiles = walker < walkers && walker < num_tiles ? (num_tiles - walker + walkers - 1) / walkers : 0;
  const int k_slice0 = slice * kDecodeSliceK;
  int active_warps = (K - k_slice0) / kDecodeChunkK;  // K chunks in this slice (K is a multiple of 256)
  if (active_warps > kDecodeWarps) active_warps = kDecodeWarps;
  // Warps without a K chunk still run the barrier protocol and their share of the reductions, so
  // that every arrival count is the constant 16.
  const bool has_chunk = warp < active_warps;
  const int kc = k_slice0 + warp * kDecodeChunkK;
  // Staged layout of a tile: rows 0..7 at `pitch` bytes each, then (bulk-copy path: 64 bytes off the
  // bank alignment) rows 8..15. Fragment row g (and g + 8) of the MMA is tile row (g & 1) * 8 + (g >> 1) (+ 4): a
  // quarter warp holds one even and one odd g, i.e. one row of each block.
  const uint32_t pitch = slices == 1 ? static_cast<uint32_t>(row_bytes) : static_cast<uint32_t>(kDecodeSliceK / 2);
  const uint32_t half_bytes = 8 * pitch;
  const uint32_t half_pitch = half_bytes + (slices == 1 ? kDecodeHalfSkew : 0);  // second block's offset in the stage
  const int tile_row = (g & 1) * 8 + (g >> 1);  // of fragment row g; fragment row g + 8 is tile row + 4
  const uint32_t srow_pitch = static_cast<uint32_t>(groups_per_row) * 2u;
  const uint32_t scale_tile_bytes = kDecodeTileRows * srow_pitch;

  if (threadIdx.x < 2 * kDecodeStages + 2 * kDecodeSlots) {
    // one barrier per thread: weights full (1 arrival), weights empty (16), chunk sums full (16), empty (1)
    const int i = threadIdx.x;
    const bool sixteen = (i >= kDecodeStages && i < 2 * kDecodeStages) ||
                         (i >= 2 * kDecodeStages && i < 2 * kDecodeStages + kDecodeSlots);
    mbar_init(bars + 8u * i, sixteen ? kDecodeWarps : 1);
    if (i == 0) *abort_flag = 0;
    mbar_fence_init();
  }
  // The next kernel on the stream may be scheduled as soon as this one's blocks leave their SMs:
  // it will fetch its first weight tiles (weights and scales are inputs of the whole program, no
  // kernel writes them) and then wait, below, for this kernel to finish.
  grid_launch_dependents();
  __syncthreads();

  // Feeding the weight ring is a side job that rotates over the warps (tile jp is fetched by warp
  // jp % 16): lanes 0 and 1 fetch the two eight-row blocks, lane 2 the scale rows.
  if (slices > 1 && threadIdx.x == 0) tensormap_fence_acquire(wmap);
  // `st` / `empty_parity`: the stage tile jp goes into and the phase of its "empty" barrier to wait for
  // (the main loop keeps both as running values instead of dividing).
  auto produce = [&](int jp, int st, uint32_t empty_parity) -> bool {
    if (!decode_wait(wempty_bar(st), empty_parity, abort_flag, status, kStatusDecodeStage, jp, N)) return false;
    const size_t row0 = static_cast<size_t>(walker + jp * walkers) * kDecodeTileRows;
    // a TMA box always delivers its full 8 x 2048 bytes (columns past the row's end arrive as zeros)
    if (lane == 0) mbar_arrive_expect_tx(wfull_bar(st), 2 * half_bytes + scale_tile_bytes);
    __syncwarp();
    if (lane < 2) {
      const uint32_t dst = wring + st * kDecodeStageBytes + lane * half_pitch;
      if (slices == 1)
        bulk_load(dst, wq + (row0 + 8 * lane) * row_bytes, half_bytes, wfull_bar(st));
      else
        tma_load_2d(dst, wmap, wfull_bar(st), slice * (kDecodeSliceK / 16), static_cast<int>(row0) + 8 * lane);
    } else if (lane == 2) {
      bulk_load(sring + st * kDecodeScaleStageBytes, scales + row0 * groups_per_row, scale_tile_bytes, wfull_bar(st));
    }
    return true;
  };
  bool ok = true;
  for (int jp = 0; jp < kDecodeStages && jp < my_tiles; ++jp)
    if (warp == jp) ok = produce(jp, jp, 1u) && ok;

  // ---- activations of this warp's chunk, kept in registers in the order the MMAs want ---------------
  // A weight word holds the eight k = k0 .. k0 + 7, k0 = kc + 128 s + 32 q + 8 i for step s, thread
  // column q and word i; the lop3 pairs pick nibbles (0,4), (1,5), (2,6), (3,7), so the B fragments
  // pair the activations the same way. Each warp reads its chunk of eight activation rows with
  // coalesced 256-byte requests, parks it in its corner of the chunk-sum area (not in use yet) and
  // picks up the 64 bytes per row and step it needs.
  // Activations, the scratch and the output may belong to the preceding kernel until it is done.
  grid_dependency_wait();
  uint32_t bfrag[MH][2][4][4];
  float offs[MH][2][2];  // 1032 S_lo + 72 S_hi per step and output column (2q, 2q + 1)
  if (has_chunk && my_tiles > 0) {
    const uint32_t tmp = sums + warp * 2048;
#pragma unroll
    for (int mh = 0; mh < MH; ++mh)
#pragma unroll
      for (int s = 0; s < 2; ++s)
#pragma unroll
        for (int it = 0; it < 4; ++it) {  // 8 rows x 256 bytes, half a warp per row
          const int m = 2 * it + (lane >> 4) + 8 * mh;
          uint4 x = make_uint4(0, 0, 0, 0);
          if (m < M) x = *reinterpret_cast<const uint4*>(a + static_cast<size_t>(m) * K + kc + 128 * s + 8 * (lane & 15));
          bfrag[mh][s][it][0] = x.x;
          bfrag[mh][s][it][1] = x.y;
          bfrag[mh][s][it][2] = x.z;
          bfrag[mh][s][it][3] = x.w;
        }
#pragma unroll
    for (int mh = 0; mh < MH; ++mh)
#pragma unroll
      for (int s = 0; s < 2; ++s) {
#pragma unroll
        for (int it = 0; it < 4; ++it)
          sts128(tmp + (2 * it + (lane >> 4)) * 256 + (lane & 15) * 16,
                 make_uint4(bfrag[mh][s][it][0], bfrag[mh][s][it][1], bfrag[mh][s][it][2], bfrag[mh][s][it][3]));
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 x = lds128(tmp + g * 256 + 64 * q + 16 * i);
          // x = (e0,e1), y = (e2,e3), z = (e4,e5), w = (e6,e7) of the thread's eight k
          bfrag[mh][s][i][0] = __byte_perm(x.x, x.z, 0x5410);  // (e0, e4)
          bfrag[mh][s][i][1] = __byte_perm(x.x, x.z, 0x7632);  // (e1, e5)
          bfrag[mh][s][i][2] = __byte_perm(x.y, x.w, 0x5410);  // (e2, e6)
          bfrag[mh][s][i][3] = __byte_perm(x.y, x.w, 0x7632);  // (e3, e7)
        }
        __syncwarp();
        float s_lo[4] = {0.f, 0.f, 0.f, 0.f}, s_hi[4] = {0.f, 0.f, 0.f, 0.f};
        const uint32_t ones = 0x3c003c00u;  // (1.0, 1.0)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          mma_m16n8k16(s_lo, ones, ones, ones, ones, bfrag[mh][s][i][0], bfrag[mh][s][i][2]);
          mma_m16n8k16(s_hi, ones, ones, ones, ones, bfrag[mh][s][i][1], bfrag[mh][s][i][3]);
        }
        offs[mh][s][0] = -(1032.f * s_lo[0] + 72.f * s_hi[0]);
        offs[mh][s][1] = -(1032.f * s_lo[1] + 72.f * s_hi[1]);
      }
  }
  // The staging corners become chunk-sum slots only after every warp is done with them.
  __syncthreads();
  const uint32_t my_offsets = offsets + ((warp * MH * 2) * 32 + lane) * 8;  // + (mh * 2 + s) * 256
  if (has_chunk && my_tiles > 0) {
#pragma unroll
    for (int mh = 0; mh < MH; ++mh)
#pragma unroll
      for (int s = 0; s < 2; ++s) sts64f(my_offsets + (mh * 2 + s) * 256, offs[mh][s][0], offs[mh][s][1]);
  }
  __syncwarp();

  // Adds the K chunks of tile jf in chunk order (so the result does not depend on arrival order),
  // frees the slot and writes the 16 x M results (one slice) or hands the partial tile to the
  // slice reduction. One warp per tile, in rotation.
  // Fragment order: vals[mh][c] is tile row tile_row + 4 (c / 2), activation row 2 q + (c & 1) + 8 mh.
  auto finalize = [&](int jf, int slot, uint32_t full_parity) -> bool {
    const int tile = walker + jf * walkers;
    if (!decode_wait(pfull_bar(slot), full_parity, abort_flag, status, kStatusDecodeSlotFull, jf, N)) return false;
    float vals[MH][4];
#pragma unroll
    for (int mh = 0; mh < MH; ++mh)
#pragma unroll
      for (int c = 0; c < 4; ++c) vals[mh][c] = 0.f;
    const uint32_t cell0 = sums + ((slot * kDecodeWarps) * 32 + lane) * 16 * MH;
    // a batch of loads first, then the adds: sixteen dependent load-add steps would cost sixteen
    // shared-memory latencies
    constexpr int kBatch = 8 / MH;
#pragma unroll
    for (int first = 0; first < kDecodeWarps; first += kBatch) {
      float4 v[kBatch][MH];
#pragma unroll
      for (int k = 0; k < kBatch; ++k)
#pragma unroll
        for (int mh = 0; mh < MH; ++mh) v[k][mh] = lds128f(cell0 + (first + k) * 32 * 16 * MH + mh * 16);
#pragma unroll
      for (int k = 0; k < kBatch; ++k)
#pragma unroll
        for (int mh = 0; mh < MH; ++mh) {
          vals[mh][0] += v[k][mh].x;
          vals[mh][1] += v[k][mh].y;
          vals[mh][2] += v[k][mh].z;
          vals[mh][3] += v[k][mh].w;
        }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(pempty_bar(slot));  // hand the slot to tile jf + kDecodeSlots
    if (slices > 1) {
      // Several K slices: this CTA's partial tile goes to global memory; the slices meet once, when
      // the CTAs are done (below). No fence and no counting here: a fence under a saturated memory
      // system stalls the warp for microseconds, and every other warp of the CTA soon waits for it.
      float4* parts = reinterpret_cast<float4*>(static_cast<uint8_t*>(scratch) + DecodeScratchLayout::counter_bytes(N)) +
                      (static_cast<size_t>(tile) * slices + slice) * 64 + lane * 2;
#pragma unroll
      for (int mh = 0; mh < MH; ++mh)
        __stcg(parts + mh, make_float4(vals[mh][0], vals[mh][1], vals[mh][2], vals[mh][3]));
      return true;
    }
#pragma unroll
    for (int mh = 0; mh < MH; ++mh)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int r = tile_row + 4 * (c >> 1), m = 2 * q + (c & 1) + 8 * mh;
        if (m < M) out[static_cast<size_t>(m) * ldo + n_off + tile * kDecodeTileRows + r] = __float2half_rn(vals[mh][c]);
      }
    return true;
  };

  // Per-thread addresses inside a stage: weights of this thread's two tile rows at this warp's chunk
  // and this thread's 16-byte column; scales of the chunk's two groups (adjacent f16) of the same rows.
  const uint32_t w_addr0 = wring + (g & 1) * half_pitch + (g >> 1) * pitch + warp * (kDecodeChunkK / 2) + 16 * q;
  const uint32_t s_addr0 = sring + tile_row * srow_pitch + static_cast<uint32_t>(k_slice0 >> 6) + warp * 4;
  const uint32_t sum_addr0 = sums + (warp * 32 + lane) * 16 * MH;

  // Running ring positions (stage / slot index, phase bit, addresses) instead of divisions per tile.
  int st = 0, slot = 0, fslot = 0;       // stage of tile j, chunk-sum slot of tile j, slot of the tile to finalise
  uint32_t wph = 0, sph = 0, fph = 0;    // phase bits of the same
  uint32_t wa = w_addr0, sa = s_addr0, cell = sum_addr0;
  for (int j = 0; j < my_tiles && ok; ++j) {
    if (!decode_wait(wfull_bar(st), wph, abort_flag, status, kStatusDecodeWeights, j, N)) break;
    uint4 w[2][2];
    uint32_t sc[2] = {0, 0};
    if (has_chunk) {
#pragma unroll
      for (int s = 0; s < 2; ++s)
#pragma unroll
        for (int h = 0; h < 2; ++h) w[s][h] = lds128(wa + 64 * s + h * 4 * pitch);
      sc[0] = lds32(sa);
      sc[1] = lds32(sa + 4 * srow_pitch);
    }
    __syncwarp();  // the whole warp has read this stage
    if (lane == 0) mbar_arrive(wempty_bar(st));
    float acc[MH][4];
#pragma unroll
    for (int mh = 0; mh < MH; ++mh)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[mh][c] = 0.f;
    if (has_chunk) {
      // One step is exactly one scale group of the thread's two tile rows.
      const float2 s_g = __half22float2(as_half2(sc[0]));
      const float2 s_g8 = __half22float2(as_half2(sc[1]));
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        float d[MH][4];
#pragma unroll
        for (int mh = 0; mh < MH; ++mh) {
          const float2 o = lds64f(my_offsets + (mh * 2 + s) * 256);
          d[mh][0] = o.x;
          d[mh][1] = o.y;
          d[mh][2] = o.x;
          d[mh][3] = o.y;
        }
        const uint32_t wl[4] = {w[s][0].x, w[s][0].y, w[s][0].z, w[s][0].w};  // fragment row g
        const uint32_t wh[4] = {w[s][1].x, w[s][1].y, w[s][1].z, w[s][1].w};  // fragment row g + 8
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t l8 = wl[i] >> 8, h8 = wh[i] >> 8;
          const uint32_t lo_a = lop3_and_xor(wl[i], 0x000f000fu, 0x64086408u);  // (w0, w4) + 1032
          const uint32_t lo_b = lop3_and_xor(wh[i], 0x000f000fu, 0x64086408u);
          const uint32_t lo_c = lop3_and_xor(l8, 0x000f000fu, 0x64086408u);     // (w2, w6) + 1032
          const uint32_t lo_d = lop3_and_xor(h8, 0x000f000fu, 0x64086408u);
          const uint32_t hi_a = lop3_and_xor(wl[i], 0x00f000f0u, 0x54805480u);  // (w1, w5) + 72
          const uint32_t hi_b = lop3_and_xor(wh[i], 0x00f000f0u, 0x54805480u);
          const uint32_t hi_c = lop3_and_xor(l8, 0x00f000f0u, 0x54805480u);     // (w3, w7) + 72
          const uint32_t hi_d = lop3_and_xor(h8, 0x00f000f0u, 0x54805480u);
#pragma unroll
          for (int mh = 0; mh < MH; ++mh) {
            mma_m16n8k16(d[mh], lo_a, lo_b, lo_c, lo_d, bfrag[mh][s][i][0], bfrag[mh][s][i][2]);
            mma_m16n8k16(d[mh], hi_a, hi_b, hi_c, hi_d, bfrag[mh][s][i][1], bfrag[mh][s][i][3]);
          }
        }
        const float sg = s ? s_g.y : s_g.x, sg8 = s ? s_g8.y : s_g8.x;
#pragma unroll
        for (int mh = 0; mh < MH; ++mh) {
          acc[mh][0] = fmaf(sg, d[mh][0], acc[mh][0]);
          acc[mh][1] = fmaf(sg, d[mh][1], acc[mh][1]);
          acc[mh][2] = fmaf(sg8, d[mh][2], acc[mh][2]);
          acc[mh][3] = fmaf(sg8, d[mh][3], acc[mh][3]);
        }
      }
    }

    // ---- leave this K chunk's sums in the tile's slot ----------------------------------------------
    {
      if (!decode_wait(pempty_bar(slot), sph ^ 1u, abort_flag, status, kStatusDecodeSlotFree, j, N)) break;
#pragma unroll
      for (int mh = 0; mh < MH; ++mh) sts128f(cell + mh * 16, acc[mh][0], acc[mh][1], acc[mh][2], acc[mh][3]);
      __syncwarp();
      if (lane == 0) mbar_arrive(pfull_bar(slot));
    }
    // Refill of the stage this tile came from: it is free once every warp has read it, which by now
    // is almost always the case. Asking here, rather than when the next tile lands, keeps one more
    // tile in flight (the stream needs bytes in flight more than anything else).
    {
      const int jp = j + kDecodeStages;  // same stage; its "empty" phase to wait for is this tile's phase
      if (jp < my_tiles && warp == (jp & (kDecodeWarps - 1)) && !produce(jp, st, wph)) break;
    }
    // Tile j - 2 is finished off by warp (j - 2) % 16: by now every chunk has arrived, so the wait
    // is short, and no warp needs another warp's answer on its critical path.
    if (j >= kDecodeFinalizeLag) {
      if (warp == ((j - kDecodeFinalizeLag) & (kDecodeWarps - 1))) ok = finalize(j - kDecodeFinalizeLag, fslot, fph);
      if (++fslot == kDecodeSlots) fslot = 0, fph ^= 1u;
    }
    if (++st == kDecodeStages) {
      st = 0, wph ^= 1u, wa = w_addr0, sa = s_addr0;
    } else {
      wa += kDecodeStageBytes, sa += kDecodeScaleStageBytes;
    }
    if (++slot == kDecodeSlots) {
      slot = 0, sph ^= 1u, cell = sum_addr0;
    } else {
      cell += kDecodeWarps * 32 * 16 * MH;
    }
  }
  for (int jf = my_tiles > kDecodeFinalizeLag ? my_tiles - kDecodeFinalizeLag : 0; jf < my_tiles; ++jf) {
    if (warp == (jf & (kDecodeWarps - 1)) && ok && !*abort_flag) ok = finalize(jf, fslot, fph);
    if (++fslot == kDecodeSlots) fslot = 0, fph ^= 1u;
  }

  if (slices > 1) {
    // The slices of a walker's tiles meet here, once per CTA: everybody's partial tiles are issued
    // (barrier), one thread publishes them (fence) and counts; the CTA that counts last reads all
    // slices of every tile past the L1, adds them in slice order and writes the results.
    __syncthreads();
    volatile uint32_t* last_flag = abort_flag + 1;
    if (threadIdx.x == 0) {
      uint32_t* counters = reinterpret_cast<uint32_t*>(scratch);
      uint32_t is_last = 0;
      if (!*abort_flag && my_tiles > 0) {
        __threadfence();
        is_last = atomicAdd(&counters[walker], 1u) == static_cast<uint32_t>(slices - 1);
        if (is_last) {
          __threadfence();
          counters[walker] = 0;  // clean for the next launch
        }
      }
      *last_flag = is_last;
    }
    __syncthreads();
    if (*last_flag) {
      const float4* all = reinterpret_cast<const float4*>(static_cast<const uint8_t*>(scratch) + DecodeScratchLayout::counter_bytes(N));
      for (int jf = warp; jf < my_tiles; jf += kDecodeWarps) {
        const int tile = walker + jf * walkers;
        float total[MH][4];
#pragma unroll
        for (int mh = 0; mh < MH; ++mh)
#pragma unroll
          for (int c = 0; c < 4; ++c) total[mh][c] = 0.f;
        for (int sl = 0; sl < slices; ++sl) {
#pragma unroll
          for (int mh = 0; mh < MH; ++mh) {
            const float4 v = __ldcg(all + (static_cast<size_t>(tile) * slices + sl) * 64 + lane * 2 + mh);
            total[mh][0] += v.x;
            total[mh][1] += v.y;
            total[mh][2] += v.z;
            total[mh][3] += v.w;
          }
        }
#pragma unroll
        for (int mh = 0; mh < MH; ++mh)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int r = tile_row + 4 * (c >> 1), m = 2 * q + (c & 1) + 8 * mh;
            if (m < M) out[static_cast<size_t>(m) * ldo + n_off + tile * kDecodeTileRows + r] = __float2half_rn(total[mh][c]);
          }
      }
    }
  }

  // Teardown: everyone meets here, also after a wait ran out. Bulk copies may then still be
  // landing in shared memory, so they get a bounded grace period before the CTA exits.
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
  }
}

}  // namespace b200
