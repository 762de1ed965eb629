// Fused "dequantise int4 weights, then contract" for few activation rows (M <= 16) on the tensor
// cores: the same operand roles as b200_w4a16_gemm_wt (weights = the 128-row operand, expanded
// straight into tensor memory; activations = the shared-memory operand, here only 16 rows wide),
// arranged for a product that is bound by streaming the weights out of HBM once.
//
//   w_f16[n,k] = f16( f16(sext(wq[n,k])) * scale[n, k/128] )      (exactly the dequant generic)
//   out[m,n]   = f16( sum_k f32(a[m,k]) * f32(w_f16[n,k]) )
//
// Work is cut into units of 128 weight rows x 512 K (32 KiB of int4). The units are numbered tile
// by tile and dealt to the CTAs as equal contiguous ranges, so every SM streams the same number of
// bytes whatever N and K are. A range that starts or ends inside a tile yields a partial sum: it
// goes to the CTA's slot in the workspace (f32, [16 m][128 n]); when the CTA is done it bumps the
// tile's counter, and whoever arrives last adds the tile's partial sums in CTA order (the result
// does not depend on who that is) and writes the f16 result.
//
// The weights have a ring of their own that only the dequant warps read (the MMAs never touch it).
// Each box takes 256 contiguous bytes per weight row (two 128-byte lines); with 128-byte boxes the
// same loop streams a quarter slower.
//
//   warp 0      TMA producer of the raw weights: one box of 128 rows x 2 x 128 bytes per unit, five
//               stages of 32 KiB
//   warp 2      TMA producer of the activations (eight boxes of 16 rows x 64 K per unit; rows >= M
//               and columns >= K arrive as zeros), three stages of 16 KiB; owns the tensor-memory
//               allocation
//   warp 3      scales of the unit's 128 rows x 4 groups, cp.async into a ring beside the raw stages
//   warps 8-23  dequant, four groups of four warps; group g expands the g-th and (g+4)-th 64 K of
//               every unit: 32 raw bytes of the thread's row -> 32 registers of f16 pairs ->
//               tcgen05.st into the block's 32 columns of tensor memory
//   warp 1      one thread issues tcgen05.mma (A from tensor memory, B from shared memory,
//               M = 128, N = 16), four per 64 K; a tcgen05.mma of this shape takes the tensor pipe
//               about 46 cycles whatever N is, so the 32 per unit cost about as long as the unit's
//               32 KiB take to arrive from HBM
//   warps 4-7   epilogue: tcgen05.ld -> result or partial sum; the meeting of partial sums
//
// Every wait is bounded; a wait that runs out records where in the status words and the kernel
// returns. The waits poll without a suspend hint: this kernel is latency-bound, nearly every wait
// finds its barrier not yet complete, and a suspended warp comes back microseconds late.
// No load here touches another GPU's memory and nothing uses cluster multicast.
#include <cuda_fp16.h>
#include <stdint.h>

#include "sm100_ptx.cuh"
#include "w4a16_decode.cuh"
#include "w4a16_decode_tc.h"

namespace b200 {

constexpr int kTcRawStages = 5;
constexpr int kTcRawBytes = kTcWRows * (kTcUnitK / 2);     // 32 KiB: 128 rows x 2 lines of 128 bytes
constexpr int kTcActStages = 3;
constexpr int kTcActPieceBytes = kTcARows * 128;           // 2 KiB: 16 rows x 64 f16
constexpr int kTcBlocks = kTcUnitK / 64;                   // 64-K blocks per unit = A stages in tensor memory
constexpr int kTcActBytes = kTcBlocks * kTcActPieceBytes;  // 16 KiB
constexpr int kTcScaleBytes = kTcWRows * 8;                // per unit: 128 rows x 4 groups x f16
constexpr int kTcAStageColumns = 32;                       // 64 K as f16 pairs
constexpr int kTcAccColumns = 32;                          // per accumulator buffer; 16 in use
constexpr int kTcDequantWarps = 16;
constexpr int kTcBarrierBytes = 512;
static_assert(kTcThreads == (8 + kTcDequantWarps) * 32, "role layout");
static_assert(kTcBlocks == 8, "two blocks per dequant group and unit");
static_assert(kTcSmemBytes == 1024 + kTcRawStages * (kTcRawBytes + kTcScaleBytes) + kTcActStages * kTcActBytes +
                                  kTcBarrierBytes, "shared memory");
static_assert(2 * kTcAccColumns + kTcBlocks * kTcAStageColumns <= 512, "tensor memory columns");

__device__ __forceinline__ void tc_report(uint32_t* status, uint32_t code, uint32_t info) {
  if (atomicCAS(&status[0], 0u, code) == 0u) status[1] = info;
}

__device__ __forceinline__ void cp_async_4(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst_smem), "l"(src) : "memory");
}
// Arrives on `bar` (without adding to its pending count) once this thread's cp.async so far have landed.
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// Loads from a ring stage that is handed back to its producer right afterwards. They are
// volatile at the PTX level: a weak load may be executed again later (to save registers across
// the long waits that follow), and by then the stage holds the next lap's bytes.
__device__ __forceinline__ uint2 lds64_once(uint32_t addr) {
  uint2 r;
  asm volatile("ld.volatile.shared.v2.u32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "r"(addr) : "memory");
  return r;
}
__device__ __forceinline__ uint4 lds128_once(uint32_t addr) {
  uint4 r;
  asm volatile("ld.volatile.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "r"(addr)
               : "memory");
  return r;
}

// 64 weights of one row (two 16-byte pieces, in K order) times their group's scale -> the 32
// columns of the row's lane in one A stage: column 4 i + j = (w(8 i + 2 j), w(8 i + 2 j + 1)).
__device__ __forceinline__ void tc_expand_block(const uint4& w0, const uint4& w1, __half2 s2, uint32_t taddr) {
  uint32_t e[32];
  const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    __half2 qv[4];
    unpack8_ordered(words[i], qv);
#pragma unroll
    for (int j = 0; j < 4; ++j) e[i * 4 + j] = as_u32(__hmul2(qv[j], s2));  // f16(w) * scale, one rounding
  }
  tmem_st_32x32(taddr, e);
}

__device__ __forceinline__ void decode_tc_body(const __half* __restrict__ scales, __half* __restrict__ out,
                                               uint8_t* __restrict__ ws_raw, int M, int N, int K, int ldo,
                                               int n_off) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t act_base = smem_base + kTcRawStages * kTcRawBytes;
  const uint32_t scale_base = act_base + kTcActStages * kTcActBytes;
  const uint32_t bars = scale_base + kTcRawStages * kTcScaleBytes;
  uint8_t* bars_gen = smem_gen + (bars - smem_base);
  auto raw_full = [&](int i) { return bars + 8u * i; };                              // TMA bytes of raw stage i
  auto raw_empty = [&](int i) { return bars + 8u * (kTcRawStages + i); };            // the 16 dequant warps
  auto sc_full = [&](int i) { return bars + 8u * (2 * kTcRawStages + i); };          // 32 lanes' cp.async
  auto act_full = [&](int i) { return bars + 8u * (3 * kTcRawStages + i); };
  auto act_empty = [&](int i) { return bars + 8u * (3 * kTcRawStages + kTcActStages + i); };
  constexpr int kRingBars = 3 * kTcRawStages + 2 * kTcActStages;
  // The expanded weights of a unit sit in tensor memory as two halves of four blocks; half h is
  // handed over whole (all 16 dequant warps arrive) and comes back with one commit.
  auto a_full = [&](int h) { return bars + 8u * (kRingBars + h); };
  auto a_empty = [&](int h) { return bars + 8u * (kRingBars + 2 + h); };
  constexpr int kABars = kRingBars + 4;
  auto d_full = [&](int i) { return bars + 8u * (kABars + i); };
  auto d_empty = [&](int i) { return bars + 8u * (kABars + 2 + i); };
  const uint32_t tmem_slot = bars + 8u * (kABars + 4);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * (kABars + 4));
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * (kABars + 4) + 4);
  volatile uint32_t* last_flags = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * (kABars + 5));  // two words
  static_assert(8 * (kABars + 6) <= kTcBarrierBytes, "barrier area");

  uint32_t* status = reinterpret_cast<uint32_t*>(ws_raw + 384);
  const uint8_t* map_a = ws_raw;
  const uint8_t* map_w = ws_raw + 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = (N + kTcWRows - 1) / kTcWRows;
  const int kbt = (K + kTcUnitK - 1) / kTcUnitK;  // units per tile; the last one may be half empty
  const int64_t U = static_cast<int64_t>(tiles) * kbt;
  const int64_t G = gridDim.x;
  // The workspace must have been prepared for this N and K (maps, zeroed counters): an unprepared
  // one holds no tensor map, and a TMA through it would be an illegal instruction.
  const bool bad = M <= 0 || M > kTcARows || N <= 0 || K <= 0 || (K % 256) || G > U || G > kTcMaxCtas ||
                   status[16] != kTcNoteMagic || status[17] != static_cast<uint32_t>(N) ||
                   status[18] != static_cast<uint32_t>(K);
  if (bad) {
    if (threadIdx.x == 0) tc_report(status, kStatusBadArgument, 32);
    return;
  }
  uint32_t* counters = reinterpret_cast<uint32_t*>(ws_raw + kTcCountersOffset);
  float* partials = reinterpret_cast<float*>(ws_raw + tc_partials_offset(N));
  const int u0 = static_cast<int>(blockIdx.x * U / G), u1 = static_cast<int>((blockIdx.x + 1) * U / G);

  if (threadIdx.x == 0) {
    for (int i = 0; i < kTcRawStages; ++i) {
      mbar_init(raw_full(i), 1);
      mbar_init(raw_empty(i), kTcDequantWarps);
      mbar_init(sc_full(i), 32);
    }
    for (int i = 0; i < kTcActStages; ++i) {
      mbar_init(act_full(i), 1);
      mbar_init(act_empty(i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(a_full(i), kTcDequantWarps);
      mbar_init(a_empty(i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(d_full(i), 1);
      mbar_init(d_empty(i), 4);
    }
    *abort_flag = 0;
    last_flags[0] = 0;
    last_flags[1] = 0;
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  // The next kernel on the stream may be scheduled as soon as this one's blocks leave their SMs.
  grid_launch_dependents();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const uint32_t tmem_a = tmem_base + 2 * kTcAccColumns;

  if (warp == 0) {
    // -------- TMA producer of the raw weights ----------------------------------------------------------
    // Weights are inputs of the whole program (no kernel writes them): they are requested without
    // waiting for the preceding kernel, which may still be producing the activations.
    if (lane == 0) {
      tensormap_fence_acquire(map_w);
      int st = 0;
      uint32_t parity = 1;  // of the "empty" phase to wait for; the first lap passes at once
      for (int u = u0; u < u1; ++u) {
        if (!mbar_wait<false>(raw_empty(st), parity, abort_flag)) {
          tc_report(status, kStatusTimeoutEmpty, u - u0);
          *abort_flag = 1;
          break;
        }
        const int tile = u / kbt, kb = u - tile * kbt;
        mbar_arrive_expect_tx(raw_full(st), kTcRawBytes);
        tma_load_3d(smem_base + st * kTcRawBytes, map_w, raw_full(st), 0, kb * (kTcUnitK / 256), tile * kTcWRows);
        if (++st == kTcRawStages) {
          st = 0;
          parity ^= 1u;
        }
      }
    }
  } else if (warp == 2) {
    // -------- TMA producer of the activations ----------------------------------------------------------
    if (lane == 0) {
      tensormap_fence_acquire(map_a);
      grid_dependency_wait();
      int st = 0;
      uint32_t parity = 1;
      for (int u = u0; u < u1; ++u) {
        if (!mbar_wait<false>(act_empty(st), parity, abort_flag)) {
          tc_report(status, kStatusTimeoutEmpty, 0x30000u | (u - u0));
          *abort_flag = 1;
          break;
        }
        const int kb = u % kbt;
        const uint32_t dst = act_base + st * kTcActBytes;
        mbar_arrive_expect_tx(act_full(st), kTcActBytes);
#pragma unroll
        for (int p = 0; p < kTcBlocks; ++p)
          tma_load_3d(dst + p * kTcActPieceBytes, map_a, act_full(st), kb * kTcUnitK + p * 64, 0, 0);
        if (++st == kTcActStages) {
          st = 0;
          parity ^= 1u;
        }
      }
    }
  } else if (warp == 3) {
    // -------- scales: rows of the unit's tile, groups 4 kb .. 4 kb + 3 -----------------------------------
    const int groups = K >> 7;
    int st = 0;
    uint32_t parity = 1;
    for (int u = u0; u < u1; ++u) {
      if (!__all_sync(0xffffffffu, mbar_wait<false>(raw_empty(st), parity, abort_flag))) {
        if (lane == 0) {
          tc_report(status, kStatusTimeoutEmpty, 0x10000u | (u - u0));
          *abort_flag = 1;
        }
        break;
      }
      const int tile = u / kbt, kb = u - tile * kbt;
      const int g0 = 4 * kb;
      const int g1 = g0 + 2 < groups ? g0 + 2 : g0;  // the second pair of a half-empty last unit: any finite value
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i * 32 + lane;
        int n = tile * kTcWRows + r;
        n = n < N ? n : N - 1;  // rows past N hold zero weights: any finite scale will do
        const __half* row = scales + static_cast<size_t>(n) * groups;
        cp_async_4(scale_base + st * kTcScaleBytes + r * 8, row + g0);
        cp_async_4(scale_base + st * kTcScaleBytes + r * 8 + 4, row + g1);
      }
      cp_async_arrive(sc_full(st));
      if (++st == kTcRawStages) {
        st = 0;
        parity ^= 1u;
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (warp == 1) {
    // -------- MMA issuer -----------------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_instr_desc(1u, 0u, 0u, 0u, 0u, kTcWRows, kTcARows);
      bool ok = true;
      int seg = 0, st = 0;
      uint32_t act_parity = 0;
      for (int u = u0; u < u1 && ok; ++seg) {
        const int tile = u / kbt;
        const int u_end = (tile + 1) * kbt < u1 ? (tile + 1) * kbt : u1;
        const int buf = seg & 1;
        if (!mbar_wait<false>(d_empty(buf), ((seg >> 1) & 1) ^ 1, abort_flag)) {
          tc_report(status, kStatusTimeoutTmemEmpty, seg);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kTcAccColumns;
        bool first = true;
        for (; u < u_end && ok; ++u) {
          const uint32_t a_parity = (u - u0) & 1;
          if (!mbar_wait<false>(act_full(st), act_parity, abort_flag)) {
            tc_report(status, kStatusTimeoutFull, u - u0);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t act = act_base + st * kTcActBytes;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (!ok) break;
            if (!mbar_wait<false>(a_full(h), a_parity, abort_flag)) {
              tc_report(status, kStatusTimeoutDequant, (u - u0) * 2 + h);
              *abort_flag = 1;
              ok = false;
              break;
            }
            tc_fence_after_sync();
#pragma unroll
            for (int bk = 0; bk < 16; ++bk) {  // blocks 4 h .. 4 h + 3, four k-steps each
              mma_f16_ts(d_tmem, tmem_a + h * (4 * kTcAStageColumns) + bk * 8,
                         make_smem_desc(act + (h * 4 + (bk >> 2)) * kTcActPieceBytes + (bk & 3) * 32, 16, 1024), idesc,
                         first ? 0u : 1u);
              first = false;
            }
            tc_commit(a_empty(h));
          }
          if (ok) tc_commit(act_empty(st));
          if (++st == kTcActStages) {
            st = 0;
            act_parity ^= 1u;
          }
        }
        if (ok) tc_commit(d_full(buf));
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // -------- epilogue ---------------------------------------------------------------------------------
    const int qd = warp & 3;
    const int r = qd * 32 + lane;  // weight row of the tile = accumulator lane
    const bool leader = threadIdx.x == 128;
    // the result, the partial sums and the counters may still be in use by the preceding kernel
    grid_dependency_wait();
    int part_tile[2] = {-1, -1};
    int seg = 0;
    for (int u = u0; u < u1; ++seg) {
      const int tile = u / kbt, kb0 = u - tile * kbt;
      const int u_end = (tile + 1) * kbt < u1 ? (tile + 1) * kbt : u1;
      const bool whole = kb0 == 0 && u_end == (tile + 1) * kbt;
      const int buf = seg & 1;
      if (!__all_sync(0xffffffffu, mbar_wait<false>(d_full(buf), (seg >> 1) & 1, abort_flag))) {
        if (lane == 0) {
          tc_report(status, kStatusTimeoutTmemFull, seg);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after_sync();
      uint32_t v[32];
      tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(qd * 32) << 16) + buf * kTcAccColumns, v);
      tc_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(d_empty(buf));
      const int n = tile * kTcWRows + r;
      if (whole) {
        if (n < N) {
          __half* dst = out + n_off + n;
#pragma unroll
          for (int m = 0; m < kTcARows; ++m)
            if (m < M) dst[static_cast<size_t>(m) * ldo] = __float2half_rn(__uint_as_float(v[m]));
        }
      } else {
        const int which = seg == 0 ? 0 : 1;
        part_tile[which] = tile;
        float* dst = partials + (static_cast<size_t>(blockIdx.x) * 2 + which) * (kTcARows * kTcWRows) + r;
#pragma unroll
        for (int m = 0; m < kTcARows; ++m) __stcg(dst + m * kTcWRows, __uint_as_float(v[m]));
      }
      u = u_end;
    }
    // The meeting of the partial sums, once per CTA. All four warps come here whatever happened
    // above (every wait is bounded), so the two barriers below cannot be left waiting.
    {
      __threadfence();
      named_barrier_sync(1, 128);
      const bool healthy = *abort_flag == 0;
      if (leader && healthy) {
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          if (part_tile[w] < 0) continue;
          const int64_t first_unit = static_cast<int64_t>(part_tile[w]) * kbt;
          const int c_first = static_cast<int>(((first_unit + 1) * G - 1) / U);
          const int c_last = static_cast<int>(((first_unit + kbt) * G - 1) / U);
          const uint32_t arrived = atomicAdd(&counters[part_tile[w]], 1u);
          last_flags[w] = arrived == static_cast<uint32_t>(c_last - c_first) ? 1u : 0u;
        }
        __threadfence();
      }
      named_barrier_sync(1, 128);
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        if (!healthy || part_tile[w] < 0 || !last_flags[w]) continue;
        const int tile = part_tile[w];
        const int64_t first_unit = static_cast<int64_t>(tile) * kbt;
        const int c_first = static_cast<int>(((first_unit + 1) * G - 1) / U);
        const int c_last = static_cast<int>(((first_unit + kbt) * G - 1) / U);
        float acc[kTcARows];
#pragma unroll
        for (int m = 0; m < kTcARows; ++m) acc[m] = 0.f;
        for (int c = c_first; c <= c_last; ++c) {
          const int slot = static_cast<int>(c * U / G) / kbt == tile ? 0 : 1;  // the tile opens c's range, or closes it
          const float* src = partials + (static_cast<size_t>(c) * 2 + slot) * (kTcARows * kTcWRows) + r;
#pragma unroll
          for (int m = 0; m < kTcARows; ++m) acc[m] += __ldcg(src + m * kTcWRows);
        }
        const int n = tile * kTcWRows + r;
        if (n < N) {
          __half* dst = out + n_off + n;
#pragma unroll
          for (int m = 0; m < kTcARows; ++m)
            if (m < M) dst[static_cast<size_t>(m) * ldo] = __float2half_rn(acc[m]);
        }
        if (leader) counters[tile] = 0;  // ready for the next dispatch that uses this workspace
      }
    }
  } else if (warp >= 8) {
    // -------- dequant: raw int4 (128-byte swizzled lines) -> 32 columns of this thread's lane ------------
    const int td = threadIdx.x - 256;
    const int r = td & 127;   // weight row of the tile = lane of tensor memory; td / 32 % 4 == warp % 4
    const int grp = td >> 7;  // blocks grp and grp + 4 of every unit
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    // A stage holds [row][2 lines of 128 bytes]; line l = 2 r + half sits at l * 128 with its 16-byte
    // pieces XOR-swizzled by l % 8. Block b covers pieces 2 (b % 4), 2 (b % 4) + 1 of line half b / 4.
    const uint32_t line0 = static_cast<uint32_t>(2 * r) * 128u, line1 = line0 + 128u;
    const uint32_t sw0 = (2 * r) & 7, sw1 = (2 * r + 1) & 7;
    const uint32_t off00 = line0 + (((2 * grp) ^ sw0) << 4), off01 = line0 + (((2 * grp + 1) ^ sw0) << 4);
    const uint32_t off10 = line1 + (((2 * grp) ^ sw1) << 4), off11 = line1 + (((2 * grp + 1) ^ sw1) << 4);
    const uint32_t sel = (grp & 2) ? 0x3232u : 0x1010u;
    int st = 0;
    uint32_t parity = 0;
    for (int u = u0; u < u1; ++u) {
      const bool got = mbar_wait<false>(raw_full(st), parity, abort_flag) && mbar_wait<false>(sc_full(st), parity, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) {
          tc_report(status, kStatusTimeoutFull, 0x10000u | (u - u0));
          *abort_flag = 1;
        }
        break;
      }
      const uint32_t raw = smem_base + st * kTcRawBytes;
      const uint4 w00 = lds128_once(raw + off00), w01 = lds128_once(raw + off01);
      const uint4 w10 = lds128_once(raw + off10), w11 = lds128_once(raw + off11);
      const uint2 sc = lds64_once(scale_base + st * kTcScaleBytes + r * 8);
      // The stage goes back to its producer after the unit's second expansion, not here: handing it
      // back as soon as the bytes were in registers corrupted single lanes' weights about once in
      // five launches at sixteen units per CTA (also with these volatile loads and with every loaded
      // register consumed before the arrival); with the late hand-over no run has failed.
      const int st_done = st;
      if (++st == kTcRawStages) {
        st = 0;
        parity ^= 1u;
      }
      const uint32_t a_parity = ((u - u0) & 1) ^ 1u;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int b = grp + 4 * h;
        const __half2 s2 = as_half2(__byte_perm(h ? sc.y : sc.x, 0u, sel));
        if (!__all_sync(0xffffffffu, mbar_wait<false>(a_empty(h), a_parity, abort_flag))) {
          if (lane == 0) {
            tc_report(status, kStatusTimeoutEmpty, 0x20000u | ((u - u0) * kTcBlocks + b));
            *abort_flag = 1;
          }
          u = u1;  // leave the unit loop as well
          break;
        }
        tc_fence_after_sync();
        tc_expand_block(h ? w10 : w00, h ? w11 : w01, s2, tmem_a + lane_base + b * kTcAStageColumns);
        tc_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(a_full(h));
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(raw_empty(st_done));
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
  }
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b200

using namespace b200;

// Bindings: scales, the result, the workspace (maps over the activations and the weights at bytes
// 0 and 128, status words at 384, tile counters and partial sums from byte 512 on).
extern "C" __global__ void __launch_bounds__(kTcThreads, 1)
    b200_w4a16_decode_tc(const __half* scales, __half* out, uint8_t* ws, int M, int N, int K, int ldo, int n_off) {
  decode_tc_body(scales, out, ws, M, N, K, ldo, n_off);
}
