// iree_uk_mmt4d on operands that are already tiled:
//   out[M1, N1, M0, N0] (+)= lhs[M1, K1, M0, K0] x rhs[N1, K1, N0, K0]
// (runtime/src/iree/builtins/ukernel/mmt4d.c:55-141: one tile function call per (m1, n1), walking K1).
// One launch; no operand is brought back to row-major first.
//
// A tile row of the left operand, lhs[m1, k1, :, :], is M0 * K0 contiguous elements; this kernel takes
// the tile shapes for which that row, and the right operand's, is 32 bytes (i8 16x16x2, the x86-64 VNNI
// tile; f16 / bf16 16x16x1). Seen as a matrix with the 32 bytes as its rows-of-the-product dimension and
// K1 as its reduction dimension the operand is "MN-major" with a 32-byte pitch, the layout the tensor
// core reads with the 32-byte swizzle: shared memory holds the operand bytes in memory order, only the
// two 16-byte halves of every second group of four rows trade places. The producers copy 16 bytes at a
// time with cp.async (a TMA box with 32-byte rows moves a quarter of what one with 128-byte rows does:
// measured 22 bytes per clock and SM), apply that swap in the destination address and zero-fill past
// the ends; no thread touches operand data in registers.
//
// K0 = 2 (i8): the two reduction elements of a row are interleaved with its M0 rows, so the 32 bytes
// are 16 rows x 2 reduction elements. The kernel multiplies the operands as if every (row, k0) pair were
// a row of its own, A'[(m0, k0), k1] x B'[(n0, k0'), k1], which needs no rearrangement at all, and the
// epilogue adds the two diagonal terms of every 2 x 2 block: C[m0, n0] = C'[(m0,0),(n0,0)] + C'[(m0,1),(n0,1)]
// (integer arithmetic: exact). Half of the tensor-core work is discarded; in exchange the operands
// stream without a transposition and an int8 MMA is twice as fast as an f16 one.
//
//   warps 8-15: producers, 4-stage ring of {128 A' rows, bn B' rows} x (128 / element size) K1 steps;
//               up to three stages of copies in flight per thread (cp.async groups)
//   warp 1    : one thread issues tcgen05.mma (M = 128, N = bn, both operands MN-major, 32-byte swizzle)
//   warp 2    : TMEM allocation (2 accumulators of up to 256 columns)
//   warps 4-7 : epilogue: tcgen05.ld, the diagonal sum (K0 = 2), ACCUMULATE, whole output tile rows stored
//               with 32-byte stores (a warp writes one or two complete [M0, N0] tiles, contiguous memory)
//
// Compiled in one translation unit after contraction_sm100.cu (Workspace, KindTraits, report, status codes).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace b200 {

constexpr int kMtRunBytes = 32;                         // bytes of one tile row, both operands
constexpr int kMtThreads = 512;
constexpr int kMtSmemBytes = 1024 + kStages * kStageBytes + 256;
constexpr int kMtProducerThreads = 256;                 // warps 8-15
constexpr int kMtCopyDepth = 3;                         // stages of copies in flight per producer thread
constexpr uint64_t kLayoutSwizzle32B = 6;

__device__ __forceinline__ uint64_t make_smem_desc_sw32(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3fff);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= 1ull << 46;
  d |= kLayoutSwizzle32B << 61;
  return d;
}

// 16 bytes global -> shared, bypassing L1; src_bytes = 0 writes zeros and reads nothing.
__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint4 ld_global_128(const void* p) {
  uint4 r;
  asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
  return r;
}

struct Mmt4dShape {
  int M1, N1, K1;
  int lhs_stride0, rhs_stride0, out_stride0;  // elements between consecutive outer tiles
  int bn;                                     // B' rows per tile: a multiple of 32, at most 256
  int accumulate;
};

// KIND: operand type; OUT16: results rounded to the operand type (else raw 32-bit accumulators);
// K0 = 2 for kI8, 1 for the 16-bit kinds (what makes a 16-row tile row 32 bytes).
template <int KIND, bool OUT16>
__device__ __forceinline__ void mmt4d_body(const void* __restrict__ lhs, const void* __restrict__ rhs,
                                           void* __restrict__ out, Workspace* __restrict__ ws, Mmt4dShape s) {
  using T = KindTraits<KIND>;
  constexpr int kElem = T::kElemBytes;
  constexpr bool kDoubled = KIND == kI8;                 // K0 = 2: the product is computed on (row, k0) pairs
  constexpr int kRun = kMtRunBytes / kElem;              // elements per tile row: 32 (i8) or 16
  constexpr int kStepsPerStage = kRowBytes / kElem;      // K1 steps per stage: 128 (i8) or 64
  constexpr int kUmmaK = 32 / kElem;                     // K1 steps per tcgen05.mma: 32 or 16
  constexpr int kTilesA = kBM / kRun;                    // outer tiles of the left operand per CTA tile: 4 or 8
  constexpr int kOutBytes = OUT16 ? 2 : 4;
  static_assert(kStages * kStageBytes + 1024 + 256 <= kMtSmemBytes, "ring");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = smem_base + kStages * kStageBytes;
  auto full_bar = [&](int i) { return bars + 8u * i; };
  auto empty_bar = [&](int i) { return bars + 8u * (kStages + i); };
  auto tmem_full_bar = [&](int i) { return bars + 8u * (2 * kStages + i); };
  auto tmem_empty_bar = [&](int i) { return bars + 8u * (2 * kStages + 2 + i); };
  const uint32_t tmem_slot = bars + 8u * (2 * kStages + 4);
  uint8_t* smem_generic = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_generic + kStages * kStageBytes + 8 * (2 * kStages + 4));
  volatile uint32_t* abort_flag =
      reinterpret_cast<volatile uint32_t*>(smem_generic + kStages * kStageBytes + 8 * (2 * kStages + 4) + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // What the host checks, checked again: a misaligned 16-byte copy must never reach the hardware.
  const bool bad = s.M1 <= 0 || s.N1 <= 0 || s.K1 <= 0 || s.bn < 32 || s.bn > kMaxBN || (s.bn & 31) ||
                   (reinterpret_cast<uintptr_t>(lhs) & 15) || (reinterpret_cast<uintptr_t>(rhs) & 15) ||
                   (reinterpret_cast<uintptr_t>(out) & 31) || ((static_cast<int64_t>(s.lhs_stride0) * kElem) & 15) ||
                   ((static_cast<int64_t>(s.rhs_stride0) * kElem) & 15) ||
                   ((static_cast<int64_t>(s.out_stride0) * kOutBytes) & 31) || s.lhs_stride0 <= 0 || s.rhs_stride0 <= 0;
  // The next dispatch on the stream may be launched from here on; it orders itself on the device.
  grid_launch_dependents();
  if (bad) {
    grid_dependency_wait();
    if (threadIdx.x == 0) report(ws, kStatusBadArgument, 2);
    return;
  }

  const int tiles_b = s.bn / kRun;                                 // outer tiles of the right operand per CTA tile
  const int tiles_m = (s.M1 + kTilesA - 1) / kTilesA;
  const int tiles_n = (s.N1 + tiles_b - 1) / tiles_b;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (s.K1 + kStepsPerStage - 1) / kStepsPerStage;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(full_bar(i), kMtProducerThreads);
      mbar_init(empty_bar(i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tmem_full_bar(i), 1);
      mbar_init(tmem_empty_bar(i), 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, kTmemColumns);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // Launched early under a programmatic dependency: only this CTA's shared and tensor memory was
  // touched above; global memory is read and written only once the dispatch ahead is complete.
  grid_dependency_wait();

  // m fastest inside a column of tiles: consecutive CTAs share the right operand's tiles.
  auto tile_coords = [&](int t, int& tm, int& tn) {
    tn = t / tiles_m;
    tm = t - tn * tiles_m;
  };

  if (warp >= 8) {
    // ------------------------------ producers ---------------------------------
    // A stage is (kTilesA + tiles_b) outer tiles x kStepsPerStage rows of 32 bytes, in that order (the left
    // operand's 16 KiB first). Chunk c of 16 bytes: tile c / (2 * steps), row (c / 2) % steps, half c & 1;
    // consecutive threads copy consecutive chunks, i.e. consecutive global memory. (bn is a
    // multiple of 32, so the right operand's tile count is a multiple of the tile step.)
    const int pt = threadIdx.x - (kMtThreads - kMtProducerThreads);
    constexpr int kChunksPerTile = 2 * kStepsPerStage;                    // 256 (i8) or 128
    constexpr int kTileStep = kMtProducerThreads / kChunksPerTile;       // tiles the 256 threads cover at once: 1 or 2
    constexpr int kTileBytes = kStepsPerStage * kMtRunBytes;
    static_assert(kMtProducerThreads % kChunksPerTile == 0 && kTilesA % kTileStep == 0, "chunk mapping");
    const int j0 = pt / kChunksPerTile;
    const int within = pt % kChunksPerTile;
    const int row = within >> 1, half = within & 1;
    const uint32_t dst_off = row * kMtRunBytes + ((half ^ ((row >> 2) & 1)) << 4);
    const int64_t lhs_pitch = static_cast<int64_t>(s.lhs_stride0) * kElem;
    const int64_t rhs_pitch = static_cast<int64_t>(s.rhs_stride0) * kElem;
    const uint8_t* lhs_bytes = static_cast<const uint8_t*>(lhs);
    const uint8_t* rhs_bytes = static_cast<const uint8_t*>(rhs);
    uint32_t it = 0, arrived = 0;
    bool ok = true;
    // the full barrier of stage `arrived` is told once this thread's copies into it have landed
    auto retire = [&]() {
      fence_proxy_async_smem();  // the tensor core reads these bytes through the async proxy
      mbar_arrive(full_bar(arrived % kStages));
      ++arrived;
    };
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int tm, tn;
      tile_coords(t, tm, tn);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int st = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (!mbar_wait(empty_bar(st), ph ^ 1, abort_flag)) {
          if (pt == 0) report(ws, kStatusTimeoutEmpty, it);
          *abort_flag = 1;
          ok = false;
          break;
        }
        // This thread's chunk sits at the same (row, half) of every outer tile it copies: tiles j0,
        // j0 + kTileStep, ... of the stage; only the tile's base address changes from copy to copy.
        const int k1 = kb * kStepsPerStage + row;
        const bool k_ok = k1 < s.K1;
        const int64_t k_off = static_cast<int64_t>(k1) * kMtRunBytes + half * 16;
        uint32_t dst = smem_base + st * kStageBytes + j0 * kTileBytes + dst_off;
        {
          const int first = tm * kTilesA + j0;
          const uint8_t* src = lhs_bytes + static_cast<int64_t>(first) * lhs_pitch + k_off;
#pragma unroll
          for (int j = 0; j < kTilesA / kTileStep; ++j) {
            const bool in_range = k_ok && first + j * kTileStep < s.M1;
            cp_async_16(dst, in_range ? src : lhs_bytes, in_range ? 16u : 0u);
            src += kTileStep * lhs_pitch;
            dst += kTileStep * kTileBytes;
          }
        }
        {
          const int first = tn * tiles_b + j0;
          const uint8_t* src = rhs_bytes + static_cast<int64_t>(first) * rhs_pitch + k_off;
          for (int j = j0; j < tiles_b; j += kTileStep) {
            const bool in_range = k_ok && tn * tiles_b + j < s.N1;
            cp_async_16(dst, in_range ? src : rhs_bytes, in_range ? 16u : 0u);
            src += kTileStep * rhs_pitch;
            dst += kTileStep * kTileBytes;
          }
        }
        cp_async_commit();
        if (it - arrived >= kMtCopyDepth - 1) {
          cp_async_wait_group<kMtCopyDepth - 1>();
          retire();
        }
      }
    }
    cp_async_wait_group<0>();
    if (ok)
      while (arrived < it) retire();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_instr_desc(T::kCFormat, T::kFormat, T::kFormat, 1u, 1u, kBM, s.bn);
      // One outer tile is kStepsPerStage rows of 32 bytes: the next 32 rows-of-the-product start there
      // (leading offset); eight K1 steps are 256 bytes (stride offset).
      constexpr uint32_t kLbo = kStepsPerStage * kMtRunBytes;
      constexpr uint32_t kSbo = 8 * kMtRunBytes;
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local_tile) {
        const int buf = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait(tmem_empty_bar(buf), acc_ph ^ 1, abort_flag)) {
          report(ws, kStatusTimeoutTmemEmpty, local_tile);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kMaxBN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int st = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(full_bar(st), ph, abort_flag)) {
            report(ws, kStatusTimeoutFull, it);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_src = smem_base + st * kStageBytes;
          const uint32_t b_src = a_src + kAStageBytes;
#pragma unroll
          for (int k = 0; k < kStepsPerStage / kUmmaK; ++k) {
            const uint64_t a_desc = make_smem_desc_sw32(a_src + k * (kUmmaK * kMtRunBytes), kLbo, kSbo);
            const uint64_t b_desc = make_smem_desc_sw32(b_src + k * (kUmmaK * kMtRunBytes), kLbo, kSbo);
            const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
            if constexpr (KIND == kI8) {
              mma_i8_ss(d_tmem, a_desc, b_desc, idesc, acc);
            } else {
              mma_f16_ss(d_tmem, a_desc, b_desc, idesc, acc);
            }
          }
          tc_commit(empty_bar(st));
        }
        if (ok) tc_commit(tmem_full_bar(buf));
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t local_tile = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++local_tile) {
      int tm, tn;
      tile_coords(t, tm, tn);
      const int buf = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(tmem_full_bar(buf), acc_ph, abort_flag))) {
        if (lane == 0) {
          report(ws, kStatusTimeoutTmemFull, local_tile);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after_sync();
      const uint32_t acc_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kMaxBN;
      if constexpr (kDoubled) {
        // This warp's 32 accumulator rows are the (m0, k0) pairs of one outer tile m1; a chunk of 32
        // columns is the (n0, k0') pairs of one outer tile n1. Lane 2 * m0 + k0 holds C'[(m0, k0), :]:
        // the even lane ends up with columns n0 = 0..7 of row m0, the odd lane with n0 = 8..15.
        const int m1 = tm * kTilesA + q;
        const int m0 = lane >> 1;
        const bool odd = lane & 1;
        for (int c = 0; c < tiles_b; ++c) {
          const int n1 = tn * tiles_b + c;
          if (n1 >= s.N1) break;  // warp-uniform
          uint32_t v[32];
          tmem_ld_32x32(acc_addr + c * 32, v);
          tc_wait_ld();
          uint32_t r[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t send = odd ? v[2 * i + 1] : v[16 + 2 * i];
            const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 1);
            r[i] = (odd ? v[17 + 2 * i] : v[2 * i]) + recv;
          }
          if (m1 < s.M1) {
            uint32_t* dst = reinterpret_cast<uint32_t*>(out) + static_cast<int64_t>(m1) * s.out_stride0 +
                            (static_cast<int64_t>(n1) * 16 + m0) * 16 + (odd ? 8 : 0);
            if (s.accumulate) {
              const uint4 o0 = ld_global_128(dst), o1 = ld_global_128(dst + 4);
              r[0] += o0.x, r[1] += o0.y, r[2] += o0.z, r[3] += o0.w;
              r[4] += o1.x, r[5] += o1.y, r[6] += o1.z, r[7] += o1.w;
            }
            st_global_256(dst, r[0], r[1], r[2], r[3], r[4], r[5], r[6], r[7]);
          }
        }
      } else {
        // Lane = row m0 of outer tile m1 (two tiles per warp); a chunk of 32 columns is two outer tiles n1.
        const int m1 = tm * kTilesA + q * 2 + (lane >> 4);
        const int m0 = lane & 15;
        for (int c = 0; c < s.bn / 32; ++c) {
          if (tn * tiles_b + 2 * c >= s.N1) break;  // warp-uniform
          uint32_t v[32];
          tmem_ld_32x32(acc_addr + c * 32, v);
          tc_wait_ld();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int n1 = tn * tiles_b + 2 * c + h;
            if (m1 >= s.M1 || n1 >= s.N1) continue;
            const int64_t at = static_cast<int64_t>(m1) * s.out_stride0 + (static_cast<int64_t>(n1) * 16 + m0) * 16;
            if constexpr (OUT16) {
              uint32_t w[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float f0 = __uint_as_float(v[16 * h + 2 * j]), f1 = __uint_as_float(v[16 * h + 2 * j + 1]);
                w[j] = pack_16x2<KIND>(f0, f1);
              }
              st_global_256(reinterpret_cast<uint16_t*>(out) + at, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
            } else {
              uint32_t* dst = reinterpret_cast<uint32_t*>(out) + at;
#pragma unroll
              for (int g = 0; g < 2; ++g) {
                uint32_t r[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) r[j] = v[16 * h + 8 * g + j];
                if (s.accumulate) {
                  const uint4 o0 = ld_global_128(dst + 8 * g), o1 = ld_global_128(dst + 8 * g + 4);
                  const uint32_t o[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
#pragma unroll
                  for (int j = 0; j < 8; ++j) r[j] = __float_as_uint(__uint_as_float(o[j]) + __uint_as_float(r[j]));
                }
                st_global_256(dst + 8 * g, r[0], r[1], r[2], r[3], r[4], r[5], r[6], r[7]);
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(buf));
    }
  }

  // Teardown: everyone meets here, also after an abort; copies may still be landing then.
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
  }
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemColumns);
  }
}

}  // namespace b200

// Bindings: lhs, rhs, out, workspace (status words). Constants: M1, N1, K1, the three stride0 values in
// elements, and the tile width with the ACCUMULATE flag in bit 16.
#define B200_MMT4D_EXPORT(NAME, KIND, OUT16)                                                                           \
  extern "C" __global__ void __launch_bounds__(b200::kMtThreads, 1)                                                    \
      NAME(const void* lhs, const void* rhs, void* out, void* ws, int M1, int N1, int K1, int lhs_stride0,              \
           int rhs_stride0, int out_stride0, int bn_flags) {                                                            \
    b200::Mmt4dShape s{M1, N1, K1, lhs_stride0, rhs_stride0, out_stride0, bn_flags & 0xffff, (bn_flags >> 16) & 1};    \
    b200::mmt4d_body<KIND, OUT16>(lhs, rhs, out, static_cast<b200::Workspace*>(ws), s);                                \
  }
B200_MMT4D_EXPORT(b200_mmt4d_s8s8s32, b200::kI8, false)
B200_MMT4D_EXPORT(b200_mmt4d_f16f16f32, b200::kF16, false)
B200_MMT4D_EXPORT(b200_mmt4d_f16f16f16, b200::kF16, true)
B200_MMT4D_EXPORT(b200_mmt4d_bf16bf16f32, b200::kBF16, false)
B200_MMT4D_EXPORT(b200_mmt4d_bf16bf16bf16, b200::kBF16, true)
#undef B200_MMT4D_EXPORT
