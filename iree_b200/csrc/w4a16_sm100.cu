// Fused "dequantise int4 weights, then contract" dispatch (group-wise scales, no zero point):
//   w_f16[n,k] = f16( f16(sext(wq[n,k])) * scale[n, k/128] )
//   out[m,n]   = f16( sum_k f32(a[m,k]) * f32(w_f16[n,k]) )
// wq is [N, K/2] bytes, element 2i in the low nibble of byte i; scales are [N, K/128] f16;
// a is [M, K] f16; out is f16 with row pitch `ldo` and column offset `n_off` (so a rank that
// owns a slice of N can write straight into the full-width result).
//
// Three kernels:
//   b200_w4a16_decode_m8 / _m16  M <= 8 / 16: HBM-bound weight streaming (w4a16_decode.cuh). 16 warps
//       each own a 256-wide chunk of a 4096-wide K slice and keep the activations of that chunk in
//       registers for the whole kernel; weights go global -> shared (bulk copies into a 4-stage
//       ring, 16 rows per tile) -> f16 fragments -> mma.sync (f32 accumulate); the per-group scale
//       is applied to the f32 group sum. K beyond 4096 is split over CTAs; the last CTA to finish
//       a tile adds the slices' f32 partial tiles from a global scratch.
//   b200_w4a16_gemm             larger M: tcgen05. Raw int4 tiles and activation tiles arrive by
//       TMA; 8 warps expand the weights to f16 (exactly the dequant arithmetic above) into the
//       128-byte-swizzled operand layout; one thread issues kind::f16 MMAs into TMEM. 128-row
//       tiles, or 256-row tiles sharing one expanded weight tile when M >= 256.
//   b200_w4a16_generic          any shape with K % group == 0: one thread per output.
#include <cuda_fp16.h>
#include <stdint.h>

#include "sm100_ptx.cuh"
#include "w4a16_decode.cuh"

namespace b200 {

// =============================================================================================
// tcgen05 kernel for larger M
// =============================================================================================
constexpr int kW4BM = 128;
constexpr int kW4MaxBN = 128;                       // tile width: a multiple of 16 up to this
constexpr int kW4AStageBytes = kW4BM * 128;         // 16 KiB: 128 rows x 64 f16
constexpr int kW4BStageBytes = kW4MaxBN * 128;      // 16 KiB: the expanded weights of one K block
constexpr int kW4RawStageBytes = kW4MaxBN * 64;     // 8 KiB: 128 rows x 128 int4 = one scale group
constexpr int kW4Threads = 512;
constexpr int kW4DequantWarps = 8;                  // two groups of four, alternating K blocks
// Two variants, chosen from M: 128 x bn tiles below M = 256 (weights stream once: many raw stages
// in flight), and 256 x bn tiles from there on, i.e. two 128-row accumulators sharing one expanded
// weight tile, so that every weight is expanded half as often per flop. Both fill the same shared
// memory: 5 x 32 KiB + 8 x 8 KiB, or 4 x 48 KiB + 4 x 8 KiB.
__host__ __device__ constexpr bool w4_tall_variant(int M) { return M >= 256; }
constexpr int kW4Stages = 5, kW4RawStages = 8;
constexpr int kW4TallStages = 4, kW4TallRawStages = 4;
constexpr int kW4SmemBytes = 1024 + 224 * 1024 + 256;
static_assert(kW4Stages * (kW4AStageBytes + kW4BStageBytes) + kW4RawStages * kW4RawStageBytes <= 224 * 1024, "128-row variant");
static_assert(kW4TallStages * (2 * kW4AStageBytes + kW4BStageBytes) + kW4TallRawStages * kW4RawStageBytes <= 224 * 1024, "256-row variant");
static_assert(kW4SmemBytes <= 232448, "per-CTA shared memory limit");

struct alignas(128) W4Workspace {
  uint8_t map_a[128];    // f16 [M, K], 128-byte swizzle, box 64 x 128
  uint8_t map_w[128];    // u8 [N, K/2], 64-byte swizzle, box 64 x bn
  uint8_t map_aux[128];
  uint32_t status[32];
};

__device__ __forceinline__ void w4_report(W4Workspace* ws, uint32_t code, uint32_t info) {
  if (atomicCAS(&ws->status[0], 0u, code) == 0u) ws->status[1] = info;
}

template <bool TALL>
__device__ __forceinline__ void w4gemm_body(const __half* __restrict__ scales, __half* __restrict__ out,
                                            W4Workspace* __restrict__ ws, int M, int N, int K, int ldo, int n_off,
                                            int bn) {
  constexpr int kHalves = TALL ? 2 : 1;                        // 128-row accumulators per tile
  constexpr int kTileRows = kHalves * kW4BM;
  constexpr int kAStageBytes = kHalves * kW4AStageBytes;       // the B tile follows it in the stage
  constexpr int kStageBytes = kAStageBytes + kW4BStageBytes;
  constexpr int kAccColumns = kW4MaxBN;                        // TMEM columns per accumulator
  constexpr int kS = TALL ? kW4TallStages : kW4Stages;         // f16 operand stages
  constexpr int kRS = TALL ? kW4TallRawStages : kW4RawStages;  // raw int4 stages, one scale group each
  constexpr int kRawBytes = kW4RawStageBytes;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t raw_base = smem_base + kS * kStageBytes;
  const uint32_t bars = raw_base + kRS * kRawBytes;
  uint8_t* bars_gen = smem_gen + kS * kStageBytes + kRS * kRawBytes;
  // barriers: full[stages], empty[stages], raw_full[raw stages], raw_empty[raw stages], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](int i) { return bars + 8u * i; };
  auto empty_bar = [&](int i) { return bars + 8u * (kS + i); };
  auto raw_full_bar = [&](int i) { return bars + 8u * (2 * kS + i); };
  auto raw_empty_bar = [&](int i) { return bars + 8u * (2 * kS + kRS + i); };
  auto tmem_full_bar = [&](int i) { return bars + 8u * (2 * kS + 2 * kRS + i); };
  auto tmem_empty_bar = [&](int i) { return bars + 8u * (2 * kS + 2 * kRS + 2 + i); };
  const uint32_t tmem_slot = bars + 8u * (2 * kS + 2 * kRS + 4);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * (2 * kS + 2 * kRS + 4));
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * (2 * kS + 2 * kRS + 4) + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const bool bad = M <= 0 || N <= 0 || K <= 0 || (K & 127) || bn < 16 || bn > kAccColumns || (bn & 15);
  // The next dispatch on the stream may be launched from here on; it orders itself on the device.
  grid_launch_dependents();
  if (bad) {
    grid_dependency_wait();
    if (threadIdx.x == 0) w4_report(ws, kStatusBadArgument, 0);
    return;
  }
  const int tiles_m = (M + kTileRows - 1) / kTileRows;
  const int tiles_n = (N + bn - 1) / bn;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = K / 64;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kS; ++i) {
      mbar_init(full_bar(i), 1 + kW4DequantWarps / 2);  // TMA producer + the K block's dequant group
      mbar_init(empty_bar(i), 1);
    }
    for (int i = 0; i < kRS; ++i) {
      mbar_init(raw_full_bar(i), 1);
      mbar_init(raw_empty_bar(i), kW4DequantWarps);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tmem_full_bar(i), 1);
      mbar_init(tmem_empty_bar(i), 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // Launched early under a programmatic dependency: only this CTA's shared and tensor memory was
  // touched above; global memory is read and written only once the dispatch ahead is complete.
  grid_dependency_wait();

  auto tile_coords = [&](int t, int& tm, int& tn) {
    tn = t / tiles_m;
    tm = t - tn * tiles_m;
  };

  if (warp == 0) {
    // -------- TMA producer of the activation tiles: one per K block -----------------------------
    if (lane == 0) {
      tensormap_fence_acquire(ws->map_a);
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, tm, tn);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int st = it % kS;
          const uint32_t ph = (it / kS) & 1;
          if (!mbar_wait(empty_bar(st), ph ^ 1, abort_flag)) {
            w4_report(ws, kStatusTimeoutEmpty, it);
            *abort_flag = 1;
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(full_bar(st), kAStageBytes);
#pragma unroll
          for (int h = 0; h < kHalves; ++h)
            tma_load_3d(smem_base + st * kStageBytes + h * kW4AStageBytes, ws->map_a, full_bar(st), kb * 64,
                        tm * kTileRows + h * kW4BM, 0);
        }
      }
    }
  } else if (warp == 3) {
    // -------- TMA producer of the raw weights: one scale group (128 K) per raw stage. It runs as
    // far ahead as the raw ring allows, also into the next tile, whatever the operand stages do.
    if (lane == 0) {
      tensormap_fence_acquire(ws->map_w);
      uint32_t raw_it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, tm, tn);
        for (int g = 0; g < (num_kb >> 1); ++g, ++raw_it) {
          const int rs = raw_it % kRS;
          const uint32_t rph = (raw_it / kRS) & 1;
          if (!mbar_wait(raw_empty_bar(rs), rph ^ 1, abort_flag)) {
            w4_report(ws, kStatusTimeoutEmpty, 0x10000u | raw_it);
            *abort_flag = 1;
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(raw_full_bar(rs), bn * 64);
          tma_load_3d(raw_base + rs * kRawBytes, ws->map_w, raw_full_bar(rs), g * 64, tn * bn, 0);
        }
      }
    }
  } else if (warp == 1) {
    // -------- MMA issuer ---------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_instr_desc(1u, 0u, 0u, 0u, 0u, kW4BM, bn);
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local_tile) {
        const int buf = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait(tmem_empty_bar(buf), acc_ph ^ 1, abort_flag)) {
          w4_report(ws, kStatusTimeoutTmemEmpty, local_tile);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kHalves * kAccColumns;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int st = it % kS;
          const uint32_t ph = (it / kS) & 1;
          if (!mbar_wait(full_bar(st), ph, abort_flag)) {
            w4_report(ws, kStatusTimeoutDequant, it);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_src = smem_base + st * kStageBytes;
          const uint32_t b_src = a_src + kAStageBytes;
#pragma unroll
          for (int h = 0; h < kHalves; ++h)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint64_t a_desc = make_smem_desc(a_src + h * kW4AStageBytes + k * 32, 16, 1024);
              const uint64_t b_desc = make_smem_desc(b_src + k * 32, 16, 1024);
              mma_f16_ss(d_tmem + h * kAccColumns, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
          tc_commit(empty_bar(st));
        }
        if (ok) tc_commit(tmem_full_bar(buf));
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // -------- epilogue -----------------------------------------------------------------------
    const int qd = warp & 3;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && ((ldo * 2) % 16 == 0) && ((n_off * 2) % 16 == 0);
    uint32_t local_tile = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++local_tile) {
      int tm, tn;
      tile_coords(t, tm, tn);
      const int buf = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(tmem_full_bar(buf), acc_ph, abort_flag))) {
        if (lane == 0) {
          w4_report(ws, kStatusTimeoutTmemFull, local_tile);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after_sync();
      for (int h = 0; h < kHalves; ++h) {
      const int row = tm * kTileRows + h * kW4BM + qd * 32 + lane;
      for (int c = 0; c < bn; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(qd * 32) << 16) + (buf * kHalves + h) * kAccColumns + c, v);
        tc_wait_ld();
        const int col0 = tn * bn + c;
        if (row < M && col0 < N) {
          __half* dst = out + static_cast<size_t>(row) * ldo + n_off + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (c + j >= bn) break;  // bn is a multiple of 16: the tile ends inside this 32-column read
            if (vec_ok && col0 + j + 7 < N) {
              uint4 o;
              o.x = as_u32(__floats2half2_rn(__uint_as_float(v[j]), __uint_as_float(v[j + 1])));
              o.y = as_u32(__floats2half2_rn(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])));
              o.z = as_u32(__floats2half2_rn(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5])));
              o.w = as_u32(__floats2half2_rn(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7])));
              *reinterpret_cast<uint4*>(dst + j) = o;
            } else {
              for (int e = 0; e < 8; ++e)
                if (col0 + j + e < N) dst[j + e] = __float2half_rn(__uint_as_float(v[j + e]));
            }
          }
        }
      }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(buf));
    }
  } else if (warp >= 8) {
    // -------- dequant: raw int4 (64-byte swizzled rows) -> f16 K-major 128-byte swizzled tile -----
    // A thread expands one weight row of one K block: 32 raw bytes in, one 128-byte operand row
    // out. Two groups of 128 threads take alternate K blocks, so that one group's stores and
    // proxy fence drain while the other group computes.
    const int td = threadIdx.x - 256;
    const int r = td & 127;
    const int grp = td >> 7;
    constexpr int kStep = 2;
    const int groups = K >> 7;
    // Scales of eight consecutive groups arrive as one 16-byte load, one load ahead of their use.
    const bool vec_scales = (groups & 7) == 0 && (reinterpret_cast<uintptr_t>(scales) & 15) == 0;
    uint32_t it_base = 0, raw_it_base = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, it_base += num_kb, raw_it_base += num_kb >> 1) {
      int tm, tn;
      tile_coords(t, tm, tn);
      const int n = tn * bn + r;
      const bool row_live = r < bn;
      const bool has_scales = row_live && n < N;
      const __half* srow = scales + static_cast<size_t>(n < N ? n : 0) * groups;
      __half2 s2 = __half2half2(__float2half_rn(0.f));
      uint4 sc_cur = make_uint4(0, 0, 0, 0), sc_next = make_uint4(0, 0, 0, 0);
      __half next_scale = __float2half_rn(0.f);
      if (has_scales) {
        if (vec_scales) sc_next = *reinterpret_cast<const uint4*>(srow);
        else next_scale = srow[0];
      }
      for (int kb = grp; kb < num_kb; kb += kStep) {
        const uint32_t it = it_base + kb;
        const uint32_t raw_it = raw_it_base + (kb >> 1);
        const int rs = raw_it % kRS;
        {
          const uint32_t rph = (raw_it / kRS) & 1;
          if (!__all_sync(0xffffffffu, mbar_wait(raw_full_bar(rs), rph, abort_flag))) {
            if (lane == 0) {
              w4_report(ws, kStatusTimeoutFull, 0x10000u | raw_it);
              *abort_flag = 1;
            }
            ok = false;
            break;
          }
          const int g = kb >> 1;
          if (vec_scales) {
            if ((g & 7) == 0) {
              sc_cur = sc_next;
              if (has_scales && g + 8 < groups) sc_next = *reinterpret_cast<const uint4*>(srow + g + 8);
            }
            const uint32_t word = (g & 4) ? ((g & 2) ? sc_cur.w : sc_cur.z) : ((g & 2) ? sc_cur.y : sc_cur.x);
            s2 = as_half2(__byte_perm(word, 0u, (g & 1) ? 0x3232u : 0x1010u));
          } else {
            s2 = __half2half2(next_scale);
            if (has_scales && g + 1 < groups) next_scale = srow[g + 1];
          }
        }
        const int st = it % kS;
        const uint32_t ph = (it / kS) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(empty_bar(st), ph ^ 1, abort_flag))) {
          if (lane == 0) {
            w4_report(ws, kStatusTimeoutEmpty, 0x20000u | it);
            *abort_flag = 1;
          }
          ok = false;
          break;
        }
        if (row_live) {
          // Raw stage: row r is 64 bytes; its four 16-byte chunks are XOR-swizzled by (r / 2) % 4.
          const uint8_t* raw_row = smem_gen + kS * kStageBytes + rs * kRawBytes + r * 64;
          uint8_t* b_row = smem_gen + st * kStageBytes + kAStageBytes + r * 128;
          const int sw_raw = (r >> 1) & 3, sw_b = r & 7;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int chunk = (kb & 1) * 2 + c;  // 16-byte chunk of the 64-byte raw row
            const uint4 w = *reinterpret_cast<const uint4*>(raw_row + ((chunk ^ sw_raw) << 4));
            const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              __half2 qv[4];
              unpack8_ordered(words[i], qv);
              uint4 o;
              o.x = as_u32(__hmul2(qv[0], s2));  // f16(w) * scale, one rounding: the reference's dequant
              o.y = as_u32(__hmul2(qv[1], s2));
              o.z = as_u32(__hmul2(qv[2], s2));
              o.w = as_u32(__hmul2(qv[3], s2));
              const int out_chunk = c * 4 + i;  // 8 f16 = 16 bytes of the 128-byte operand row
              *reinterpret_cast<uint4*>(b_row + ((out_chunk ^ sw_b) << 4)) = o;
            }
          }
        }
        fence_proxy_async_smem();  // make the generic-proxy writes visible to the tensor core
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(full_bar(st));
          mbar_arrive(raw_empty_bar(rs));
        }
      }
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

// Binding 4 is the dispatch's workspace: the tensor map over the weights (needed when K spans more
// than one 4096-wide slice) at byte 0, status words at byte 384 (words 16..19 note which weights,
// N and K the map was built for), the slice-reduction scratch (DecodeScratchLayout) from byte 512 on.
extern "C" __global__ void __launch_bounds__(kDecodeThreads, 1)
    b200_w4a16_decode_m8(const __half* a, const uint8_t* wq, const __half* scales, __half* out, uint8_t* ws, int M,
                         int N, int K, int ldo, int n_off) {
  decode_body<1>(a, wq, scales, out, ws + 512, reinterpret_cast<uint32_t*>(ws + 384), ws, true, M, N, K, ldo, n_off);
}
extern "C" __global__ void __launch_bounds__(kDecodeThreads, 1)
    b200_w4a16_decode_m16(const __half* a, const uint8_t* wq, const __half* scales, __half* out, uint8_t* ws, int M,
                          int N, int K, int ldo, int n_off) {
  decode_body<2>(a, wq, scales, out, ws + 512, reinterpret_cast<uint32_t*>(ws + 384), ws, true, M, N, K, ldo, n_off);
}

extern "C" __global__ void __launch_bounds__(kW4Threads, 1)
    b200_w4a16_gemm(const __half* scales, __half* out, void* ws, int M, int N, int K, int ldo, int n_off, int bn) {
  if (w4_tall_variant(M))
    w4gemm_body<true>(scales, out, reinterpret_cast<W4Workspace*>(ws), M, N, K, ldo, n_off, bn);
  else
    w4gemm_body<false>(scales, out, reinterpret_cast<W4Workspace*>(ws), M, N, K, ldo, n_off, bn);
}

// Any M, N and any K that is a multiple of the (even) group size. One thread per output
// element, sequential over K like the reference's generated loop nest.
extern "C" __global__ void __launch_bounds__(256)
    b200_w4a16_generic(const __half* a, const uint8_t* wq, const __half* scales, __half* out, int M, int N, int K,
                       int group, int ldo, int n_off) {
  const int n = blockIdx.x * 256 + threadIdx.x;
  const int m = blockIdx.y;
  if (n >= N || m >= M) return;
  const int G = K / group;
  float acc = 0.f;
  for (int gi = 0; gi < G; ++gi) {
    const __half s = scales[static_cast<size_t>(n) * G + gi];
    for (int k = gi * group; k < (gi + 1) * group; ++k) {
      const uint8_t byte = wq[static_cast<size_t>(n) * (K >> 1) + (k >> 1)];
      const int w = sext4((k & 1) ? (byte >> 4) : (byte & 0xf));
      const __half wd = __hmul(__int2half_rn(w), s);
      acc += __half2float(a[static_cast<size_t>(m) * K + k]) * __half2float(wd);
    }
  }
  out[static_cast<size_t>(m) * ldo + n_off + n] = __float2half_rn(acc);
}
