// The same contraction family as contraction_sm100.cu with CTAs working in pairs
// (thread-block cluster of two, tcgen05 cta_group::2): one 256 x BN output tile per pair, each
// CTA holding its own 128 rows of A and HALF of the B tile, the tensor cores of both SMs
// exchanging the B halves. Per flop this halves the B traffic into and out of shared memory,
// which is what limits the single-CTA kernel.
//
//   both CTAs   warp 0: TMA producer (own A rows, own half of B) into a 6-stage ring; every
//               completion is reported to the LEADER's "full" barrier
//   leader      warp 1: one thread issues tcgen05.mma.cta_group::2 (M = 256) and commits
//               "stage free" / "accumulator full" to the barriers of both CTAs
//   both CTAs   warp 2: TMEM allocation (cta_group::2); warps 4-7: epilogue of their own 128 rows;
//               "accumulator drained" is reported to the leader's barrier
//
// Launch: plain cuLaunchKernel with an even grid; the pairing comes from __cluster_dims__.
// This file is compiled in one translation unit after contraction_sm100.cu and uses its
// Workspace, KindTraits, store_row_chunk and report definitions. No TMA load here uses cluster
// multicast; the only cluster-wide signal is the tcgen05.commit arrival.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace b200 {

constexpr int kPairStages = 6;
constexpr int kPairBStageBytes = (kMaxBN / 2) * kRowBytes;             // 16 KiB: half of the B tile
constexpr int kPairStageBytes = kAStageBytes + kPairBStageBytes;       // 32 KiB
constexpr int kPairSmemBytes = 1024 + kPairStages * kPairStageBytes + kOutStageBytes + 256;  // = kGemmSmemBytes
static_assert(kPairSmemBytes <= kGemmSmemBytes, "the pair exports are launched with the 1-CTA exports' shared memory");

template <int KIND, int EPI>
__device__ __forceinline__ void gemm_pair_body(void* __restrict__ c_ptr, const float* __restrict__ row_scale,
                                               const float* __restrict__ col_scale, Workspace* __restrict__ ws,
                                               GemmShape s) {
  using T = KindTraits<KIND>;
  constexpr int kElem = T::kElemBytes;
  constexpr int kBK = kRowBytes / kElem;
  constexpr int kUmmaK = 32 / kElem;
  constexpr int kChunkN = kRowBytes / kElem;

  extern __shared__ uint8_t smem_raw[];
  __shared__ alignas(128) uint8_t out_map_stage[128];  // where the result's tensor map is assembled
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t out_stage = smem_base + kPairStages * kPairStageBytes;  // epilogue staging tiles, as in the 1-CTA kernel
  const uint32_t bars = out_stage + kOutStageBytes;
  auto full_bar = [&](int i) { return bars + 8u * i; };
  auto empty_bar = [&](int i) { return bars + 8u * (kPairStages + i); };
  auto tmem_full_bar = [&](int i) { return bars + 8u * (2 * kPairStages + i); };
  auto tmem_empty_bar = [&](int i) { return bars + 8u * (2 * kPairStages + 2 + i); };
  const uint32_t tmem_slot = bars + 8u * (2 * kPairStages + 4);
  uint8_t* bars_gen = smem_raw + (smem_base - smem_u32(smem_raw)) + kPairStages * kPairStageBytes + kOutStageBytes;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * (2 * kPairStages + 4));
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * (2 * kPairStages + 4) + 4);
  // written by the epilogue warps only, before the barrier at which all four read it: they leave together
  volatile uint32_t* epilogue_abort = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * (2 * kPairStages + 4) + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int half_bn = s.bn >> 1;

  // Both CTAs of a pair take the same decision, so an early return cannot strand a partner.
  const bool bad = s.M <= 0 || s.N <= 0 || s.K <= 0 || s.batch <= 0 || s.bn < 64 || s.bn > kMaxBN || (s.bn & 63) ||
                   (s.K * kElem) % 16 != 0 || (gridDim.x & 1) ||
                   (s.b_layout == kBLayoutKN && ((s.N * kElem) % 16 != 0 || half_bn % kChunkN != 0));
  grid_launch_dependents();
  if (bad) {
    grid_dependency_wait();
    if (threadIdx.x == 0) report(ws, kStatusBadArgument, 1);
    return;
  }

  const int tiles_m = (s.M + 2 * kBM - 1) / (2 * kBM);
  const int tiles_n = (s.N + s.bn - 1) / s.bn;
  const int tiles_per_batch = tiles_m * tiles_n;
  const int num_tiles = tiles_per_batch * s.batch;
  const int num_kb = (s.K + kBK - 1) / kBK;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kPairStages; ++i) {
      mbar_init(full_bar(i), 1);   // the leader's expect_tx arrival; bytes come from both CTAs
      mbar_init(empty_bar(i), 1);  // the leader's commit, delivered to both CTAs
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tmem_full_bar(i), 1);
      mbar_init(tmem_empty_bar(i), 8);  // four epilogue warps in each CTA (used in the leader only)
    }
    *abort_flag = 0;
    *epilogue_abort = 0;
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc_pair(tmem_slot, kTmemColumns);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs exist before anything is signalled across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  grid_dependency_wait();  // as in the 1-CTA kernel: global memory is touched only below this line

  auto tile_coords = [&](int t, int& b, int& tm, int& tn) {
    b = t / tiles_per_batch;
    int r = t - b * tiles_per_batch;
    tn = r / tiles_m;
    tm = r - tn * tiles_m;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      tensormap_fence_acquire(ws->map_a);
      tensormap_fence_acquire(ws->map_b);
      const uint32_t pair_tx = 2u * (kAStageBytes + half_bn * kRowBytes);
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int b, tm, tn;
        tile_coords(t, b, tm, tn);
        const int row0 = tm * 2 * kBM + rank * kBM;
        const int col0 = tn * s.bn + rank * half_bn;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int st = it % kPairStages;
          const uint32_t ph = (it / kPairStages) & 1;
          if (!mbar_wait(empty_bar(st), ph ^ 1, abort_flag)) {
            report(ws, kStatusTimeoutEmpty, it);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + st * kPairStageBytes;
          const uint32_t b_dst = a_dst + kAStageBytes;
          const uint32_t leader_full = map_to_cta(full_bar(st), 0);
          if (rank == 0) mbar_arrive_expect_tx(full_bar(st), pair_tx);
          tma_load_3d_pair(a_dst, ws->map_a, leader_full, kb * kBK, row0, b);
          if (s.b_layout == kBLayoutNK) {
            tma_load_3d_pair(b_dst, ws->map_b, leader_full, kb * kBK, col0, b);
          } else {
            for (int c = 0; c < half_bn / kChunkN; ++c)
              tma_load_3d_pair(b_dst + c * (kBK * kRowBytes), ws->map_b, leader_full, col0 + c * kChunkN, kb * kBK, b);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader only) ------------------------------
    if (lane == 0 && rank == 0) {
      const uint32_t b_major = (s.b_layout == kBLayoutKN) ? 1u : 0u;
      const uint32_t idesc = make_instr_desc(T::kCFormat, T::kFormat, T::kFormat, 0u, b_major, 2 * kBM, s.bn);
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs, ++local_tile) {
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
          const int st = it % kPairStages;
          const uint32_t ph = (it / kPairStages) & 1;
          if (!mbar_wait(full_bar(st), ph, abort_flag)) {
            report(ws, kStatusTimeoutFull, it);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_src = smem_base + st * kPairStageBytes;
          const uint32_t b_src = a_src + kAStageBytes;
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint64_t a_desc = make_smem_desc(a_src + k * 32, 16, 1024);
            const uint64_t b_desc = (s.b_layout == kBLayoutNK)
                                        ? make_smem_desc(b_src + k * 32, 16, 1024)
                                        : make_smem_desc(b_src + k * (kUmmaK * kRowBytes), kBK * kRowBytes, 1024);
            const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
            if constexpr (KIND == kI8) {
              mma_i8_ss_pair(d_tmem, a_desc, b_desc, idesc, acc);
            } else {
              mma_f16_ss_pair(d_tmem, a_desc, b_desc, idesc, acc);
            }
          }
          tc_commit_pair(empty_bar(st));  // frees the stage in both CTAs
        }
        if (ok) tc_commit_pair(tmem_full_bar(buf));
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue (both CTAs, own 128 rows) ----------------------
    const int q = warp & 3;
    constexpr int kOutBytes = (EPI == kEpiRaw) ? 4 : 2;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(c_ptr) % 16 == 0) && ((s.N * kOutBytes) % 16 == 0);
    const bool wide_ok = (reinterpret_cast<uintptr_t>(c_ptr) % 32 == 0) && ((s.N * kOutBytes) % 32 == 0);
    // Results leave through the TMA unit when it can address their rows (the 1-CTA kernel's epilogue: 128
    // bytes of every row staged in a swizzled tile, one store per tile, the map assembled from map_a; both
    // CTAs of every pair publish the same 128 bytes to the workspace's third slot).
    constexpr int kPassCols = 128 / kOutBytes;
    const bool tma_out = vec_ok && (s.bn % kPassCols) == 0;
    const bool store_thread = threadIdx.x == 128;
    if (tma_out && q == 0) {
      reinterpret_cast<uint32_t*>(out_map_stage)[lane] = reinterpret_cast<const uint32_t*>(ws->map_a)[lane];
      __syncwarp();
      if (lane == 0) {
        const uint32_t m = smem_u32(out_map_stage);
        const uint64_t pitch = static_cast<uint64_t>(s.N) * kOutBytes;
        tensormap_replace_address(m, c_ptr);
        tensormap_replace_dim0(m, static_cast<uint32_t>(pitch / kElem));
        tensormap_replace_dim1(m, s.M);
        tensormap_replace_dim2(m, s.batch);
        tensormap_replace_stride0(m, pitch);
        tensormap_replace_stride1(m, pitch * s.M);
        tensormap_replace_box0(m, 128 / kElem);
        tensormap_replace_box1(m, kBM);
        tensormap_replace_box2(m, 1);
        reinterpret_cast<uint32_t*>(out_map_stage)[16] = kOutTileBytes;
        tensormap_set_span_class(out_map_stage, pitch * s.M * s.batch);
      }
      __syncwarp();
      tensormap_publish(ws->map_aux, smem_u32(out_map_stage));
      if (lane == 0) tensormap_fence_acquire(ws->map_aux);
    }
    uint32_t local_tile = 0, pass = 0;
    for (int t = pair; t < num_tiles; t += num_pairs, ++local_tile) {
      int b, tm, tn;
      tile_coords(t, b, tm, tn);
      const int buf = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      const bool acc_ready = __all_sync(0xffffffffu, mbar_wait(tmem_full_bar(buf), acc_ph, abort_flag));
      if (!acc_ready && lane == 0) {
        report(ws, kStatusTimeoutTmemFull, local_tile);
        *abort_flag = 1;
        *epilogue_abort = 1;
      }
      if (tma_out) {
        named_barrier_sync(1, 128);  // the four warps agree before they meet at the barriers below
        if (*epilogue_abort) break;
      } else if (!acc_ready) {
        break;
      }
      tc_fence_after_sync();
      const int row = tm * 2 * kBM + rank * kBM + q * 32 + lane;
      const int64_t row_offset = (static_cast<int64_t>(b) * s.M + row) * s.N;
      float rs = 1.f;
      if constexpr (EPI == kEpiRequantF16) rs = (row < s.M) ? row_scale[row] : 0.f;
      if (tma_out) {
        const uint32_t my_row = static_cast<uint32_t>(q * 32 + lane) * 128u;
        const uint32_t swz = static_cast<uint32_t>(lane & 7);
        const int cols_here = s.N - tn * s.bn < s.bn ? s.N - tn * s.bn : s.bn;
        for (int c0 = 0; c0 < cols_here; c0 += kPassCols, ++pass) {
          uint32_t wv[32];
          if constexpr (kOutBytes == 4) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kMaxBN + c0, v);
            tc_wait_ld();
            convert_row_chunk<KIND, EPI>(v, tn * s.bn + c0, s.N, rs, col_scale, wv);
          } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t v[32], wh[32];
              tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kMaxBN + c0 + 32 * h, v);
              tc_wait_ld();
              convert_row_chunk<KIND, EPI>(v, tn * s.bn + c0 + 32 * h, s.N, rs, col_scale, wh);
#pragma unroll
              for (int j = 0; j < 16; ++j) wv[16 * h + j] = wh[j];
            }
          }
          if (c0 + kPassCols >= cols_here) {  // the accumulator is in registers: the leader may reuse it
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(tmem_empty_bar(buf), 0));
          }
          if (store_thread) bulk_wait_group_read<1>();  // the store that read this staging tile two passes ago is done with it
          named_barrier_sync(1, 128);
          const uint32_t tile = out_stage + (pass & 1) * kOutTileBytes;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            stage_st128(tile + my_row + ((static_cast<uint32_t>(j) ^ swz) << 4), wv[4 * j], wv[4 * j + 1], wv[4 * j + 2],
                        wv[4 * j + 3]);
          fence_proxy_async_smem();
          named_barrier_sync(1, 128);
          if (store_thread) {
            // (a CTA whose 128 rows all lie past M stores nothing: no store starts outside the tensor)
            if (tm * 2 * kBM + static_cast<int>(rank) * kBM < s.M)
              tma_store_3d(ws->map_aux, tile, (tn * s.bn + c0) * kOutBytes / kElem, tm * 2 * kBM + rank * kBM, b);
            bulk_commit_group();
          }
        }
        continue;
      }
      for (int c = 0; c < s.bn; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kMaxBN + c, v);
        tc_wait_ld();
        const int col0 = tn * s.bn + c;
        if (row < s.M && col0 < s.N) store_row_chunk<KIND, EPI>(v, c_ptr, row_offset, col0, s.N, rs, col_scale, vec_ok, wide_ok);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tmem_empty_bar(buf), 0));
    }
    if (tma_out && store_thread) bulk_wait_group<0>();
  }

  // Teardown: neither CTA may leave while its partner can still signal its barriers.
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
  }
  cluster_sync_all();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemColumns);
  }
}

}  // namespace b200

using namespace b200;

#define B200_GEMM_PAIR_EXPORT(NAME, KIND, EPI)                                                                \
  extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)                         \
      NAME(void* c, void* ws, int M, int N, int K, int batch, int b_layout, int bn) {                         \
    gemm_pair_body<KIND, EPI>(c, nullptr, nullptr, reinterpret_cast<Workspace*>(ws),                          \
                              GemmShape{M, N, K, batch, b_layout, bn});                                       \
  }
B200_GEMM_PAIR_EXPORT(b200_matmul_pair_f16_f16, kF16, kEpiCast)
B200_GEMM_PAIR_EXPORT(b200_matmul_pair_f16_f32, kF16, kEpiRaw)
B200_GEMM_PAIR_EXPORT(b200_matmul_pair_bf16_bf16, kBF16, kEpiCast)
B200_GEMM_PAIR_EXPORT(b200_matmul_pair_bf16_f32, kBF16, kEpiRaw)
B200_GEMM_PAIR_EXPORT(b200_matmul_pair_i8_i32, kI8, kEpiRaw)
extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    b200_matmul_pair_i8_requant_f16(void* c, const float* a_scale, const float* w_scale, void* ws, int M, int N, int K,
                                    int batch, int b_layout, int bn) {
  gemm_pair_body<kI8, kEpiRequantF16>(c, a_scale, w_scale, reinterpret_cast<Workspace*>(ws),
                                      GemmShape{M, N, K, batch, b_layout, bn});
}
