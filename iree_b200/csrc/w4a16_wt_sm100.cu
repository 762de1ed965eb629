// Fused "dequantise int4 weights, then contract" for more than a few activation rows (M > 16), with the
// operand roles swapped: the WEIGHTS are the 128-row operand of the tensor core and live in
// tensor memory, the activations are the (128- or 256-row) shared-memory operand, and the
// accumulator holds the transposed tile D[n, m].
//
//   w_f16[n,k] = f16( f16(sext(wq[n,k])) * scale[n, k/128] )      (exactly the dequant generic)
//   out[m,n]   = f16( sum_k f32(a[m,k]) * f32(w_f16[n,k]) )
//
// Why: with the expanded weights as a shared-memory operand (b200_w4a16_gemm) every 64-wide K
// block moves ~120 KiB through shared memory against 512 cycles of MMA, and the kernel is bound by
// shared-memory bandwidth. Here a dequant thread owns one weight row = one TMEM lane and writes its
// 64 expanded weights of a K block straight into tensor memory (tcgen05.st, no shared-memory round
// trip, no proxy fence); shared memory carries only the activation tile (TMA in, tensor core out)
// and the raw int4 bytes: ~72 KiB per 512 cycles of MMA.
//
//   warp 0      TMA producer of the activation tiles: 256 rows x 64 K per stage (two 128-row boxes)
//   warp 3      TMA producer of the raw int4 tiles: 128 rows x 128 K (one scale group) per stage
//   warps 8-15  dequant, two groups of four taking K blocks in turn (a third group changed
//               nothing: the groups are not what the tensor pipe waits for): 32 raw bytes of the
//               thread's row -> 32 registers of f16 pairs -> tcgen05.st into one of eight 32-column
//               A stages
//   warp 1      one thread issues tcgen05.mma (A from TMEM, B from shared memory, M = 128, N = 256)
//   warp 2      owns the TMEM allocation: 256 accumulator columns + 8 x 32 columns of A stages
//   warps 4-7   epilogue: tcgen05.ld -> f16 -> transposed into a shared-memory staging tile of
//               64 result rows x 128 columns -> one TMA store per destination
//
// Destinations: the epilogue stores each staged piece once per output tensor map in the workspace.
// One map (the dispatch's own result) is the plain case. With `world` > 1 there is one map per
// rank of the channel, each over that rank's full-width [M, N_total] result as mapped into this
// process: the rank's column block lands in every rank's buffer while the main loop of the next
// tile runs, which replaces the all-gather that would otherwise follow the dispatch. When a CTA
// has finished, its stores are complete; the last CTA of the grid then raises this rank's arrival
// word (value `epoch`, non-zero) in every rank's flag array. b200_wait_arrivals is the consumer side.
// No load in this file touches another GPU's memory and nothing here uses cluster multicast.
#include <cuda_fp16.h>
#include <stdint.h>

#include "sm100_ptx.cuh"
#include "w4a16_decode.cuh"

namespace b200 {

constexpr int kWtWRows = 128;                             // weight rows per tile = TMEM lanes (MMA M)
constexpr int kWtARows = 256;                             // activation rows per tile (MMA N)
constexpr int kWtActStagesLog2 = 2;
constexpr int kWtActStages = 1 << kWtActStagesLog2;
constexpr int kWtActStageBytes = kWtARows * 128;          // 32 KiB: 256 rows x 64 f16
constexpr int kWtRawStages = 6;
constexpr int kWtRawStageBytes = kWtWRows * 64;           // 8 KiB: 128 rows x 128 int4 = one scale group
constexpr int kWtAStagesLog2 = 3;
constexpr int kWtAStages = 1 << kWtAStagesLog2;
constexpr int kWtPairStages = kWtAStages / 2;             // pairs of K blocks (128 K) in flight: one barrier pair each                             // expanded-weight stages in tensor memory
constexpr int kWtAStageColumns = 32;                      // 64 K as f16 pairs
constexpr int kWtOutRows = 64;                            // result rows per staged piece
constexpr int kWtOutStageBytes = kWtOutRows * kWtWRows * 2;  // 16 KiB
constexpr int kWtDequantGroups = 2;                       // = K blocks per pair: group g expands the pair's block g
constexpr int kWtThreads = 256 + kWtDequantGroups * 128;
constexpr int kWtMaxDestinations = 8;
constexpr int kWtBarrierBytes = 512;
constexpr int kWtSmemBytes = 1024 + kWtActStages * kWtActStageBytes + kWtRawStages * kWtRawStageBytes +
                             2 * kWtOutStageBytes + kWtBarrierBytes;
static_assert(kWtSmemBytes <= 232448, "per-CTA shared memory limit");
static_assert(kWtARows + kWtAStages * kWtAStageColumns <= 512, "tensor memory columns");

// Workspace of this kernel: the 512-byte header of the other W4A16 kernels, then the output maps
// and the arrival-flag pointers.
struct alignas(128) WtWorkspace {
  uint8_t map_a[128];    // f16 [M, K], 128-byte swizzle, box 64 x 128
  uint8_t map_w[128];    // u8 [N, K/2], 64-byte swizzle, box 64 x 128
  uint8_t map_aux[128];
  uint32_t status[32];   // [0], [1] report; [8] counts finished CTAs
  uint8_t map_out[kWtMaxDestinations][128];  // f16 [M, n_off + N] with row pitch ldo, no swizzle, box 128 x 64
  uint32_t* flags[kWtMaxDestinations];       // rank p's arrival words (this rank writes word `rank`)
};

__device__ __forceinline__ void wt_report(WtWorkspace* ws, uint32_t code, uint32_t info) {
  if (atomicCAS(&ws->status[0], 0u, code) == 0u) ws->status[1] = info;
}

__device__ __forceinline__ void wt_body(const __half* __restrict__ scales, WtWorkspace* __restrict__ ws, int M, int N,
                                        int K, int n_off, int world, int rank, int epoch) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t raw_base = smem_base + kWtActStages * kWtActStageBytes;
  const uint32_t out_base = raw_base + kWtRawStages * kWtRawStageBytes;
  const uint32_t bars = out_base + 2 * kWtOutStageBytes;
  uint8_t* bars_gen = smem_gen + (bars - smem_base);
  // barriers: act full (eight slots, four in use with 256-row tiles; an activation stage comes back through
  // the A-stage barrier of the K block that held it), raw full / empty, A-stage full / empty, accumulator full / empty
  auto act_early = [&](int i) { return bars + 8u * i; };  // "the first block of a pair is done with activation stage i"
  auto raw_full = [&](int i) { return bars + 8u * (2 * kWtActStages + i); };
  auto raw_empty = [&](int i) { return bars + 8u * (2 * kWtActStages + kWtRawStages + i); };
  auto a_full = [&](int i) { return bars + 8u * (2 * kWtActStages + 2 * kWtRawStages + i); };
  auto a_empty = [&](int i) { return bars + 8u * (2 * kWtActStages + 2 * kWtRawStages + kWtAStages + i); };
  constexpr int kNumRingBars = 2 * kWtActStages + 2 * kWtRawStages + 2 * kWtAStages;
  const uint32_t d_full = bars + 8u * kNumRingBars, d_empty = bars + 8u * (kNumRingBars + 1);
  const uint32_t tmem_slot = bars + 8u * (kNumRingBars + 2);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * (kNumRingBars + 2));
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * (kNumRingBars + 2) + 4);
  static_assert(8 * (kNumRingBars + 3) <= kWtBarrierBytes, "barrier area");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool bad = M <= 0 || N <= 0 || K <= 0 || (K & 127) || world < 1 || world > kWtMaxDestinations || (n_off & 7);
  // The next dispatch on the stream may be launched from here on; it orders itself on the device.
  grid_launch_dependents();
  if (bad) {
    grid_dependency_wait();
    if (threadIdx.x == 0) wt_report(ws, kStatusBadArgument, 0);
    return;
  }
  // Up to 128 activation rows: tiles of 128 (MMA N = 128, half the tensor-pipe time per K block and
  // no zero rows to multiply); above that tiles of 256.
  const int a_rows = M <= 128 ? 128 : kWtARows;
  // The activation ring holds 128 KiB either way: four stages of 256 rows or eight of 128 (a tile of
  // 128 rows finishes its MMAs in half the time, so it needs twice the stages in flight).
  const int act_stages = a_rows == 128 ? 2 * kWtActStages : kWtActStages;
  const uint32_t act_pitch = static_cast<uint32_t>(a_rows) * 128u;
  const bool early_release = act_stages == kWtActStages;  // four stages: hand an activation stage back per block, not per pair
  const int tiles_m = (M + a_rows - 1) / a_rows;
  const int tiles_n = (N + kWtWRows - 1) / kWtWRows;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = K / 64;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2 * kWtActStages; ++i) {  // 128-row tiles run eight half-size activation stages
      mbar_init(act_early(i), 1);
    }
    for (int i = 0; i < kWtRawStages; ++i) {
      mbar_init(raw_full(i), 1);
      mbar_init(raw_empty(i), 8);  // a raw stage holds two K blocks: the four warps of each block's group
    }
    for (int i = 0; i < kWtPairStages; ++i) {
      mbar_init(a_full(i), 9);     // the eight dequant warps (four per K block of the pair) + the activation tiles' expect_tx
      mbar_init(a_empty(i), 1);
    }
    mbar_init(d_full, 1);
    mbar_init(d_empty, 4);
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
  const uint32_t tmem_a = tmem_base + kWtARows;  // A stages follow the accumulator columns

  // Consecutive tiles of a CTA share the weight rows and walk down the activations.
  auto tile_coords = [&](int t, int& tm, int& tn) {
    tn = t / tiles_m;
    tm = t - tn * tiles_m;
  };

  if (warp == 0) {
    // -------- TMA producer of the activation tiles ------------------------------------------------
    if (lane == 0) {
      tensormap_fence_acquire(ws->map_a);
      const uint32_t act_mask = static_cast<uint32_t>(act_stages) - 1u, act_pairs = static_cast<uint32_t>(act_stages) >> 1;
      const uint32_t act_shift = act_stages == 2 * kWtActStages ? kWtActStagesLog2 + 1 : kWtActStagesLog2;
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, tm, tn);
        // Two K blocks (one scale group, 128 K) at a time: the pair shares one "full" and one "empty" barrier
        // (slot pair % kWtPairStages of a_full / a_empty), so the issuing thread waits and commits once per
        // eight MMAs. Its loop period, not the tensor pipe, is what bounds this kernel: a wait costs it ~125
        // cycles even when the phase is long complete, a commit ~46, an MMA ~75. The activation tiles of the
        // pair report to the pair's "full" barrier next to the dequant warps' arrivals.
        for (int kb = 0; kb < num_kb; kb += 2, it += 2) {
          const uint32_t pair = it >> 1;
          // The two activation stages' previous tenants were the blocks of pair - act_pairs; their MMAs'
          // completion is what the pair's "empty" barrier reports.
          // With four stages (256-row tiles) a pair's lead would be one pair of MMAs, less than a load takes:
          // there the issuing thread reports the first block's MMAs on a barrier of their own (act_early), so
          // that each stage is refilled as soon as its block is done, four blocks ahead as before.
          const uint32_t prev = pair - act_pairs;
          const uint32_t full = a_full(pair % kWtPairStages);
          bool waited = true;
          if (pair >= act_pairs && early_release) {
            const uint32_t prev_block = it - act_stages;
            waited = mbar_wait(act_early(prev_block & act_mask), (prev_block >> act_shift) & 1, abort_flag);
          } else if (pair >= act_pairs) {
            waited = mbar_wait(a_empty(prev % kWtPairStages), (prev / kWtPairStages) & 1, abort_flag);
          }
          if (waited) {
            mbar_arrive_expect_tx(full, 2 * a_rows * 128);
            const uint32_t dst = smem_base + (it & act_mask) * act_pitch;
            tma_load_3d(dst, ws->map_a, full, kb * 64, tm * a_rows, 0);
            if (a_rows > 128) tma_load_3d(dst + 128 * 128, ws->map_a, full, kb * 64, tm * a_rows + 128, 0);
            if (pair >= act_pairs && early_release)
              waited = mbar_wait(a_empty(prev % kWtPairStages), (prev / kWtPairStages) & 1, abort_flag);
          }
          if (!waited) {
            wt_report(ws, kStatusTimeoutEmpty, it);
            *abort_flag = 1;
            ok = false;
            break;
          }
          {
            const uint32_t dst = smem_base + ((it + 1) & act_mask) * act_pitch;
            tma_load_3d(dst, ws->map_a, full, (kb + 1) * 64, tm * a_rows, 0);
            if (a_rows > 128) tma_load_3d(dst + 128 * 128, ws->map_a, full, (kb + 1) * 64, tm * a_rows + 128, 0);
          }
        }
      }
    }
  } else if (warp == 3) {
    // -------- TMA producer of the raw weights: one scale group (128 K) per stage --------------------
    if (lane == 0) {
      tensormap_fence_acquire(ws->map_w);
      uint32_t raw_it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, tm, tn);
        for (int g = 0; g < (num_kb >> 1); ++g, ++raw_it) {
          const int rs = raw_it % kWtRawStages;
          if (!mbar_wait(raw_empty(rs), ((raw_it / kWtRawStages) & 1) ^ 1, abort_flag)) {
            wt_report(ws, kStatusTimeoutEmpty, 0x10000u | raw_it);
            *abort_flag = 1;
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(raw_full(rs), kWtRawStageBytes);
          tma_load_3d(raw_base + rs * kWtRawStageBytes, ws->map_w, raw_full(rs), g * 64, tn * kWtWRows, 0);
        }
      }
    }
  } else if (warp == 1) {
    // -------- MMA issuer ---------------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_instr_desc(1u, 0u, 0u, 0u, 0u, kWtWRows, a_rows);
      // This thread's instruction stream is what a K block waits for (measured: ~700 cycles per block with
      // divisions by the run-time stage count and four descriptor constructions in it, against 512 of
      // MMA), so everything per block is an add, a shift or a mask: the stage counts are powers of two,
      // and a descriptor differs from the first stage's only in its address field (16-byte units).
      const uint32_t act_mask = static_cast<uint32_t>(act_stages) - 1u;
      const uint64_t desc0 = make_smem_desc(smem_base, 16, 1024);
      const uint32_t stage_units = act_pitch >> 4;
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local_tile) {
        if (!mbar_wait(d_empty, (local_tile & 1) ^ 1, abort_flag)) {
          wt_report(ws, kStatusTimeoutTmemEmpty, local_tile);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        for (int kb = 0; kb < num_kb; kb += 2, it += 2) {
          const uint32_t pair = it >> 1, ps = pair & (kWtPairStages - 1);
          if (!mbar_wait(a_full(ps), (pair / kWtPairStages) & 1, abort_flag)) {  // both blocks' weights and activations
            wt_report(ws, kStatusTimeoutDequant, it);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint64_t bd = desc0 + ((it + h) & act_mask) * stage_units;                    // + 2 per 32 bytes of K
            const uint32_t a_t = tmem_a + ((it + h) & (kWtAStages - 1)) * kWtAStageColumns;     // + 8 columns per 16 K
            if (kb == 0 && h == 0) mma_f16_ts_first(tmem_base, a_t, bd, idesc);
            else mma_f16_ts_more(tmem_base, a_t, bd, idesc);
            mma_f16_ts_more(tmem_base, a_t + 8, bd + 2, idesc);
            mma_f16_ts_more(tmem_base, a_t + 16, bd + 4, idesc);
            mma_f16_ts_more(tmem_base, a_t + 24, bd + 6, idesc);
            if (h == 0 && early_release) tc_commit(act_early(it & act_mask));
          }
          tc_commit(a_empty(ps));
        }
        if (ok) tc_commit(d_full);
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // -------- epilogue: D[n, m] -> staged [m, n] f16 pieces -> TMA stores -----------------------------
    const int qd = warp & 3;
    const bool issuer = threadIdx.x == 128;
    if (issuer)
      for (int p = 0; p < world; ++p) tensormap_fence_acquire(ws->map_out[p]);
    uint32_t local_tile = 0, piece_it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++local_tile) {
      int tm, tn;
      tile_coords(t, tm, tn);
      if (!__all_sync(0xffffffffu, mbar_wait(d_full, local_tile & 1, abort_flag))) {
        if (lane == 0) {
          wt_report(ws, kStatusTimeoutTmemFull, local_tile);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after_sync();
      const int rows_left = M - tm * a_rows;
      const int pieces = rows_left >= a_rows ? a_rows / kWtOutRows : (rows_left + kWtOutRows - 1) / kWtOutRows;
      for (int pc = 0; pc < a_rows / kWtOutRows; ++pc) {
        uint32_t v0[32], v1[32];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(qd * 32) << 16) + pc * kWtOutRows;
        tmem_ld_32x32(taddr, v0);
        tmem_ld_32x32(taddr + 32, v1);
        tc_wait_ld();
        if (pc == a_rows / kWtOutRows - 1) {
          // the accumulator is in registers / already stored: the next tile's MMAs may start
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(d_empty);
        }
        if (pc >= pieces) continue;  // rows beyond M: nothing to store (warp-uniform)
        const uint32_t stage = out_base + (piece_it & 1) * kWtOutStageBytes;
        // the stores issued from this staging buffer two pieces ago must have read it
        if (issuer) bulk_wait_group_read<1>();
        named_barrier_sync(1, 128);
        const uint32_t dst = stage + (qd * 32 + lane) * 2;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const uint16_t h0 = __half_as_ushort(__float2half_rn(__uint_as_float(v0[j])));
          const uint16_t h1 = __half_as_ushort(__float2half_rn(__uint_as_float(v1[j])));
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(dst + j * (kWtWRows * 2)), "h"(h0) : "memory");
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(dst + (j + 32) * (kWtWRows * 2)), "h"(h1) : "memory");
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, 128);
        if (issuer) {
          const int x = n_off + tn * kWtWRows, y = tm * a_rows + pc * kWtOutRows;
          for (int p = 0; p < world; ++p) {
            const int dest = (rank + p) % world;  // start with the own buffer, then round the ring
            tma_store_2d(ws->map_out[dest], stage, x, y);
          }
          bulk_commit_group();
        }
        ++piece_it;
      }
    }
    if (issuer) {
      bulk_wait_group<0>();  // every store of this CTA is complete and visible to this thread
      if (epoch != 0 && !*abort_flag) {  // a pushing dispatch: tell every destination that this rank's block is there
        __threadfence_system();
        const uint32_t finished = atomicAdd(&ws->status[8], 1u);
        if (finished == gridDim.x - 1) {
          // every CTA's stores are ordered before this point (fence / atomic / fence)
          ws->status[8] = 0;
          __threadfence_system();
          for (int p = 0; p < world; ++p) st_release_sys(ws->flags[(rank + p) % world] + rank, static_cast<uint32_t>(epoch));
        }
      }
    }
  } else if (warp >= 8) {
    // -------- dequant: raw int4 (64-byte swizzled rows) -> 32 columns of this thread's TMEM lane ------
    const int td = threadIdx.x - 256;
    const int r = td & 127;   // weight row of the tile = TMEM lane; td / 32 % 4 == warp % 4
    const int grp = td >> 7;  // K blocks grp, grp + kWtDequantGroups, ...
    const int groups = K >> 7;
    // Scales of eight consecutive groups arrive as one 16-byte load, one load ahead of their use.
    const bool vec_scales = (groups & 7) == 0 && (reinterpret_cast<uintptr_t>(scales) & 15) == 0;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t it_base = 0, raw_it_base = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, it_base += num_kb, raw_it_base += num_kb >> 1) {
      int tm, tn;
      tile_coords(t, tm, tn);
      const int n = tn * kWtWRows + r;
      const bool has_scales = n < N;
      const __half* srow = scales + static_cast<size_t>(has_scales ? n : 0) * groups;
      __half2 s2 = __half2half2(__float2half_rn(0.f));
      uint4 sc_cur = make_uint4(0, 0, 0, 0), sc_next = make_uint4(0, 0, 0, 0);
      __half next_scale = __float2half_rn(0.f);
      int cur_octet = -1;  // which eight groups sc_cur holds; sc_next holds the eight after them
      if (has_scales) {
        if (vec_scales) sc_next = *reinterpret_cast<const uint4*>(srow);
        else if ((grp >> 1) < groups) next_scale = srow[grp >> 1];
      }
      for (int kb = grp; kb < num_kb; kb += kWtDequantGroups) {
        const uint32_t it = it_base + kb;
        const uint32_t raw_it = raw_it_base + (kb >> 1);
        const int rs = raw_it % kWtRawStages;
        if (!__all_sync(0xffffffffu, mbar_wait(raw_full(rs), (raw_it / kWtRawStages) & 1, abort_flag))) {
          if (lane == 0) {
            wt_report(ws, kStatusTimeoutFull, 0x10000u | raw_it);
            *abort_flag = 1;
          }
          ok = false;
          break;
        }
        {
          const int g = kb >> 1;
          if (vec_scales) {
            if ((g >> 3) != cur_octet) {  // a group's blocks advance g by one or two: never past a whole octet
              sc_cur = sc_next;
              cur_octet = g >> 3;
              if (has_scales && (cur_octet + 1) * 8 < groups)
                sc_next = *reinterpret_cast<const uint4*>(srow + (cur_octet + 1) * 8);
            }
            const uint32_t word = (g & 4) ? ((g & 2) ? sc_cur.w : sc_cur.z) : ((g & 2) ? sc_cur.y : sc_cur.x);
            s2 = as_half2(__byte_perm(word, 0u, (g & 1) ? 0x3232u : 0x1010u));
          } else {
            s2 = __half2half2(next_scale);
            const int g_next = (kb + kWtDequantGroups) >> 1;  // this group's next block
            if (has_scales && g_next < groups) next_scale = srow[g_next];
          }
        }
        const int as = it % kWtAStages;
        const uint32_t pair = it >> 1, ps = pair % kWtPairStages;  // the pair this block belongs to (block = 2 * pair + grp)
        if (!__all_sync(0xffffffffu, mbar_wait(a_empty(ps), ((pair / kWtPairStages) & 1) ^ 1, abort_flag))) {
          if (lane == 0) {
            wt_report(ws, kStatusTimeoutEmpty, 0x20000u | it);
            *abort_flag = 1;
          }
          ok = false;
          break;
        }
        tc_fence_after_sync();
        // Raw stage: row r is 64 bytes; its four 16-byte chunks are XOR-swizzled by (r / 2) % 4.
        const uint32_t raw_row = raw_base + rs * kWtRawStageBytes + r * 64;
        const int sw_raw = (r >> 1) & 3;
        uint32_t e[32];  // e[4 i + j] = (w(8 i + 2 j), w(8 i + 2 j + 1)) * scale: column 4 i + j of the stage
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int chunk = (kb & 1) * 2 + c;  // 16-byte chunk of the 64-byte raw row
          const uint4 w = lds128(raw_row + ((chunk ^ sw_raw) << 4));
          const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            __half2 qv[4];
            unpack8_ordered(words[i], qv);
#pragma unroll
            for (int j = 0; j < 4; ++j) e[(c * 4 + i) * 4 + j] = as_u32(__hmul2(qv[j], s2));  // f16(w) * scale, one rounding
          }
        }
        tmem_st_32x32(tmem_a + lane_base + as * kWtAStageColumns, e);
        tc_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(a_full(ps));
          mbar_arrive(raw_empty(rs));
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

// Bindings: scales, the result (named for the host program's data flow; the kernel reaches it
// through the workspace's output maps), the workspace. world_rank = world << 8 | rank.
extern "C" __global__ void __launch_bounds__(kWtThreads, 1)
    b200_w4a16_gemm_wt(const __half* scales, __half* out, void* ws, int M, int N, int K, int ldo, int n_off,
                       int world_rank, int epoch) {
  (void)out;
  (void)ldo;
  wt_body(scales, reinterpret_cast<WtWorkspace*>(ws), M, N, K, n_off, world_rank >> 8, world_rank & 0xff, epoch);
}

// Consumer side of the arrival words: returns once every rank's word in `flags` has reached
// `epoch`, i.e. once every rank's column block of the result has landed in this rank's buffer.
// The wait is bounded (about two seconds); if it runs out, the status words of `ws` say so and
// the kernel returns, leaving the context usable.
extern "C" __global__ void __launch_bounds__(32, 1)
    b200_wait_arrivals(const uint32_t* flags, void* ws_raw, int world, int epoch) {
  WtWorkspace* ws = reinterpret_cast<WtWorkspace*>(ws_raw);
  const int lane = threadIdx.x;
  if (lane < world) {
    const uint64_t t0 = global_timer_ns();
    uint32_t polls = 0;
    while (static_cast<int32_t>(ld_acquire_sys(flags + lane) - static_cast<uint32_t>(epoch)) < 0) {
      if ((++polls & 0x3f) == 0 && global_timer_ns() - t0 > kDefaultWaitLimitNs) {
        wt_report(ws, kStatusTimeoutFull, 0x40000u | static_cast<uint32_t>(lane));
        break;
      }
    }
  }
  __syncwarp();
}
