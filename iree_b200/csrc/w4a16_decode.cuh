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

// Exact signed values of weights (j, j+4) for j = 0..3 of one word, as four half2:
//   p[0] = (w0, w4), p[1] = (w1, w5), p[2] = (w2, w6), p[3] = (w3, w7).
// 0x6400 | x is the f16 1024 + x; flipping the nibble's top bit turns two's complement into
// "value + 8", so 1024 + (n ^ 8) - 1032 = w, and for the nibble four bits up
// (1024 + 16 (n ^ 8)) / 16 - 72 = w. Both are exact in f16.
__device__ __forceinline__ void unpack8_strided(uint32_t v, __half2 (&p)[4]) {
  const __half2 k1032 = __floats2half2_rn(1032.f, 1032.f);
  const __half2 k16th = __floats2half2_rn(0.0625f, 0.0625f);
  const __half2 km72 = __floats2half2_rn(-72.f, -72.f);
  const uint32_t v8 = v >> 8;
  p[0] = __hsub2(as_half2(lop3_and_xor(v, 0x000f000fu, 0x64086408u)), k1032);
  p[1] = __hfma2(as_half2(lop3_and_xor(v, 0x00f000f0u, 0x64806480u)), k16th, km72);
  p[2] = __hsub2(as_half2(lop3_and_xor(v8, 0x000f000fu, 0x64086408u)), k1032);
  p[3] = __hfma2(as_half2(lop3_and_xor(v8, 0x00f000f0u, 0x64806480u)), k16th, km72);
}

// Exact signed values of weights in memory order: q[j] = (w(2j), w(2j+1)), j = 0..3 (byte j).
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

__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// =============================================================================================
// Decode kernel
// =============================================================================================
constexpr int kDecodeThreads = 512;
constexpr int kDecodeWarps = 16;
constexpr int kDecodeChunkK = 256;                           // K per warp
constexpr int kDecodeSliceK = kDecodeWarps * kDecodeChunkK;  // K per CTA and pass: 4096
constexpr int kDecodeTileRows = 16;                          // weight rows per tile
// Weight tiles resident in shared memory. All of them are requested before the activations are
// fetched, so that the memory system stays busy during the prologue; in steady state one is being
// read and three are in flight.
constexpr int kDecodeStages = 4;
constexpr int kDecodeSlots = 4;                              // tiles whose partial sums are live at the same time
// A staged row is the 2048 B of the CTA's K slice, so a full-width tile (K = 4096) is one contiguous
// 32 KiB copy. Rows g and g + 1 then start in the same banks; the reads are arranged so that odd
// rows fetch the other 64-byte half first (see the main loop).
constexpr int kDecodeRowPitch = kDecodeSliceK / 2;
constexpr int kDecodeMaxScaleBytes = 16 * 128 * 2;          // scale tile: 16 rows x up to 128 groups (K <= 16384)

// Dynamic shared memory of the decode kernel:
//   weight ring  [stage][row][2048 B]      the tile's rows of the CTA's K slice: one bulk copy per tile when
//                                          the slice is the whole row, else one per row
//   scale ring   [stage][row][K / 128] f16 the tile's scale rows, one bulk copy
//   partial sums [slot][warp][lane][4 MH] f32   (MMA fragment order, one per K chunk); doubles as
//                                          the staging area of the activation prologue
//   mbarriers: weights full / empty per stage, partials full / empty per slot; abort word
//   (M > 8 only) offset corrections [warp][mh][step][lane] float2: the 16-row variant has no registers left for them
__host__ __device__ constexpr int decode_smem_bytes(int mh) {
  return kDecodeStages * kDecodeTileRows * kDecodeRowPitch + kDecodeStages * kDecodeMaxScaleBytes +
         kDecodeSlots * kDecodeWarps * 32 * 4 * mh * 4 + (2 * kDecodeStages + 2 * kDecodeSlots) * 8 + 16 +
         (mh == 2 ? kDecodeWarps * 4 * 32 * 8 : 0);
}

// Scratch for K beyond one slice: f32 partial sums [16][n_pad] (followed by one spare word per
// 16-row tile, kept for layout compatibility). Must be zero before the first launch; the kernel
// leaves it zeroed.
struct DecodeScratchLayout {
  __host__ __device__ static size_t partial_floats(int N) { return static_cast<size_t>(16) * N; }
  __host__ __device__ static size_t bytes(int N) { return partial_floats(N) * 4 + static_cast<size_t>(N / 16) * 4; }
};

__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// Untiled bulk copy global -> shared, completion reported to an mbarrier as transaction bytes.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Development aid: with -DB200_DECODE_TRACE warps 0 and 15 of every CTA record clock stamps (cycles
// since kernel entry) into the scratch buffer, 32 per warp: [cta][2][32] int64.
#ifdef B200_DECODE_TRACE
#define DECODE_STAMP()                                                                              \
  do {                                                                                              \
    if (lane == 0 && (warp == 0 || warp == 15) && trace_n < 32)                                     \
      reinterpret_cast<long long*>(scratch)[(blockIdx.x * 2 + (warp ? 1 : 0)) * 32 + trace_n++] =  \
          clock64() - trace_t0;                                                                     \
  } while (0)
#else
#define DECODE_STAMP() do { } while (0)
#endif

// The weights enter the MMA as the biased halves the bit trick produces, without a subtract:
//   low nibbles  -> 1032 + w      0x6400 | (n ^ 8): the nibble sits in the last mantissa bits of 1024
//   high nibbles ->   72 + w      0x5400 | ((n ^ 8) << 4): in f16, 64 has a mantissa step of 1/16, so
//                                 a nibble four bits up adds exactly its value
// Both feed the same accumulator; with S_lo / S_hi the sums of the activations that met the low /
// high nibbles, the group sum is d - (1032 S_lo + 72 S_hi). All of this is exact for integer data
// and loses < 1e-4 relative on normal data (f32 accumulation of terms ~1e3 |a|).
template <int MH>
__device__ __forceinline__ void decode_body(const __half* __restrict__ a, const uint8_t* __restrict__ wq,
                                            const __half* __restrict__ scales, __half* __restrict__ out,
                                            float* __restrict__ scratch, int M, int N, int K, int ldo, int n_off) {
  constexpr int kDecodeWRingBytes = kDecodeStages * kDecodeTileRows * kDecodeRowPitch;
  constexpr int kDecodeSRingBytes = kDecodeStages * kDecodeMaxScaleBytes;
  extern __shared__ __align__(128) uint8_t decode_smem[];
  uint8_t* wring = decode_smem;
  uint8_t* sring = wring + kDecodeWRingBytes;
  float* accs = reinterpret_cast<float*>(sring + kDecodeSRingBytes);
  uint8_t* bar_mem = reinterpret_cast<uint8_t*>(accs + kDecodeSlots * kDecodeWarps * 32 * 4 * MH);
  const uint32_t bars = smem_u32(bar_mem);
  auto wfull_bar = [&](int i) { return bars + 8u * i; };
  auto wempty_bar = [&](int i) { return bars + 8u * (kDecodeStages + i); };
  auto pfull_bar = [&](int i) { return bars + 8u * (2 * kDecodeStages + i); };
  auto pempty_bar = [&](int i) { return bars + 8u * (2 * kDecodeStages + kDecodeSlots + i); };
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bar_mem + (2 * kDecodeStages + 2 * kDecodeSlots) * 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
#ifdef B200_DECODE_TRACE
  const long long trace_t0 = clock64();
  int trace_n = 0;
#endif
  const int groups_per_row = K >> 7;
  const int row_bytes = K >> 1;
  const int num_tiles = N / kDecodeTileRows;
  // K beyond one slice (4096) is covered by several passes of this CTA over its tiles: partial
  // sums wait in the f32 scratch between passes; nobody else touches them, so no atomics and no
  // fences. The grid is one-dimensional.
  const int num_passes = (K + kDecodeSliceK - 1) / kDecodeSliceK;
  const int my_tiles = blockIdx.x < num_tiles ? (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const uint32_t scale_tile_bytes = kDecodeTileRows * groups_per_row * 2;
  bool dead = false;  // a wait ran out: skip the work, keep meeting the CTA-wide barriers
  // The next kernel on the stream may be scheduled as soon as this one's blocks leave their SMs:
  // it will fetch its first weight tiles (weights and scales are inputs of the whole program, no
  // kernel writes them) and then wait, below, for this kernel to finish.
  grid_launch_dependents();

  for (int pass = 0; pass < num_passes; ++pass) {
    const int k_slice0 = pass * kDecodeSliceK;
    const int kc = k_slice0 + warp * kDecodeChunkK;  // this warp's K chunk (K is a multiple of 256)
    int active_warps = (K - k_slice0) / kDecodeChunkK;  // K chunks in this slice
    if (active_warps > kDecodeWarps) active_warps = kDecodeWarps;
    // Warps without a K chunk in this slice still run the barrier protocol and their share of
    // the reduction, so that every arrival count is the constant 16.
    const bool has_chunk = warp < active_warps;
    const uint32_t slice_row_bytes = active_warps * (kDecodeChunkK / 2);
    const bool first_pass = pass == 0, last_pass = pass == num_passes - 1;

    __syncthreads();  // every warp is done with the previous pass (and its global partial sums)
    if (threadIdx.x == 0) {
      if (pass > 0)  // the barriers of the previous pass are quiescent: retire them before re-use
        for (int i = 0; i < 2 * kDecodeStages + 2 * kDecodeSlots; ++i) mbar_inval(bars + 8u * i);
      for (int i = 0; i < kDecodeStages; ++i) {
        mbar_init(wfull_bar(i), 1);
        mbar_init(wempty_bar(i), kDecodeWarps);
      }
      for (int i = 0; i < kDecodeSlots; ++i) {
        mbar_init(pfull_bar(i), kDecodeWarps);
        mbar_init(pempty_bar(i), 1);
      }
      if (pass == 0) *abort_flag = 0;
      mbar_fence_init();
    }
    __syncthreads();
    if (dead || *abort_flag) continue;
    DECODE_STAMP();  // 0: barriers initialised

    // Feeding the weight ring is a side job that rotates over the warps (tile jp is fetched by warp
    // jp % 16): bulk copies are asynchronous, so nobody blocks on their completion. When the CTA's
    // slice is the whole row (K = 4096) a tile is one contiguous 32 KiB copy, otherwise one copy per
    // weight row (lanes 0..15); its scale rows are one more copy.
    const bool whole_rows = slice_row_bytes == static_cast<uint32_t>(row_bytes) && slice_row_bytes == kDecodeRowPitch;
    auto produce = [&](int jp) -> bool {
      if (jp >= my_tiles || warp != jp % kDecodeWarps) return true;
      const int st = jp % kDecodeStages;
      if (!__all_sync(0xffffffffu, mbar_wait<false>(wempty_bar(st), ((jp / kDecodeStages) & 1) ^ 1, abort_flag))) {
        *abort_flag = 1;
        return false;
      }
      const size_t row0 = static_cast<size_t>(blockIdx.x + jp * gridDim.x) * kDecodeTileRows;
      const uint32_t dst = smem_u32(wring) + st * kDecodeTileRows * kDecodeRowPitch;
      if (lane == 0) {
        mbar_arrive_expect_tx(wfull_bar(st), kDecodeTileRows * slice_row_bytes + scale_tile_bytes);
        bulk_load(smem_u32(sring) + st * kDecodeMaxScaleBytes, scales + row0 * groups_per_row, scale_tile_bytes,
                  wfull_bar(st));
        if (whole_rows) bulk_load(dst, wq + row0 * row_bytes, kDecodeTileRows * slice_row_bytes, wfull_bar(st));
      }
      __syncwarp();
      if (!whole_rows && lane < kDecodeTileRows)
        bulk_load(dst + lane * kDecodeRowPitch, wq + (row0 + lane) * row_bytes + (k_slice0 >> 1), slice_row_bytes,
                  wfull_bar(st));
      return true;
    };
    for (int jp = 0; jp < kDecodeStages; ++jp)
      if (!produce(jp)) break;
    DECODE_STAMP();  // 1: first weight tiles requested

    // ---- activations of this warp's chunk, kept in registers in the order the MMAs want -----------
    // For step s, word i: the thread's eight k are k0 = kc + 128 s + 32 q + 8 i .. k0 + 7, paired
    // (0,4), (1,5), (2,6), (3,7) like the nibbles of a weight word. Each warp reads its chunk of every
    // activation row with coalesced 256-byte requests, parks it in its corner of the partial-sum
    // area (not in use yet) and picks up the 64 bytes per row and step it needs.
    // Activations, the scratch and the output may belong to the preceding kernel until it is done.
    if (pass == 0) grid_dependency_wait();
    uint32_t bfrag[MH][2][4][4];
    float bias[MH][2][2];  // 1032 S_lo + 72 S_hi per step and output column (2q, 2q + 1)
    float2* bias_smem = reinterpret_cast<float2*>(bar_mem + (2 * kDecodeStages + 2 * kDecodeSlots) * 8 + 16) + warp * 4 * 32 + lane;
    if (has_chunk) {
      uint8_t* tmp = reinterpret_cast<uint8_t*>(accs) + warp * 2048;
      // All global loads first (they land in the registers that will hold the fragments), then the
      // per-step shuffles through shared memory, so the load latency is paid once.
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
            *reinterpret_cast<uint4*>(tmp + (2 * it + (lane >> 4)) * 256 + (lane & 15) * 16) =
                make_uint4(bfrag[mh][s][it][0], bfrag[mh][s][it][1], bfrag[mh][s][it][2], bfrag[mh][s][it][3]);
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 x = *reinterpret_cast<const uint4*>(tmp + g * 256 + 64 * q + 16 * i);
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
          bias[mh][s][0] = 1032.f * s_lo[0] + 72.f * s_hi[0];
          bias[mh][s][1] = 1032.f * s_lo[1] + 72.f * s_hi[1];
          if (MH == 2) bias_smem[(2 * mh + s) * 32] = make_float2(bias[mh][s][0], bias[mh][s][1]);
        }
    }
    DECODE_STAMP();  // 2: activation fragments ready
    // The staging corners become partial-sum slots only after every warp is done with them.
    __syncthreads();
    DECODE_STAMP();  // 3: staging area released

    // Partial sums of one tile: [slot][K chunk][fragment lane] float4 x MH.
    auto partial_cell = [&](int slot, int chunk, int frag_lane) -> float4* {
      return reinterpret_cast<float4*>(accs) + ((slot * kDecodeWarps + chunk) * 32 + frag_lane) * MH;
    };
    // Adds the K chunks of tile jf in chunk order (so the result does not depend on arrival
    // order), frees the slot and writes the 16 x M results. One warp per tile, in rotation.
    // Fragment order: vals[4 mh + c] is weight row g + 8 (c / 2), activation row 2 q + (c & 1) + 8 mh.
    auto finalize = [&](int jf) -> bool {
      const int slot = jf % kDecodeSlots;
      const int tile = blockIdx.x + jf * gridDim.x;
      if (!__all_sync(0xffffffffu, mbar_wait<false>(pfull_bar(slot), (jf / kDecodeSlots) & 1, abort_flag))) {
        *abort_flag = 1;
        return false;
      }
      float vals[4 * MH];
#pragma unroll
      for (int c = 0; c < 4 * MH; ++c) vals[c] = 0.f;
      // a batch of loads first, then the adds: sixteen dependent load-add steps would cost sixteen
      // shared-memory latencies
      constexpr int kBatch = 8 / MH;
#pragma unroll
      for (int first = 0; first < kDecodeWarps; first += kBatch) {
        float4 v[kBatch][MH];
#pragma unroll
        for (int k = 0; k < kBatch; ++k)
#pragma unroll
          for (int mh = 0; mh < MH; ++mh)
            v[k][mh] = (first + k) < active_warps ? partial_cell(slot, first + k, lane)[mh] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < kBatch; ++k)
#pragma unroll
          for (int mh = 0; mh < MH; ++mh) {
            vals[4 * mh + 0] += v[k][mh].x;
            vals[4 * mh + 1] += v[k][mh].y;
            vals[4 * mh + 2] += v[k][mh].z;
            vals[4 * mh + 3] += v[k][mh].w;
          }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(pempty_bar(slot));  // hand the slot to tile jf + kDecodeSlots
#pragma unroll
      for (int it = 0; it < 4 * MH; ++it) {
        const int r = g + 8 * ((it >> 1) & 1), m = 2 * q + (it & 1) + 8 * (it >> 2);
        float* cell = &scratch[static_cast<size_t>(m) * N + tile * kDecodeTileRows + r];
        float total = vals[it];
        if (!first_pass) total += __ldcg(cell);      // what the earlier K slices left here
        if (!last_pass) {
          __stcg(cell, total);
        } else {
          if (num_passes > 1) __stcg(cell, 0.f);     // leave the scratch clean for the next launch
          if (m < M) out[static_cast<size_t>(m) * ldo + n_off + tile * kDecodeTileRows + r] = __float2half_rn(total);
        }
      }
      return true;
    };

    bool ok = true;
    for (int j = 0; j < my_tiles && ok; ++j) {
      const int st = j % kDecodeStages;
      if (!__all_sync(0xffffffffu, mbar_wait<false>(wfull_bar(st), (j / kDecodeStages) & 1, abort_flag))) {
        *abort_flag = 1;
        break;
      }
      DECODE_STAMP();  // 4 + 5 j: tile j has landed
      uint4 w[2][2];
      uint32_t sc_lo = 0, sc_hi = 0;
      if (has_chunk) {
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int h = 0; h < 2; ++h)
            w[n][h] = *reinterpret_cast<const uint4*>(wring + (st * kDecodeTileRows + g + 8 * h) * kDecodeRowPitch +
                                                      warp * (kDecodeChunkK / 2) + 64 * (n ^ (g & 1)) + 16 * q);
        // Odd rows fetched step 1 first (their rows start in the same banks as the even row next
        // to them, and a quarter warp holds one even and one odd row): put the steps back in order.
        if (g & 1) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint4 t = w[0][h];
            w[0][h] = w[1][h];
            w[1][h] = t;
          }
        }
        // the chunk's two groups are adjacent f16 in the row's scale vector
        const uint8_t* stile = sring + st * kDecodeMaxScaleBytes + (((kc - 0) >> 7) << 1);
        sc_lo = *reinterpret_cast<const uint32_t*>(stile + g * (groups_per_row << 1));
        sc_hi = *reinterpret_cast<const uint32_t*>(stile + (g + 8) * (groups_per_row << 1));
      }
      __syncwarp();  // the whole warp has read this stage
      if (lane == 0) mbar_arrive(wempty_bar(st));
      // Refill: the stage that tile j - 1 used is free once every warp has read it, which is
      // almost always already the case here.
      if (j >= 1 && !produce(j + kDecodeStages - 1)) break;
      DECODE_STAMP();  // 5 + 5 j: weights in registers, refill requested

      float acc[MH][4];
#pragma unroll
      for (int mh = 0; mh < MH; ++mh)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[mh][c] = 0.f;
      if (has_chunk) {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          float d[MH][4];
#pragma unroll
          for (int mh = 0; mh < MH; ++mh)
#pragma unroll
            for (int c = 0; c < 4; ++c) d[mh][c] = 0.f;
          const uint32_t wl[4] = {w[s][0].x, w[s][0].y, w[s][0].z, w[s][0].w};  // weight row g
          const uint32_t wh[4] = {w[s][1].x, w[s][1].y, w[s][1].z, w[s][1].w};  // weight row g + 8
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
          // One step is exactly one scale group of rows g and g + 8.
          const float s_lo = __half2float(__ushort_as_half(static_cast<uint16_t>(s ? (sc_lo >> 16) : (sc_lo & 0xffff))));
          const float s_hi = __half2float(__ushort_as_half(static_cast<uint16_t>(s ? (sc_hi >> 16) : (sc_hi & 0xffff))));
#pragma unroll
          for (int mh = 0; mh < MH; ++mh) {
            const float2 off = MH == 2 ? bias_smem[(2 * mh + s) * 32] : make_float2(bias[mh][s][0], bias[mh][s][1]);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const float group_sum = d[mh][c] - ((c & 1) ? off.y : off.x);
              acc[mh][c] = fmaf(c < 2 ? s_lo : s_hi, group_sum, acc[mh][c]);
            }
          }
        }
      }
      DECODE_STAMP();  // 6 + 5 j: MMAs issued and group sums folded

      // ---- leave this K chunk's partial sums in the tile's slot ------------------------------------
      {
        const int slot = j % kDecodeSlots;
        if (!__all_sync(0xffffffffu, mbar_wait<false>(pempty_bar(slot), ((j / kDecodeSlots) & 1) ^ 1, abort_flag))) {
          *abort_flag = 1;
          break;
        }
        if (has_chunk) {
#pragma unroll
          for (int mh = 0; mh < MH; ++mh)
            partial_cell(slot, warp, lane)[mh] = make_float4(acc[mh][0], acc[mh][1], acc[mh][2], acc[mh][3]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(pfull_bar(slot));
      }
      DECODE_STAMP();  // 7 + 5 j: partial sums handed over
      // Tile j - 2 is finished off by warp (j - 2) % 16: by now every chunk has arrived, so the wait
      // is short, and no warp needs another warp's answer on its critical path.
      if (j >= 2 && warp == (j - 2) % kDecodeWarps) ok = finalize(j - 2);
      DECODE_STAMP();  // 8 + 5 j: finalizer duty (if any) done
    }
    for (int jf = my_tiles > 2 ? my_tiles - 2 : 0; jf < my_tiles && ok; ++jf)
      if (warp == jf % kDecodeWarps && !*abort_flag) ok = finalize(jf);
    DECODE_STAMP();  // last: all tiles reduced
    if (*abort_flag) dead = true;
  }  // pass
}

}  // namespace b200
