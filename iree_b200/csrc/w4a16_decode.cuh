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
constexpr int kDecodeChunkK = 256;                          // K per warp
constexpr int kDecodeSliceK = kDecodeWarps * kDecodeChunkK;  // K per CTA: 4096
constexpr int kDecodeTileRows = 16;                         // weight rows per tile
constexpr int kDecodePrefetch = 2;                          // tiles of weights in flight per thread

// Scratch for the split-K reduction: f32 partial sums [16][n_pad] followed by one arrival
// counter per 16-row tile. Must be zero before the first launch; the last-arriving CTA of a
// tile reads the sums, writes the result and zeroes what it used.
struct DecodeScratchLayout {
  __host__ __device__ static size_t partial_floats(int N) { return static_cast<size_t>(16) * N; }
  __host__ __device__ static size_t bytes(int N) { return partial_floats(N) * 4 + static_cast<size_t>(N / 16) * 4; }
};

template <int MH>
__device__ __forceinline__ void decode_body(const __half* __restrict__ a, const uint8_t* __restrict__ wq,
                                            const __half* __restrict__ scales, __half* __restrict__ out,
                                            float* __restrict__ scratch, int M, int N, int K, int ldo, int n_off) {
  __shared__ float red[2][kDecodeWarps][32][4 * MH];
  __shared__ int last_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int ksplit = gridDim.y;
  const int k_slice0 = blockIdx.y * kDecodeSliceK;
  const int kc = k_slice0 + warp * kDecodeChunkK;  // this warp's K chunk
  const bool active = kc < K;                      // K is a multiple of 256
  const int groups_per_row = K >> 7;
  const int row_bytes = K >> 1;
  const int num_tiles = N / kDecodeTileRows;

  // ---- activations of this warp's chunk, kept in registers in the order the MMAs want -------------
  // For step s, word i: the thread's eight k are k0 = kc + 128 s + 32 q + 8 i .. k0 + 7. The weight
  // unpack yields pairs (0,4), (1,5), (2,6), (3,7); the activations are paired the same way.
  uint32_t bfrag[MH][2][4][4];  // [m half][step][word][(0,4), (1,5), (2,6), (3,7)]
#pragma unroll
  for (int mh = 0; mh < MH; ++mh) {
    const int m = g + 8 * mh;
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 x = make_uint4(0, 0, 0, 0);
        if (active && m < M) x = *reinterpret_cast<const uint4*>(a + static_cast<size_t>(m) * K + kc + 128 * s + 32 * q + 8 * i);
        // x.x = (e0,e1), x.y = (e2,e3), x.z = (e4,e5), x.w = (e6,e7)
        bfrag[mh][s][i][0] = __byte_perm(x.x, x.z, 0x5410);  // (e0, e4)
        bfrag[mh][s][i][1] = __byte_perm(x.x, x.z, 0x7632);  // (e1, e5)
        bfrag[mh][s][i][2] = __byte_perm(x.y, x.w, 0x5410);  // (e2, e6)
        bfrag[mh][s][i][3] = __byte_perm(x.y, x.w, 0x7632);  // (e3, e7)
      }
  }

  // ---- weight prefetch ring --------------------------------------------------------------------
  uint4 wreg[kDecodePrefetch][2][2];      // [slot][step][row g / row g+8]
  uint16_t sreg[kDecodePrefetch][2][2];   // matching scales
  auto issue = [&](int slot, int tile) {
    if (!active || tile >= num_tiles) return;
    const int r0 = tile * kDecodeTileRows + g;
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const size_t row = static_cast<size_t>(r0 + 8 * h);
        wreg[slot][s][h] = ld_stream_v4(wq + row * row_bytes + (kc >> 1) + 64 * s + 16 * q);
        sreg[slot][s][h] = __ldg(reinterpret_cast<const uint16_t*>(scales) + row * groups_per_row + (kc >> 7) + s);
      }
  };

#pragma unroll
  for (int p = 0; p < kDecodePrefetch; ++p) issue(p, blockIdx.x + p * gridDim.x);

  int iter = 0;
  for (int tile0 = blockIdx.x; tile0 < num_tiles; tile0 += kDecodePrefetch * gridDim.x) {
#pragma unroll
    for (int p = 0; p < kDecodePrefetch; ++p) {
      const int tile = tile0 + p * gridDim.x;
      if (tile >= num_tiles) break;
      float acc[MH][4];
#pragma unroll
      for (int mh = 0; mh < MH; ++mh)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[mh][c] = 0.f;
      if (active) {
        uint4 w[2][2];
        uint16_t sc[2][2];
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            w[s][h] = wreg[p][s][h];
            sc[s][h] = sreg[p][s][h];
          }
        issue(p, tile + kDecodePrefetch * gridDim.x);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          float d[MH][4];
#pragma unroll
          for (int mh = 0; mh < MH; ++mh)
#pragma unroll
            for (int c = 0; c < 4; ++c) d[mh][c] = 0.f;
          const uint32_t wl[4] = {w[s][0].x, w[s][0].y, w[s][0].z, w[s][0].w};
          const uint32_t wh[4] = {w[s][1].x, w[s][1].y, w[s][1].z, w[s][1].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            __half2 pl[4], ph[4];
            unpack8_strided(wl[i], pl);  // weight row g
            unpack8_strided(wh[i], ph);  // weight row g + 8
#pragma unroll
            for (int mh = 0; mh < MH; ++mh) {
              mma_m16n8k16(d[mh], as_u32(pl[0]), as_u32(ph[0]), as_u32(pl[1]), as_u32(ph[1]), bfrag[mh][s][i][0],
                           bfrag[mh][s][i][1]);
              mma_m16n8k16(d[mh], as_u32(pl[2]), as_u32(ph[2]), as_u32(pl[3]), as_u32(ph[3]), bfrag[mh][s][i][2],
                           bfrag[mh][s][i][3]);
            }
          }
          // One step is exactly one scale group of rows g and g + 8.
          const float s_lo = __half2float(__ushort_as_half(sc[s][0]));
          const float s_hi = __half2float(__ushort_as_half(sc[s][1]));
#pragma unroll
          for (int mh = 0; mh < MH; ++mh) {
            acc[mh][0] = fmaf(s_lo, d[mh][0], acc[mh][0]);
            acc[mh][1] = fmaf(s_lo, d[mh][1], acc[mh][1]);
            acc[mh][2] = fmaf(s_hi, d[mh][2], acc[mh][2]);
            acc[mh][3] = fmaf(s_hi, d[mh][3], acc[mh][3]);
          }
        }
      }
      // ---- reduce the 16 K-chunks through shared memory ----------------------------------------
      const int buf = iter & 1;
      ++iter;
#pragma unroll
      for (int mh = 0; mh < MH; ++mh)
        *reinterpret_cast<float4*>(&red[buf][warp][lane][4 * mh]) =
            make_float4(acc[mh][0], acc[mh][1], acc[mh][2], acc[mh][3]);
      __syncthreads();
      // Thread t < 128 * MH owns output (m = t / 16, weight row r = t % 16) of this tile.
      const int t = threadIdx.x;
      const bool owner = t < 128 * MH;
      const int m = t >> 4, r = t & 15;
      float sum = 0.f;
      if (owner) {
        const int src_lane = (r & 7) * 4 + ((m & 7) >> 1);
        const int src_reg = (m >> 3) * 4 + (r >> 3) * 2 + (m & 1);
#pragma unroll
        for (int w2 = 0; w2 < kDecodeWarps; ++w2) sum += red[buf][w2][src_lane][src_reg];
      }
      const int n = tile * kDecodeTileRows + r;
      if (ksplit == 1) {
        if (owner && m < M) out[static_cast<size_t>(m) * ldo + n_off + n] = __float2half_rn(sum);
      } else {
        float* partial = scratch;
        int* counters = reinterpret_cast<int*>(scratch + DecodeScratchLayout::partial_floats(N));
        if (owner) atomicAdd(&partial[static_cast<size_t>(m) * N + n], sum);
        __threadfence();
        __syncthreads();
        if (t == 0) last_flag = (atomicAdd(&counters[tile], 1) == ksplit - 1);
        __syncthreads();
        if (last_flag) {
          __threadfence();
          if (owner) {
            float* cell = &partial[static_cast<size_t>(m) * N + n];
            const float total = __ldcg(cell);
            if (m < M) out[static_cast<size_t>(m) * ldo + n_off + n] = __float2half_rn(total);
            __stcg(cell, 0.f);  // leave the scratch clean for the next launch
          }
          if (t == 0) counters[tile] = 0;
        }
      }
    }
  }
}

}  // namespace b200
