// CPU oracle for the contraction dispatches. TEST INFRASTRUCTURE ONLY.
//
// This file is a plain-C restatement of what the reference computes on its llvm-cpu path for
// a contraction dispatch. It is loaded by tests/, by the smoke check and by the CPU-baseline
// leg of bench.py. Nothing in the shipped package links, loads or calls it.
//
// Parity status:
//   * pack / mmt4d / unpack and the matmul chains built from them are PINNED: the tests
//     compare them bit-for-bit with the reference's own ukernels (compiled from the
//     reference sources into oracle/_ref/libiree_uk.so) on the shapes of
//     runtime/src/iree/builtins/ukernel/tools/mmt4d_test.c:449-504 and on the e2e shape sets
//     of tests/e2e/matmul/generate_e2e_matmul_tests.py:125-198.
//   * the grouped int4 dequant + contraction and the W8A8 requant epilogue have no numeric
//     golden in the reference (llvm-cpu generates that code; it is not a ukernel):
//     PARITY UNPINNED beyond the element-order fixture tests/e2e/linalg/subbyte_to_fp.mlir
//     and the linalg bodies of
//     compiler/src/iree/compiler/Dialect/Flow/Transforms/test/pipeline_tests.mlir:53-78.
//
// Floating point: f16 <-> f32 conversions use the compiler's _Float16 (IEEE round to nearest
// even, subnormals kept), which is what the reference's AVX-512 tiles (vcvtph2ps/vcvtps2ph,
// arch/x86_64/mmt4d_x86_64_avx512_base.c:68-131) and llvm-cpu's truncf do. The reference's
// portable software conversion (builtins/ukernel/common.h:700-790) flushes subnormals; the
// two agree on every normal value. Built with -std=c11 so a*b+c is never contracted to an FMA.

#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef int64_t idx_t;

enum {
  ORACLE_TYPE_F32F32F32 = 1,  // numbering follows IREE_UK_FLAG_MMT4D_TYPE_* (exported_bits.h:29-42)
  ORACLE_TYPE_S8S8S32 = 2,
  ORACLE_TYPE_F16F16F32 = 3,
  ORACLE_TYPE_BF16BF16F32 = 5,
};

static inline float f16_to_f32(uint16_t h) {
  _Float16 v;
  memcpy(&v, &h, 2);
  return (float)v;
}
static inline uint16_t f32_to_f16(float f) {
  _Float16 v = (_Float16)f;
  uint16_t h;
  memcpy(&h, &v, 2);
  return h;
}
static inline float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
// Round to nearest even by adding a bias before truncating, as common.h:744-752 does.
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return (uint16_t)((u >> 16) | ((u & 0xffffu) ? 0x40 : 0));
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

uint16_t oracle_f32_to_f16(float f) { return f32_to_f16(f); }
float oracle_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
uint16_t oracle_f32_to_bf16(float f) { return f32_to_bf16(f); }
float oracle_bf16_to_f32(uint16_t b) { return bf16_to_f32(b); }
// Array forms: which = 0 f16 -> f32, 1 f32 -> f16, 2 bf16 -> f32, 3 f32 -> bf16.
void oracle_convert_n(int which, const void* in, void* out, idx_t n) {
  for (idx_t i = 0; i < n; ++i) {
    if (which == 0) ((float*)out)[i] = f16_to_f32(((const uint16_t*)in)[i]);
    else if (which == 1) ((uint16_t*)out)[i] = f32_to_f16(((const float*)in)[i]);
    else if (which == 2) ((float*)out)[i] = bf16_to_f32(((const uint16_t*)in)[i]);
    else ((uint16_t*)out)[i] = f32_to_bf16(((const float*)in)[i]);
  }
}

static int lhs_elem_size(int type) {
  switch (type) {
    case ORACLE_TYPE_F32F32F32: return 4;
    case ORACLE_TYPE_S8S8S32: return 1;
    default: return 2;
  }
}

// ---------------------------------------------------------------------------------------
// pack: row-major 2-D -> 4-D tiled, zero (or pattern) padded.
// Follows iree_uk_pack (builtins/ukernel/pack.h:26-34, pack.c, pack_tile.c:9-75).
// out has shape [out0][out1][out2][out3] in memory. TRANSPOSE_OUTER swaps which input
// dimension the two outer indices walk; TRANSPOSE_INNER does the same for the inner ones
// (exported_bits.h:64-66). Strides are in elements.
// ---------------------------------------------------------------------------------------
void oracle_pack(const void* in, idx_t in_size0, idx_t in_size1, idx_t in_stride0,
                 void* out, idx_t out0, idx_t out1, idx_t out2, idx_t out3,
                 idx_t out_stride0, int elem_size, int transpose_inner,
                 int transpose_outer, uint64_t padding_value) {
  const char* src = (const char*)in;
  char* dst = (char*)out;
  for (idx_t a = 0; a < out0; ++a)
    for (idx_t b = 0; b < out1; ++b)
      for (idx_t c = 0; c < out2; ++c)
        for (idx_t d = 0; d < out3; ++d) {
          idx_t outer0 = transpose_outer ? b : a, outer1 = transpose_outer ? a : b;
          idx_t tile0 = transpose_inner ? out3 : out2, tile1 = transpose_inner ? out2 : out3;
          idx_t inner0 = transpose_inner ? d : c, inner1 = transpose_inner ? c : d;
          idx_t r = outer0 * tile0 + inner0, col = outer1 * tile1 + inner1;
          char* o = dst + (a * out_stride0 + b * out2 * out3 + c * out3 + d) * elem_size;
          if (r < in_size0 && col < in_size1)
            memcpy(o, src + (r * in_stride0 + col) * elem_size, elem_size);
          else
            memcpy(o, &padding_value, elem_size);  // little-endian low bytes, as pack.h:14-17
        }
}

// unpack: the inverse, dropping the padding. Follows iree_uk_unpack (unpack.h:17-25).
void oracle_unpack(const void* in, idx_t in0, idx_t in1, idx_t in2, idx_t in3,
                   idx_t in_stride0, void* out, idx_t out_size0, idx_t out_size1,
                   idx_t out_stride0, int elem_size, int transpose_inner,
                   int transpose_outer) {
  const char* src = (const char*)in;
  char* dst = (char*)out;
  for (idx_t a = 0; a < in0; ++a)
    for (idx_t b = 0; b < in1; ++b)
      for (idx_t c = 0; c < in2; ++c)
        for (idx_t d = 0; d < in3; ++d) {
          idx_t outer0 = transpose_outer ? b : a, outer1 = transpose_outer ? a : b;
          idx_t tile0 = transpose_inner ? in3 : in2, tile1 = transpose_inner ? in2 : in3;
          idx_t inner0 = transpose_inner ? d : c, inner1 = transpose_inner ? c : d;
          idx_t r = outer0 * tile0 + inner0, col = outer1 * tile1 + inner1;
          if (r < out_size0 && col < out_size1)
            memcpy(dst + (r * out_stride0 + col) * elem_size,
                   src + (a * in_stride0 + b * in2 * in3 + c * in3 + d) * elem_size, elem_size);
        }
}

// ---------------------------------------------------------------------------------------
// mmt4d: out[i,j,i0,j0] (+)= sum_k sum_k0 lhs[i,k,i0,k0] * rhs[j,k,j0,k0]
// Follows iree_uk_mmt4d (mmt4d.h:14-21, outer loops mmt4d.c:55-99) with the generic tile
// bodies: s8s8s32 mmt4d_tile_generic.c:54-78, f16f16f32 :199-225 (sequential f32
// accumulation over k then k0, operands widened first). Strides are in elements.
// ---------------------------------------------------------------------------------------
void oracle_mmt4d(int type, const void* lhs, idx_t lhs_stride0, const void* rhs,
                  idx_t rhs_stride0, void* out, idx_t out_stride0, idx_t M1, idx_t N1,
                  idx_t K1, int M0, int N0, int K0, int accumulate) {
  for (idx_t i = 0; i < M1; ++i)
    for (idx_t j = 0; j < N1; ++j)
      for (int i0 = 0; i0 < M0; ++i0)
        for (int j0 = 0; j0 < N0; ++j0) {
          idx_t o = i * out_stride0 + j * M0 * N0 + i0 * N0 + j0;
          if (type == ORACLE_TYPE_S8S8S32) {
            const int8_t* l = (const int8_t*)lhs + i * lhs_stride0;
            const int8_t* r = (const int8_t*)rhs + j * rhs_stride0;
            int32_t acc = accumulate ? ((int32_t*)out)[o] : 0;
            for (idx_t k = 0; k < K1; ++k)
              for (int k0 = 0; k0 < K0; ++k0)
                acc += (int32_t)l[k * M0 * K0 + i0 * K0 + k0] * (int32_t)r[k * N0 * K0 + j0 * K0 + k0];
            ((int32_t*)out)[o] = acc;
          } else {
            float acc = accumulate ? ((float*)out)[o] : 0.f;
            for (idx_t k = 0; k < K1; ++k)
              for (int k0 = 0; k0 < K0; ++k0) {
                idx_t li = i * lhs_stride0 + k * M0 * K0 + i0 * K0 + k0;
                idx_t ri = j * rhs_stride0 + k * N0 * K0 + j0 * K0 + k0;
                float a, b;
                if (type == ORACLE_TYPE_F32F32F32) {
                  a = ((const float*)lhs)[li];
                  b = ((const float*)rhs)[ri];
                } else if (type == ORACLE_TYPE_F16F16F32) {
                  a = f16_to_f32(((const uint16_t*)lhs)[li]);
                  b = f16_to_f32(((const uint16_t*)rhs)[ri]);
                } else {
                  a = bf16_to_f32(((const uint16_t*)lhs)[li]);
                  b = bf16_to_f32(((const uint16_t*)rhs)[ri]);
                }
                acc += a * b;
              }
            ((float*)out)[o] = acc;
          }
        }
}

// ---------------------------------------------------------------------------------------
// The data-tiled matmul llvm-cpu runs: pack(LHS) + pack(RHS, both transposes) + mmt4d +
// unpack, chained exactly like builtins/ukernel/tools/e2e_matmul_benchmark.c:173-286.
// lhs is [M,K] row-major, rhs is [K,N] row-major, out is [M,N] row-major in the accumulator
// type (i32 or f32). With accumulate != 0 the existing out is packed first and added to.
// ---------------------------------------------------------------------------------------
int oracle_matmul_data_tiled(int type, idx_t M, idx_t N, idx_t K, const void* lhs,
                             const void* rhs, void* out, int M0, int N0, int K0,
                             int accumulate) {
  const int es = lhs_elem_size(type);
  const idx_t M1 = (M + M0 - 1) / M0, N1 = (N + N0 - 1) / N0, K1 = (K + K0 - 1) / K0;
  const idx_t ls0 = K1 * M0 * K0, rs0 = K1 * N0 * K0, os0 = N1 * M0 * N0;
  void* pl = calloc((size_t)(M1 * ls0 + 1), es);
  void* pr = calloc((size_t)(N1 * rs0 + 1), es);
  void* po = calloc((size_t)(M1 * os0 + 1), 4);
  if (!pl || !pr || !po) {
    free(pl); free(pr); free(po);
    return 1;
  }
  oracle_pack(lhs, M, K, K, pl, M1, K1, M0, K0, ls0, es, 0, 0, 0);
  oracle_pack(rhs, K, N, N, pr, N1, K1, N0, K0, rs0, es, 1, 1, 0);
  if (accumulate) oracle_pack(out, M, N, N, po, M1, N1, M0, N0, os0, 4, 0, 0, 0);
  oracle_mmt4d(type, pl, ls0, pr, rs0, po, os0, M1, N1, K1, M0, N0, K0, accumulate);
  oracle_unpack(po, M1, N1, M0, N0, os0, out, M, N, N, 4, 0, 0);
  free(pl); free(pr); free(po);
  return 0;
}

// Naive row-major matmul with sequential accumulation over k, the whole-dispatch reference
// of tools/testing/e2e/iree-e2e-matmul-test.cc:28-131. Used to cross-check the tiled chain.
void oracle_matmul_naive(int type, idx_t M, idx_t N, idx_t K, const void* lhs,
                         const void* rhs, void* out, int accumulate) {
  for (idx_t m = 0; m < M; ++m)
    for (idx_t n = 0; n < N; ++n) {
      if (type == ORACLE_TYPE_S8S8S32) {
        int32_t acc = accumulate ? ((int32_t*)out)[m * N + n] : 0;
        for (idx_t k = 0; k < K; ++k)
          acc += (int32_t)((const int8_t*)lhs)[m * K + k] * (int32_t)((const int8_t*)rhs)[k * N + n];
        ((int32_t*)out)[m * N + n] = acc;
      } else {
        float acc = accumulate ? ((float*)out)[m * N + n] : 0.f;
        for (idx_t k = 0; k < K; ++k) {
          float a, b;
          if (type == ORACLE_TYPE_F32F32F32) {
            a = ((const float*)lhs)[m * K + k];
            b = ((const float*)rhs)[k * N + n];
          } else if (type == ORACLE_TYPE_F16F16F32) {
            a = f16_to_f32(((const uint16_t*)lhs)[m * K + k]);
            b = f16_to_f32(((const uint16_t*)rhs)[k * N + n]);
          } else {
            a = bf16_to_f32(((const uint16_t*)lhs)[m * K + k]);
            b = bf16_to_f32(((const uint16_t*)rhs)[k * N + n]);
          }
          acc += a * b;
        }
        ((float*)out)[m * N + n] = acc;
      }
    }
}

// truncf consumer fused after unpack (FormDispatchRegions.cpp:548-573): f32 -> f16 / bf16.
void oracle_truncf(const float* in, uint16_t* out, idx_t count, int to_bf16) {
  for (idx_t i = 0; i < count; ++i) out[i] = to_bf16 ? f32_to_bf16(in[i]) : f32_to_f16(in[i]);
}

// W8A8 requant consumer: out[m,n] = f16( (f32(acc[m,n]) * a_scale[m]) * w_scale[n] ), the
// elementwise generic (sitofp, mulf, mulf, truncf) that fuses with unpack.
void oracle_requant_f16(const int32_t* acc, const float* a_scale, const float* w_scale,
                        uint16_t* out, idx_t M, idx_t N) {
  for (idx_t m = 0; m < M; ++m)
    for (idx_t n = 0; n < N; ++n) {
      float v = (float)acc[m * N + n];
      v = v * a_scale[m];
      v = v * w_scale[n];
      out[m * N + n] = f32_to_f16(v);
    }
}

// ---------------------------------------------------------------------------------------
// Fused int4 dequant + grouped contraction (the dispatch of pipeline_tests.mlir:53-99 with
// extsi and no zero point; dequant arithmetic in f16 as in
// compiler/src/iree/compiler/Codegen/LLVMGPU/test/config_matvec.mlir:134-141).
//   wq      : [N, K/2] bytes; element 2i is the low nibble of byte i, 2i+1 the high nibble
//             (mmt4d_tile_generic.c:35-44, tests/e2e/linalg/subbyte_to_fp.mlir:1-40)
//   scales  : [N, K/group] f16
//   a       : [M, K] f16
//   dequant : w_f16[n,g,k] = f16( f16(sext(wq)) * scales[n,g] )          (one f16 rounding)
//   contract: c[m,n] = sum_g sum_k f32(a[m,g,k]) * f32(w_f16[n,g,k])     (sequential f32)
//   out     : f16(c)
// ---------------------------------------------------------------------------------------
static inline int sext4(unsigned nib) { return (int)((nib ^ 8u) & 0xfu) - 8; }

static void w4a16_rows(const uint16_t* a, const uint8_t* wq, const uint16_t* scales,
                       uint16_t* out, idx_t M, idx_t N, idx_t K, int group, idx_t n_begin,
                       idx_t n_end) {
  const idx_t G = K / group;
  float* wrow = (float*)malloc(sizeof(float) * (size_t)K);
  for (idx_t n = n_begin; n < n_end; ++n) {
    for (idx_t g = 0; g < G; ++g) {
      float s = f16_to_f32(scales[n * G + g]);
      for (int k = 0; k < group; ++k) {
        idx_t kk = g * group + k;
        uint8_t byte = wq[n * (K / 2) + kk / 2];
        int w = sext4((kk & 1) ? (byte >> 4) : (byte & 0xf));
        // f16*f16 is exact in f32 (11+11 significand bits), so rounding the f32 product
        // once gives the IEEE f16 product.
        wrow[kk] = f16_to_f32(f32_to_f16((float)w * s));
      }
    }
    for (idx_t m = 0; m < M; ++m) {
      float acc = 0.f;
      const uint16_t* am = a + m * K;
      for (idx_t kk = 0; kk < K; ++kk) acc += f16_to_f32(am[kk]) * wrow[kk];
      out[m * N + n] = f32_to_f16(acc);
    }
  }
  free(wrow);
}

typedef struct {
  const uint16_t* a; const uint8_t* wq; const uint16_t* scales; uint16_t* out;
  idx_t M, N, K; int group; idx_t n_begin, n_end;
} w4_job_t;

static void* w4_thread(void* p) {
  w4_job_t* j = (w4_job_t*)p;
  w4a16_rows(j->a, j->wq, j->scales, j->out, j->M, j->N, j->K, j->group, j->n_begin, j->n_end);
  return NULL;
}

// `threads` strips of output columns, one pthread each (N is the parallel dimension, as in
// the reference's workgroup distribution of contraction dispatches).
int oracle_w4a16(const uint16_t* a, const uint8_t* wq, const uint16_t* scales, uint16_t* out,
                 idx_t M, idx_t N, idx_t K, int group, int threads) {
  if (group <= 0 || K % group || (K & 1)) return 1;
  if (threads < 1) threads = 1;
  if (threads > 256) threads = 256;
  pthread_t tid[256];
  w4_job_t jobs[256];
  idx_t per = (N + threads - 1) / threads;
  int started = 0;
  for (int t = 0; t < threads; ++t) {
    idx_t b = t * per, e = b + per < N ? b + per : N;
    if (b >= e) break;
    jobs[t] = (w4_job_t){a, wq, scales, out, M, N, K, group, b, e};
    if (t == threads - 1 || e == N) {  // run the last strip on the calling thread
      w4_thread(&jobs[t]);
      break;
    }
    pthread_create(&tid[t], NULL, w4_thread, &jobs[t]);
    ++started;
  }
  for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
  return 0;
}

// i4 -> f32 element values in memory order; checks the nibble order fixture.
void oracle_unpack_i4(const uint8_t* bytes, idx_t count, float* out) {
  for (idx_t i = 0; i < count; ++i) {
    uint8_t b = bytes[i / 2];
    out[i] = (float)sext4((i & 1) ? (b >> 4) : (b & 0xf));
  }
}
