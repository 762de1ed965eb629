// Driver that runs the REFERENCE's own ukernels (oracle/_ref/libiree_uk.so, compiled from the
// reference sources where they lie) the way llvm-cpu runs a data-tiled matmul:
//   pack(LHS) -> pack(RHS, transposed) -> iree_uk_mmt4d -> unpack
// chained as builtins/ukernel/tools/e2e_matmul_benchmark.c:173-286 does, with the M1 x N1
// outer tiles split over a pthread pool in contiguous strips (the role the local-task
// workgroup distribution of Codegen/LLVMCPU/KernelDispatch.cpp:1519-1573 plays).
// TEST INFRASTRUCTURE ONLY: used to pin oracle/contraction_oracle.c and as the timed CPU
// baseline. Built into oracle/_ref/ (never committed), needs the reference headers.

#define _POSIX_C_SOURCE 200809L
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "iree/builtins/ukernel/api.h"
#include "iree/builtins/ukernel/exported_bits.h"

static double now_s(void) {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

// cpu_data field 0 for this host, bit positions from
// runtime/src/iree/schemas/cpu_feature_bits.inl:85-117. mode 0 = no features (forces the
// generic tile functions), 1 = what the host supports.
uint64_t uk_chain_cpu_data0(int mode) {
  if (!mode) return 0;
  uint64_t d = 0;
  __builtin_cpu_init();
  if (__builtin_cpu_supports("fma")) d |= 1ull << 11;
  if (__builtin_cpu_supports("f16c")) d |= 1ull << 14;
  if (__builtin_cpu_supports("avx2")) d |= 1ull << 15;
  if (__builtin_cpu_supports("avx512f")) d |= 1ull << 20;
  if (__builtin_cpu_supports("avx512cd")) d |= 1ull << 21;
  if (__builtin_cpu_supports("avx512vl")) d |= 1ull << 22;
  if (__builtin_cpu_supports("avx512dq")) d |= 1ull << 23;
  if (__builtin_cpu_supports("avx512bw")) d |= 1ull << 24;
  if (__builtin_cpu_supports("avx512vnni")) d |= 1ull << 28;
  if (__builtin_cpu_supports("avx512bf16")) d |= 1ull << 31;
  return d;
}

static int elem_size_of(uint32_t mmt4d_type) {
  switch (mmt4d_type) {
    case IREE_UK_FLAG_MMT4D_TYPE_F32F32F32: return 4;
    case IREE_UK_FLAG_MMT4D_TYPE_S8S8S32: return 1;
    default: return 2;
  }
}
static uint32_t pack_flag_of(uint32_t mmt4d_type) {
  switch (mmt4d_type) {
    case IREE_UK_FLAG_MMT4D_TYPE_F32F32F32: return IREE_UK_FLAG_PACK_TYPE_F32F32;
    case IREE_UK_FLAG_MMT4D_TYPE_S8S8S32: return IREE_UK_FLAG_PACK_TYPE_I8I8;
    case IREE_UK_FLAG_MMT4D_TYPE_F16F16F32: return IREE_UK_FLAG_PACK_TYPE_F16F16;
    default: return IREE_UK_FLAG_PACK_TYPE_BF16BF16;
  }
}

typedef struct {
  uint32_t type;
  const void *pl, *pr;
  void* po;
  int64_t M1, N1, K1;
  int M0, N0, K0;
  int64_t ls0, rs0, os0;
  int64_t i_begin, i_end;  // strip of M1 (or of N1 when M1 is too small to split)
  int split_n;
  uint32_t flags;
  const iree_uk_uint64_t* cpu_data;
} mm_job_t;

static void* mm_thread(void* p) {
  mm_job_t* j = (mm_job_t*)p;
  const int es = elem_size_of(j->type);
  if (!j->split_n) {
    iree_uk_mmt4d((const char*)j->pl + j->i_begin * j->ls0 * es, 0, j->ls0, j->pr, 0, j->rs0,
                  (char*)j->po + j->i_begin * j->os0 * 4, 0, j->os0, j->i_end - j->i_begin, j->N1,
                  j->K1, j->M0, j->N0, j->K0, j->flags, j->cpu_data);
  } else {
    iree_uk_mmt4d(j->pl, 0, j->ls0, (const char*)j->pr + j->i_begin * j->rs0 * es, 0, j->rs0,
                  (char*)j->po + j->i_begin * j->M0 * j->N0 * 4, 0, j->os0, j->M1,
                  j->i_end - j->i_begin, j->K1, j->M0, j->N0, j->K0, j->flags, j->cpu_data);
  }
  return NULL;
}

// out is [M,N] row-major i32 / f32. times[0..3] = seconds for pack lhs, pack rhs, mmt4d,
// unpack (may be NULL). Returns 0 on success.
int uk_chain_matmul(uint32_t mmt4d_type, int64_t M, int64_t N, int64_t K, const void* lhs,
                    const void* rhs, void* out, int M0, int N0, int K0, int accumulate,
                    int cpu_mode, int threads, double* times) {
  iree_uk_uint64_t cpu_data[8] = {0};
  cpu_data[0] = uk_chain_cpu_data0(cpu_mode);
  const int es = elem_size_of(mmt4d_type);
  const int64_t M1 = (M + M0 - 1) / M0, N1 = (N + N0 - 1) / N0, K1 = (K + K0 - 1) / K0;
  const int64_t ls0 = K1 * M0 * K0, rs0 = K1 * N0 * K0, os0 = N1 * M0 * N0;
  void* pl = malloc((size_t)(M1 * ls0 + 1) * es);
  void* pr = malloc((size_t)(N1 * rs0 + 1) * es);
  void* po = malloc((size_t)(M1 * os0 + 1) * 4);
  if (!pl || !pr || !po) {
    free(pl); free(pr); free(po);
    return 1;
  }
  const uint32_t pflag = pack_flag_of(mmt4d_type);
  const uint32_t oflag_pack = mmt4d_type == IREE_UK_FLAG_MMT4D_TYPE_S8S8S32
                                  ? IREE_UK_FLAG_PACK_TYPE_I32I32 : IREE_UK_FLAG_PACK_TYPE_F32F32;
  const uint32_t oflag_unpack = mmt4d_type == IREE_UK_FLAG_MMT4D_TYPE_S8S8S32
                                    ? IREE_UK_FLAG_UNPACK_TYPE_I32I32 : IREE_UK_FLAG_UNPACK_TYPE_F32F32;
  double t0 = now_s();
  iree_uk_pack(lhs, 0, K, 1, pl, 0, ls0, (int64_t)M0 * K0, M, K, M1, K1, M0, K0, 0, pflag, cpu_data);
  double t1 = now_s();
  iree_uk_pack(rhs, 0, N, 1, pr, 0, rs0, (int64_t)N0 * K0, K, N, N1, K1, N0, K0, 0,
               pflag | IREE_UK_FLAG_PACK_TRANSPOSE_INNER | IREE_UK_FLAG_PACK_TRANSPOSE_OUTER, cpu_data);
  if (accumulate)
    iree_uk_pack(out, 0, N, 1, po, 0, os0, (int64_t)M0 * N0, M, N, M1, N1, M0, N0, 0, oflag_pack, cpu_data);
  double t2 = now_s();

  uint32_t flags = mmt4d_type | IREE_UK_FLAG_MMT4D_ALLOW_GENERIC_FALLBACK_TILE_FUNCTION |
                   IREE_UK_FLAG_MMT4D_SKIP_INTERMEDIATE_ROUNDINGS |
                   (accumulate ? IREE_UK_FLAG_MMT4D_ACCUMULATE : 0);
  if (threads < 1) threads = 1;
  if (threads > 256) threads = 256;
  const int split_n = M1 < threads;
  const int64_t extent = split_n ? N1 : M1;
  if (threads > extent) threads = extent > 0 ? (int)extent : 1;
  pthread_t tid[256];
  mm_job_t jobs[256];
  int started = 0;
  for (int t = 0; t < threads; ++t) {
    int64_t b = extent * t / threads, e = extent * (t + 1) / threads;
    jobs[t] = (mm_job_t){mmt4d_type, pl, pr, po, M1, N1, K1, M0, N0, K0, ls0, rs0, os0,
                         b, e, split_n, flags, cpu_data};
    if (t == threads - 1) {
      mm_thread(&jobs[t]);
    } else {
      pthread_create(&tid[t], NULL, mm_thread, &jobs[t]);
      ++started;
    }
  }
  for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
  double t3 = now_s();
  iree_uk_unpack(po, 0, os0, (int64_t)M0 * N0, out, 0, N, 1, M1, N1, M0, N0, M, N, oflag_unpack, cpu_data);
  double t4 = now_s();
  if (times) {
    times[0] = t1 - t0; times[1] = t2 - t1; times[2] = t3 - t2; times[3] = t4 - t3;
  }
  free(pl); free(pr); free(po);
  return 0;
}

// Raw passthroughs so tests can pin pack / mmt4d / unpack one at a time with any flags.
void uk_chain_pack(const void* in, int64_t in_stride0, void* out, int64_t out_stride0,
                   int64_t in_size0, int64_t in_size1, int64_t o0, int64_t o1, int64_t o2, int64_t o3,
                   uint64_t padding, uint32_t flags, int cpu_mode) {
  iree_uk_uint64_t cpu_data[8] = {0};
  cpu_data[0] = uk_chain_cpu_data0(cpu_mode);
  iree_uk_pack(in, 0, in_stride0, 1, out, 0, out_stride0, o2 * o3, in_size0, in_size1, o0, o1, o2, o3,
               padding, flags, cpu_data);
}
void uk_chain_unpack(const void* in, int64_t in_stride0, void* out, int64_t out_stride0, int64_t i0,
                     int64_t i1, int64_t i2, int64_t i3, int64_t out_size0, int64_t out_size1,
                     uint32_t flags, int cpu_mode) {
  iree_uk_uint64_t cpu_data[8] = {0};
  cpu_data[0] = uk_chain_cpu_data0(cpu_mode);
  iree_uk_unpack(in, 0, in_stride0, i2 * i3, out, 0, out_stride0, 1, i0, i1, i2, i3, out_size0,
                 out_size1, flags, cpu_data);
}
void uk_chain_mmt4d(const void* lhs, int64_t ls0, const void* rhs, int64_t rs0, void* out, int64_t os0,
                    int64_t M1, int64_t N1, int64_t K1, int M0, int N0, int K0, uint32_t flags,
                    int cpu_mode) {
  iree_uk_uint64_t cpu_data[8] = {0};
  cpu_data[0] = uk_chain_cpu_data0(cpu_mode);
  iree_uk_mmt4d(lhs, 0, ls0, rhs, 0, rs0, out, 0, os0, M1, N1, K1, M0, N0, K0, flags, cpu_data);
}
uint32_t uk_chain_mmt4d_info(int M0, int N0, int K0, uint32_t flags, int cpu_mode) {
  iree_uk_uint64_t cpu_data[8] = {0};
  cpu_data[0] = uk_chain_cpu_data0(cpu_mode);
  return iree_uk_mmt4d_info(M0, N0, K0, flags, cpu_data);
}
