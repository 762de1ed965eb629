// Thin inline-PTX wrappers for the sm_100a features the contraction kernels use:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (alloc / mma / commit / ld) and the
// device-side tensor-map edit instructions. Every wait is bounded: a wait that runs out
// reports through the kernel's status words instead of spinning forever.
#pragma once
#include <stdint.h>

namespace b200 {

// Status codes a kernel leaves in Workspace::status[0] (0 = ok).
enum : uint32_t {
  kStatusOk = 0,
  kStatusTimeoutFull = 1,       // MMA warp gave up waiting for a TMA stage
  kStatusTimeoutEmpty = 2,      // producer gave up waiting for a free stage
  kStatusTimeoutTmemFull = 3,   // epilogue gave up waiting for an accumulator
  kStatusTimeoutTmemEmpty = 4,  // MMA warp gave up waiting for a drained accumulator
  kStatusBadArgument = 5,       // shape / alignment precondition violated; nothing was computed
  kStatusTimeoutDequant = 6,    // MMA warp gave up waiting for a dequantised weight stage
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier -------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
// Required before the storage of a barrier is initialised again.
__device__ __forceinline__ void mbar_inval(uint32_t bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Two flavours of polling. With a suspend-time hint the hardware keeps the warp asleep until the
// phase completes (or the hint runs out): a waiting role then issues almost nothing, which is
// what the tensor-core kernels want (their producer / issuer / epilogue roles mostly wait, and
// the quieter they are the higher the clocks stay under the power cap; C2 4096^3: 106 -> 102 us).
// Without the hint the warp comes back at once when the phase flips; the decode kernel, whose 16
// warps all do arithmetic and wait only briefly, is faster that way (9.0 vs 9.4 us).
constexpr uint32_t kTryWaitSuspendHintNs = 20000;
template <bool SUSPEND>
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  if (SUSPEND) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kTryWaitSuspendHintNs)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
  }
  return ok != 0;
}
// Waits for the phase with the given parity to complete. Gives up after ~2 s of wall time or
// as soon as another role has raised the CTA-wide abort flag; returns false then.
constexpr uint64_t kDefaultWaitLimitNs = 2000000000ull;
template <bool SUSPEND = true>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint64_t limit_ns = kDefaultWaitLimitNs) {
  if (mbar_try_wait<SUSPEND>(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t polls = 0;
  while (true) {
    if (mbar_try_wait<SUSPEND>(bar, parity)) return true;
    // with the hint one poll already lasts microseconds: look at the clock every time
    if (SUSPEND || (++polls & 0xff) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > limit_ns) return false;
    }
  }
}

// ---- programmatic dependent launch ------------------------------------------------------
// Both are no-ops in a kernel that was launched without a programmatic dependency.
// launch_dependents: this block no longer holds back the launch of the next kernel on the stream
// (which happens once every block of this grid has said so or has exited).
// wait: returns once every kernel this one depends on has completed and its writes are visible;
// nothing that a preceding kernel may produce is read, and nothing it may read is written, before it.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- proxies / fences ---------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tensormap_fence_acquire(const void* gmem_map) {
  asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(gmem_map) : "memory");
}

// ---- TMA --------------------------------------------------------------------------------
// x is the innermost coordinate: x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const void* tmap, uint32_t bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst_smem), "l"(tmap), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tmap, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst_smem), "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// ---- tcgen05 ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives once on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; `accumulate` == 0 overwrites D.
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives lane (base_lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  // .sync.aligned: every lane must execute it together. Lanes that polled a barrier leave their
  // loops one by one and a vote does not bring them back into step; without this the instruction
  // has been seen to drop single lanes' data.
  __syncwarp();
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns, registers -> tensor memory: thread t of the warp writes
// lane (base_lane + t). A warp reaches only the 32 lanes of its own quarter (warp index % 4).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&v)[32]) {
  __syncwarp();  // see tmem_ld_32x32
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
      "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
      "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
      "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem]: the 128 x 16 A operand sits in tensor memory, row i in lane i,
// two 16-bit elements of K per 32-bit column (8 columns per instruction).
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] += A[smem] * B[smem] with the accumulate flag fixed at compile time (no predicate to compute).
__device__ __forceinline__ void mma_f16_ss_more(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc)
      : "memory");
}
__device__ __forceinline__ void mma_i8_ss_more(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc)
      : "memory");
}

// The same with the accumulate flag fixed at compile time (no predicate to compute per instruction):
// `first` overwrites D, `more` adds to it.
__device__ __forceinline__ void mma_f16_ts_first(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc)
      : "memory");
}
__device__ __forceinline__ void mma_f16_ts_more(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc)
      : "memory");
}

// ---- TMA stores (shared -> global), bulk async-groups -------------------------------------------
// x is the innermost coordinate: x * element size must be a multiple of 16 bytes. Elements outside
// the tensor's extents are not written.
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src_smem, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(tmap), "r"(src_smem), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void* tmap, uint32_t src_smem, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(tmap), "r"(src_smem), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_4d(const void* tmap, uint32_t src_smem, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(tmap), "r"(src_smem), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const void* tmap, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst_smem), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns once at most N of this thread's groups are still reading their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Returns once at most N groups are incomplete; a complete group's writes are visible to this thread.
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Barrier among `count` threads (a multiple of 32) of the CTA; id 0 is __syncthreads' barrier.
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
// System-scope flag accesses (other GPUs of the node read / write these words).
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ---- descriptors ------------------------------------------------------------------------
// Shared-memory matrix descriptor (tcgen05): start address, leading / stride byte offsets
// (all in 16-byte units), descriptor version 1, layout type in bits 61-63.
constexpr uint64_t kLayoutSwizzle128B = 2;
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3fff);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= 1ull << 46;  // descriptor version for sm_100
  d |= kLayoutSwizzle128B << 61;
  return d;
}

// Instruction descriptor for kind::f16 / kind::i8 (dense, no negate, no saturate).
//   c_format: 1 = f32, 2 = s32;  a/b format: f16 = 0, bf16 = 1 (kind::f16); s8 = 1 (kind::i8)
//   major: 0 = K-major, 1 = MN-major
__host__ __device__ constexpr uint32_t make_instr_desc(uint32_t c_format, uint32_t a_format, uint32_t b_format,
                                                       uint32_t a_major, uint32_t b_major, uint32_t m, uint32_t n) {
  return (c_format << 4) | (a_format << 7) | (b_format << 10) | (a_major << 15) | (b_major << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---- device-side tensor-map editing -----------------------------------------------------------
__device__ __forceinline__ void tensormap_replace_address(uint32_t smem_map, const void* gptr) {
  asm volatile("tensormap.replace.tile.global_address.shared::cta.b1024.b64 [%0], %1;" ::"r"(smem_map), "l"(gptr)
               : "memory");
}
#define B200_TENSORMAP_REPLACE_DIM(ORD)                                                                       \
  __device__ __forceinline__ void tensormap_replace_dim##ORD(uint32_t smem_map, uint32_t v) {               \
    asm volatile("tensormap.replace.tile.global_dim.shared::cta.b1024.b32 [%0], " #ORD ", %1;" ::"r"(smem_map), \
                 "r"(v)                                                                                       \
                 : "memory");                                                                                 \
  }
B200_TENSORMAP_REPLACE_DIM(0)
B200_TENSORMAP_REPLACE_DIM(1)
B200_TENSORMAP_REPLACE_DIM(2)
B200_TENSORMAP_REPLACE_DIM(3)
#undef B200_TENSORMAP_REPLACE_DIM
// Stride ordinal i is the byte stride of dimension i + 1 (dimension 0 is contiguous).
#define B200_TENSORMAP_REPLACE_STRIDE(ORD)                                                                       \
  __device__ __forceinline__ void tensormap_replace_stride##ORD(uint32_t smem_map, uint64_t bytes) {           \
    asm volatile("tensormap.replace.tile.global_stride.shared::cta.b1024.b64 [%0], " #ORD ", %1;" ::"r"(smem_map), \
                 "l"(bytes)                                                                                      \
                 : "memory");                                                                                    \
  }
B200_TENSORMAP_REPLACE_STRIDE(0)
B200_TENSORMAP_REPLACE_STRIDE(1)
B200_TENSORMAP_REPLACE_STRIDE(2)
#undef B200_TENSORMAP_REPLACE_STRIDE
#define B200_TENSORMAP_REPLACE_BOX(ORD)                                                                       \
  __device__ __forceinline__ void tensormap_replace_box##ORD(uint32_t smem_map, uint32_t v) {               \
    asm volatile("tensormap.replace.tile.box_dim.shared::cta.b1024.b32 [%0], " #ORD ", %1;" ::"r"(smem_map), \
                 "r"(v)                                                                                       \
                 : "memory");                                                                                 \
  }
B200_TENSORMAP_REPLACE_BOX(0)
B200_TENSORMAP_REPLACE_BOX(1)
B200_TENSORMAP_REPLACE_BOX(2)
B200_TENSORMAP_REPLACE_BOX(3)
#undef B200_TENSORMAP_REPLACE_BOX
// Copies the edited 128-byte map from shared to global memory and releases it to the
// tensor-map proxy. Must be executed by a full warp.
__device__ __forceinline__ void tensormap_publish(void* gmem_map, uint32_t smem_map) {
  asm volatile(
      "tensormap.cp_fenceproxy.global.shared::cta.tensormap::generic.release.gpu.sync.aligned [%0], [%1], 128;"
      ::"l"(gmem_map), "r"(smem_map)
      : "memory");
}

// ---- CTA pairs (cluster of two, tcgen05 cta_group::2) -------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion may be reported to a barrier in the other CTA of the pair.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst_smem, const void* tmap, uint32_t bar_cluster_addr, int x,
                                                 int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
      "%5}], [%2];" ::"r"(dst_smem),
      "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
// Arrives on `bar` (same offset) in both CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(both)
               : "memory");
}
__device__ __forceinline__ void mma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_i8_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

}  // namespace b200
