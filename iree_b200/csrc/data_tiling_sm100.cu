// Data-tiling kernels for sm_100a: row-major 2-D <-> 4-D tiled layouts.
//
// These are the GPU counterparts of the reference's pack / unpack micro kernels
// (runtime/src/iree/builtins/ukernel/pack.h:14-34, unpack.h:14-25, semantics in pack.c:52-100 and
// unpack.c:32-80): `pack` copies a row-major matrix [size0, size1] into a tiled array
// [o0, o1, o2, o3], padding the ragged edge with a fill value; `unpack` is the inverse and drops
// the padding. TRANSPOSE_OUTER swaps which matrix dimension the two outer indices walk,
// TRANSPOSE_INNER does the same for the two tile indices (exported_bits.h:64-66, 82-83); the flag
// values are the reference's.
//
// Both directions are pure data movement, so the bound is HBM. A CTA owns a region of the matrix
// made of whole tiles (at most 64 rows by 256..512 bytes of columns), stages it in shared memory
// and touches global memory only in runs that are contiguous on that side: rows on the row-major
// side, whole tiles (consecutive along o1) on the tiled side. Tiles too large for the staging
// buffer take a direct path, one thread per element.
//
// Kernel ABI (as every export of this cubin): bindings first, then i32 constants.
//   b200_pack_b{8,16,32}:   (in, out; in_size0, in_size1, in_stride0, in_stride1, out_size0, out_size1,
//                            out_size2, out_size3, out_stride0, flags, padding, in_offset, out_offset)
//   b200_unpack_b{8,16,32}: (in, out; in_size0, in_size1, in_size2, in_size3, in_stride0, out_size0,
//                            out_size1, out_stride0, out_stride1, flags, in_offset, out_offset)
// Sizes, strides and offsets are in elements. One region per CTA: grid.x = region count (the
// host computes it with tiling_regions() below, restated in the host library and the planner).
#include <cstdint>

namespace b200_tiling {

constexpr uint32_t kFlagTransposeInner = 0x100;   // IREE_UK_FLAG_PACK_TRANSPOSE_INNER
constexpr uint32_t kFlagTransposeOuter = 0x200;   // IREE_UK_FLAG_PACK_TRANSPOSE_OUTER
constexpr uint32_t kFlagAccumulateI32 = 0x10000;  // pack only, 32-bit elements: out += in (integer add)
constexpr uint32_t kFlagAccumulateF32 = 0x20000;  // pack only, 32-bit elements: out += in (float add)
constexpr int kThreads = 256;
constexpr int kMaxRegionRows = 64;
constexpr int kRegionRowBytes = 256;
constexpr int kStageBytes = kMaxRegionRows * (2 * kRegionRowBytes + 16);

// Geometry shared by both directions. "rows/cols" are matrix coordinates.
struct Geometry {
  uint32_t tile0, tile1;      // tile extent along matrix rows / cols
  uint32_t outer0, outer1;    // number of tiles along matrix rows / cols
  uint32_t nr, nc;            // tiles per region along rows / cols
  uint32_t regions0, regions1;
  bool staged;                // false: tiles do not fit the staging buffer
};

__host__ __device__ inline Geometry make_geometry(uint32_t o0, uint32_t o1, uint32_t o2, uint32_t o3, uint32_t flags,
                                                  uint32_t elem_bytes) {
  Geometry g;
  const bool ti = flags & kFlagTransposeInner, to = flags & kFlagTransposeOuter;
  g.tile0 = ti ? o3 : o2;
  g.tile1 = ti ? o2 : o3;
  g.outer0 = to ? o1 : o0;
  g.outer1 = to ? o0 : o1;
  g.staged = g.tile0 > 0 && g.tile1 > 0 && g.tile0 <= (uint32_t)kMaxRegionRows &&
             g.tile1 * elem_bytes <= 2u * kRegionRowBytes;
  if (g.staged) {
    g.nr = kMaxRegionRows / g.tile0;
    g.nc = (kRegionRowBytes / elem_bytes) / g.tile1;
    if (g.nc == 0) g.nc = 1;
  } else {
    g.nr = g.nc = 1;
  }
  g.regions0 = (g.outer0 + g.nr - 1) / g.nr;
  g.regions1 = (g.outer1 + g.nc - 1) / g.nc;
  return g;
}

// n / d for n < 2^16 and 1 <= d <= 2^16 with one multiply: m = floor((2^32 - 1) / d) + 1 makes
// umulhi(n, m) exact whenever n * d < 2^32.
struct FastDiv {
  uint32_t m, d;
  __device__ explicit FastDiv(uint32_t divisor) : m(divisor > 1 ? 0xFFFFFFFFu / divisor + 1u : 0u), d(divisor) {}
  __device__ __forceinline__ uint32_t div(uint32_t n) const { return d > 1 ? __umulhi(n, m) : n; }
};

template <typename T>
__device__ __forceinline__ void combine(T* dst, T v, uint32_t flags) {
  *dst = v;
}
template <>
__device__ __forceinline__ void combine<uint32_t>(uint32_t* dst, uint32_t v, uint32_t flags) {
  if (flags & kFlagAccumulateI32) {
    *dst = *dst + v;  // two's complement: the same bits as a signed add
  } else if (flags & kFlagAccumulateF32) {
    *dst = __float_as_uint(__uint_as_float(*dst) + __uint_as_float(v));
  } else {
    *dst = v;
  }
}

// rm: the row-major matrix [S0, S1] with element strides (rs0, rs1).
// tl: the tiled array [o0, o1, o2, o3] with element stride ts0 on the outermost dimension.
template <typename T, bool PACK>
__device__ __forceinline__ void tiling_body(T* __restrict__ rm, T* __restrict__ tl, uint32_t S0, uint32_t S1,
                                            int64_t rs0, int64_t rs1, uint32_t o0, uint32_t o1, uint32_t o2,
                                            uint32_t o3, int64_t ts0, uint32_t flags, T padding) {
  extern __shared__ __align__(16) uint8_t stage_raw[];
  T* stage = reinterpret_cast<T*>(stage_raw);
  const Geometry g = make_geometry(o0, o1, o2, o3, flags, sizeof(T));
  const bool ti = flags & kFlagTransposeInner, to = flags & kFlagTransposeOuter;
  const uint32_t tile_elems = o2 * o3;
  if (tile_elems == 0 || o0 == 0 || o1 == 0) return;

  if (!g.staged) {
    // Direct path: one thread per tiled element, grid-stride.
    const uint64_t total = (uint64_t)o0 * o1 * tile_elems;
    for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (uint64_t)gridDim.x * blockDim.x) {
      const uint32_t t = (uint32_t)(e % tile_elems);
      const uint64_t ab = e / tile_elems;
      const uint32_t b = (uint32_t)(ab % o1), a = (uint32_t)(ab / o1);
      const uint32_t c = t / o3, d = t % o3;
      const uint64_t row = (uint64_t)(to ? b : a) * g.tile0 + (ti ? d : c);
      const uint64_t col = (uint64_t)(to ? a : b) * g.tile1 + (ti ? c : d);
      T* tp = tl + (int64_t)a * ts0 + (int64_t)b * tile_elems + t;
      const bool inside = row < S0 && col < S1;
      if (PACK) {
        combine<T>(tp, inside ? rm[(int64_t)row * rs0 + (int64_t)col * rs1] : padding, flags);
      } else if (inside) {
        rm[(int64_t)row * rs0 + (int64_t)col * rs1] = *tp;
      }
    }
    return;
  }

  const uint32_t region = blockIdx.x;
  if (region >= g.regions0 * g.regions1) return;
  // Regions advance fastest along the direction in which the tiled side is contiguous.
  uint32_t reg0, reg1;
  if (to) {
    reg0 = region % g.regions0;
    reg1 = region / g.regions0;
  } else {
    reg1 = region % g.regions1;
    reg0 = region / g.regions1;
  }
  const uint32_t out0_first = reg0 * g.nr, out1_first = reg1 * g.nc;
  const uint32_t nr = min(g.nr, g.outer0 - out0_first), nc = min(g.nc, g.outer1 - out1_first);
  const uint32_t R = nr * g.tile0, Ccols = nc * g.tile1;
  // Row pitch of the staging buffer: whole 16-byte vectors plus one, so that rows start in different banks.
  const uint32_t pitch = (((g.nc * g.tile1 * (uint32_t)sizeof(T) + 15u) & ~15u) + 16u) / (uint32_t)sizeof(T);
  const uint64_t row_first = (uint64_t)out0_first * g.tile0, col_first = (uint64_t)out1_first * g.tile1;
  const uint32_t count = R * Ccols;  // at most 64 x 512: every index below fits 16 bits, which FastDiv needs

  // Both sides move 16-byte vectors when their layout allows it, else 4-byte words, else elements.
  constexpr uint32_t E16 = 16 / sizeof(T), E4 = 4 / sizeof(T);
  union Vec {
    uint4 q;
    uint32_t w[4];
    T e[E16];
  };
  auto width_for = [&](const void* base, int64_t stride, uint64_t first, uint32_t extent) -> uint32_t {
    const uintptr_t p = reinterpret_cast<uintptr_t>(base);
    if ((p & 15) == 0 && stride % E16 == 0 && first % E16 == 0 && extent % E16 == 0) return E16;
    if (E4 > 1 && (p & 3) == 0 && stride % E4 == 0 && first % E4 == 0 && extent % E4 == 0) return E4;
    return 1;
  };
  // elements per unit on the row-major side (rows must be contiguous) and on the tiled side
  const uint32_t rm_step = rs1 == 1 ? width_for(rm, rs0, col_first, Ccols) : 1u;
  const uint32_t tl_step = width_for(tl, ts0, 0, tile_elems);
  // a unit of the tiled side is one vector of a staged row when tile rows are long enough and not transposed
  const bool tl_contiguous = !ti && (o3 % tl_step) == 0;

  const uint32_t rm_per_row = Ccols / rm_step, rm_units = R * rm_per_row, tl_units = count / tl_step;
  const FastDiv div_cols(rm_per_row), div_tile(tile_elems), div_o3(o3), div_span(to ? nr : nc);

  // Global loads are issued kBatch at a time before their values are stored, so that each
  // thread keeps several requests in flight.
  constexpr int kBatch = 4;

  struct RmUnit {
    T* staged;
    T* global;
    uint32_t valid;  // elements of the unit inside the matrix (0..step)
  };
  auto rm_unit = [&](uint32_t i) -> RmUnit {
    const uint32_t r = div_cols.div(i), c = (i - r * rm_per_row) * rm_step;
    const uint64_t row = row_first + r, col = col_first + c;
    RmUnit u;
    u.staged = stage + r * pitch + c;
    u.global = rm + (int64_t)row * rs0 + (int64_t)col * rs1;
    u.valid = row < S0 ? (col + rm_step <= S1 ? rm_step : (col < S1 ? (uint32_t)(S1 - col) : 0u)) : 0u;
    return u;
  };
  // Tiled side: unit u covers `tl_step` consecutive elements of one tile; tiles follow each
  // other along the outer direction that is contiguous in memory.
  struct TlUnit {
    T* global;
    uint32_t base_r, base_c, c, d;
  };
  auto tl_unit = [&](uint32_t u) -> TlUnit {
    const uint32_t e = u * tl_step;
    const uint32_t tile = div_tile.div(e), t = e - tile * tile_elems;
    const uint32_t hi = div_span.div(tile), lo = tile - hi * (to ? nr : nc);
    const uint32_t l0 = to ? lo : hi, l1 = to ? hi : lo;
    const uint32_t a = to ? out1_first + l1 : out0_first + l0;
    const uint32_t b = to ? out0_first + l0 : out1_first + l1;
    TlUnit x;
    x.c = div_o3.div(t);
    x.d = t - x.c * o3;
    x.base_r = l0 * g.tile0;
    x.base_c = l1 * g.tile1;
    x.global = tl + (int64_t)a * ts0 + (int64_t)b * tile_elems + t;
    return x;
  };
  // Staged position of tile element (c, d) of the tile whose staged origin is (base_r, base_c).
  auto staged_at = [&](uint32_t base_r, uint32_t base_c, uint32_t c, uint32_t d) -> T* {
    return stage + (base_r + (ti ? d : c)) * pitch + base_c + (ti ? c : d);
  };
  auto load_vec = [&](const T* p, uint32_t step) -> Vec {
    Vec v;
    if (step == E16) v.q = *reinterpret_cast<const uint4*>(p);
    else if (E4 > 1 && step == E4) v.w[0] = *reinterpret_cast<const uint32_t*>(p);
    else v.e[0] = *p;
    return v;
  };
  auto store_vec = [&](T* p, const Vec& v, uint32_t step) {
    if (step == E16) *reinterpret_cast<uint4*>(p) = v.q;
    else if (E4 > 1 && step == E4) *reinterpret_cast<uint32_t*>(p) = v.w[0];
    else *p = v.e[0];
  };
  // Bytes, transposed tiles two elements deep (the VNNI-style right-hand side, e.g. 16 x 2): a
  // 16-byte unit is eight columns of two consecutive staged rows, interleaved. The unit starts at
  // d = 0 and at a multiple of eight columns, so both rows are read as one aligned 8-byte word.
  const bool interleave2 = sizeof(T) == 1 && ti && o3 == 2 && tl_step == 16 && (g.tile1 % 8) == 0;
  // Tiles whose rows are 2, 4 or 8 bytes long (K0 = 2 for bytes, ...), not transposed: a 16-byte
  // unit is 8, 4 or 2 whole tile rows, each an aligned word of its own staged row.
  const uint32_t run_bytes = (!ti && tl_step == E16 && (o3 * sizeof(T) == 2 || o3 * sizeof(T) == 4 || o3 * sizeof(T) == 8))
                                 ? o3 * (uint32_t)sizeof(T) : 0u;
  auto staged_read = [&](const TlUnit& x) -> Vec {
    if (tl_contiguous) return load_vec(staged_at(x.base_r, x.base_c, x.c, x.d), tl_step);
    if (run_bytes) {
      Vec v;
      if (run_bytes == 2) {
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j)
          reinterpret_cast<uint16_t*>(&v)[j] = *reinterpret_cast<const uint16_t*>(staged_at(x.base_r, x.base_c, x.c + j, 0));
      } else if (run_bytes == 4) {
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) v.w[j] = *reinterpret_cast<const uint32_t*>(staged_at(x.base_r, x.base_c, x.c + j, 0));
      } else {
#pragma unroll
        for (uint32_t j = 0; j < 2; ++j)
          reinterpret_cast<uint2*>(&v)[j] = *reinterpret_cast<const uint2*>(staged_at(x.base_r, x.base_c, x.c + j, 0));
      }
      return v;
    }
    if (interleave2) {
      const uint2 a = *reinterpret_cast<const uint2*>(staged_at(x.base_r, x.base_c, x.c, 0));
      const uint2 b = *reinterpret_cast<const uint2*>(staged_at(x.base_r, x.base_c, x.c, 1));
      Vec v;
      v.w[0] = __byte_perm(a.x, b.x, 0x5140);
      v.w[1] = __byte_perm(a.x, b.x, 0x7362);
      v.w[2] = __byte_perm(a.y, b.y, 0x5140);
      v.w[3] = __byte_perm(a.y, b.y, 0x7362);
      return v;
    }
    Vec v;
    uint32_t c = x.c, d = x.d;
#pragma unroll
    for (uint32_t j = 0; j < E16; ++j) {
      if (j < tl_step) {
        v.e[j] = *staged_at(x.base_r, x.base_c, c, d);
        if (++d == o3) { d = 0; ++c; }
      }
    }
    return v;
  };
  auto staged_write = [&](const TlUnit& x, const Vec& v) {
    if (tl_contiguous) {
      store_vec(staged_at(x.base_r, x.base_c, x.c, x.d), v, tl_step);
      return;
    }
    uint32_t c = x.c, d = x.d;
#pragma unroll
    for (uint32_t j = 0; j < E16; ++j) {
      if (j < tl_step) {
        *staged_at(x.base_r, x.base_c, c, d) = v.e[j];
        if (++d == o3) { d = 0; ++c; }
      }
    }
  };

  if (PACK) {
    for (uint32_t first = threadIdx.x; first < rm_units; first += kBatch * blockDim.x) {
      RmUnit u[kBatch];
      Vec v[kBatch];
      bool live[kBatch];
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        const uint32_t i = first + k * blockDim.x;
        live[k] = i < rm_units;
        if (!live[k]) continue;
        u[k] = rm_unit(i);
        if (u[k].valid == rm_step) {
          v[k] = load_vec(u[k].global, rm_step);
        } else {
#pragma unroll
          for (uint32_t j = 0; j < E16; ++j)
            if (j < rm_step) v[k].e[j] = j < u[k].valid ? u[k].global[j] : padding;  // rm_step > 1 implies unit stride
        }
      }
#pragma unroll
      for (int k = 0; k < kBatch; ++k)
        if (live[k]) store_vec(u[k].staged, v[k], rm_step);
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < tl_units; i += blockDim.x) {
      const TlUnit x = tl_unit(i);
      const Vec v = staged_read(x);
      if (tl_step == 1) combine<T>(x.global, v.e[0], flags);
      else if (sizeof(T) == 4 && (flags & (kFlagAccumulateI32 | kFlagAccumulateF32))) {
#pragma unroll
        for (uint32_t j = 0; j < E16; ++j) combine<T>(x.global + j, v.e[j], flags);
      } else store_vec(x.global, v, tl_step);
    }
  } else {
    for (uint32_t first = threadIdx.x; first < tl_units; first += kBatch * blockDim.x) {
      TlUnit x[kBatch];
      Vec v[kBatch];
      bool live[kBatch];
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        const uint32_t i = first + k * blockDim.x;
        live[k] = i < tl_units;
        if (!live[k]) continue;
        x[k] = tl_unit(i);
        v[k] = load_vec(x[k].global, tl_step);
      }
#pragma unroll
      for (int k = 0; k < kBatch; ++k)
        if (live[k]) staged_write(x[k], v[k]);
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < rm_units; i += blockDim.x) {
      const RmUnit u = rm_unit(i);
      if (u.valid == rm_step) {
        store_vec(u.global, load_vec(u.staged, rm_step), rm_step);
      } else {
        for (uint32_t j = 0; j < u.valid; ++j) u.global[j] = u.staged[j];  // rm_step > 1 implies unit stride
      }
    }
  }
}

}  // namespace b200_tiling

#define B200_PACK_EXPORT(NAME, T)                                                                                   \
  extern "C" __global__ void __launch_bounds__(b200_tiling::kThreads)                                               \
      NAME(const T* in, T* out, int32_t in_size0, int32_t in_size1, int32_t in_stride0, int32_t in_stride1,         \
           int32_t out_size0, int32_t out_size1, int32_t out_size2, int32_t out_size3, int32_t out_stride0,         \
           int32_t flags, int32_t padding, int32_t in_offset, int32_t out_offset) {                                 \
    b200_tiling::tiling_body<T, true>(const_cast<T*>(in) + in_offset, out + out_offset, in_size0, in_size1,         \
                                      in_stride0, in_stride1, out_size0, out_size1, out_size2, out_size3,           \
                                      out_stride0, (uint32_t)flags, (T)(uint32_t)padding);                          \
  }
#define B200_UNPACK_EXPORT(NAME, T)                                                                                 \
  extern "C" __global__ void __launch_bounds__(b200_tiling::kThreads)                                               \
      NAME(const T* in, T* out, int32_t in_size0, int32_t in_size1, int32_t in_size2, int32_t in_size3,             \
           int32_t in_stride0, int32_t out_size0, int32_t out_size1, int32_t out_stride0, int32_t out_stride1,      \
           int32_t flags, int32_t in_offset, int32_t out_offset) {                                                  \
    b200_tiling::tiling_body<T, false>(out + out_offset, const_cast<T*>(in) + in_offset, out_size0, out_size1,      \
                                       out_stride0, out_stride1, in_size0, in_size1, in_size2, in_size3,            \
                                       in_stride0, (uint32_t)flags, (T)0);                                          \
  }

B200_PACK_EXPORT(b200_pack_b8, uint8_t)
B200_PACK_EXPORT(b200_pack_b16, uint16_t)
B200_PACK_EXPORT(b200_pack_b32, uint32_t)
B200_UNPACK_EXPORT(b200_unpack_b8, uint8_t)
B200_UNPACK_EXPORT(b200_unpack_b16, uint16_t)
B200_UNPACK_EXPORT(b200_unpack_b32, uint32_t)
