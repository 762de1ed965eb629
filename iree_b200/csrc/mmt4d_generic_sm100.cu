// iree_uk_mmt4d for the element types the tensor-core kernels do not take
// (runtime/src/iree/builtins/ukernel/exported_bits.h:29-42): f32f32f32, s16s16s32, s16u4s32, s16s8s32,
// s8s4s32, any tile shape. One thread per output element, the reduction in the order of the reference's
// generic tile functions (mmt4d_tile_generic.c: K1 outer, K0 inner; for the 4-bit right-hand sides two
// reduction elements per byte, low nibble first, K0 even). Integer types are exact; f32 differs from the
// reference only where its compiler contracts the multiply-add differently.
//
// Bindings: lhs, rhs, out. Constants: M1, N1, K1, M0, N0, K0, the pitch of the outermost dimension of lhs
// and of rhs in BYTES and of out in elements, the type (IREE_UK_FLAG_MMT4D_TYPE_* value), ACCUMULATE.
#include <stdint.h>

extern "C" __global__ void __launch_bounds__(256)
    b200_mmt4d_generic(const void* lhs, const void* rhs, void* out, int M1, int N1, int K1, int M0, int N0, int K0,
                       int lhs_pitch_bytes, int rhs_pitch_bytes, int out_pitch, int type, int accumulate) {
  const int64_t tile = static_cast<int64_t>(M0) * N0;
  const int64_t total = static_cast<int64_t>(M1) * N1 * tile;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int j0 = static_cast<int>(e % N0);
    const int i0 = static_cast<int>((e / N0) % M0);
    const int j = static_cast<int>((e / tile) % N1);
    const int i = static_cast<int>(e / (tile * N1));
    const int64_t o = static_cast<int64_t>(i) * out_pitch + static_cast<int64_t>(j) * tile + static_cast<int64_t>(i0) * N0 + j0;
    const uint8_t* lp = static_cast<const uint8_t*>(lhs) + static_cast<int64_t>(i) * lhs_pitch_bytes;
    const uint8_t* rp = static_cast<const uint8_t*>(rhs) + static_cast<int64_t>(j) * rhs_pitch_bytes;
    if (type == 0x01) {  // f32f32f32
      const float* l = reinterpret_cast<const float*>(lp);
      const float* r = reinterpret_cast<const float*>(rp);
      float acc = accumulate ? static_cast<float*>(out)[o] : 0.f;
      for (int k = 0; k < K1; ++k)
        for (int k0 = 0; k0 < K0; ++k0)
          acc += l[(static_cast<int64_t>(k) * M0 + i0) * K0 + k0] * r[(static_cast<int64_t>(k) * N0 + j0) * K0 + k0];
      static_cast<float*>(out)[o] = acc;
      continue;
    }
    int32_t acc = accumulate ? static_cast<int32_t*>(out)[o] : 0;
    if (type == 0x07 || type == 0x09) {  // s16s16s32, s16s8s32
      const int16_t* l = reinterpret_cast<const int16_t*>(lp);
      for (int k = 0; k < K1; ++k)
        for (int k0 = 0; k0 < K0; ++k0) {
          const int64_t ri = (static_cast<int64_t>(k) * N0 + j0) * K0 + k0;
          const int32_t b = type == 0x07 ? reinterpret_cast<const int16_t*>(rp)[ri] : reinterpret_cast<const int8_t*>(rp)[ri];
          acc += static_cast<int32_t>(l[(static_cast<int64_t>(k) * M0 + i0) * K0 + k0]) * b;
        }
    } else {  // s16u4s32 (0x08), s8s4s32 (0x0A): two reduction elements per right-hand-side byte
      const int half = K0 / 2;
      for (int k = 0; k < K1; ++k)
        for (int h = 0; h < half; ++h) {
          const int64_t li = (static_cast<int64_t>(k) * M0 + i0) * K0 + 2 * h;
          const uint8_t byte = rp[(static_cast<int64_t>(k) * N0 + j0) * half + h];
          int32_t a0, a1, b0, b1;
          if (type == 0x08) {
            a0 = reinterpret_cast<const int16_t*>(lp)[li];
            a1 = reinterpret_cast<const int16_t*>(lp)[li + 1];
            b0 = byte & 0xf;
            b1 = byte >> 4;
          } else {
            a0 = reinterpret_cast<const int8_t*>(lp)[li];
            a1 = reinterpret_cast<const int8_t*>(lp)[li + 1];
            b0 = static_cast<int32_t>(static_cast<uint32_t>(byte) << 28) >> 28;  // sign-extended low nibble
            b1 = static_cast<int32_t>(static_cast<uint32_t>(byte) << 24) >> 28;  // sign-extended high nibble
          }
          acc += a0 * b0 + a1 * b1;
        }
    }
    static_cast<int32_t*>(out)[o] = acc;
  }
}
