// The reference's own software f16 / bf16 <-> f32 conversions, exported one to one so that the
// restatement's conversions (oracle/contraction_oracle.c, which uses the compiler's _Float16)
// can be compared with them over every 16-bit pattern.
// TEST INFRASTRUCTURE ONLY. The routines are `static inline` in the reference header
// runtime/src/iree/builtins/ukernel/common.h:664-790; this file only includes that header where
// it lies and wraps the four functions. Built into oracle/_ref/ (never committed).
#include <stdint.h>

#include "iree/builtins/ukernel/common.h"

float uk_conv_f16_to_f32(uint16_t v) { return iree_uk_f16_to_f32(v); }
uint16_t uk_conv_f32_to_f16(float v) { return iree_uk_f32_to_f16(v); }
float uk_conv_bf16_to_f32(uint16_t v) { return iree_uk_bf16_to_f32(v); }
uint16_t uk_conv_f32_to_bf16(float v) { return iree_uk_f32_to_bf16(v); }

// Array forms (one call per test instead of 65536 ctypes calls).
void uk_conv_f16_to_f32_n(const uint16_t* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = iree_uk_f16_to_f32(in[i]);
}
void uk_conv_f32_to_f16_n(const float* in, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = iree_uk_f32_to_f16(in[i]);
}
void uk_conv_bf16_to_f32_n(const uint16_t* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = iree_uk_bf16_to_f32(in[i]);
}
void uk_conv_f32_to_bf16_n(const float* in, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = iree_uk_f32_to_bf16(in[i]);
}
