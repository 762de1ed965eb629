// Internal glue between the translation units of libiree_b200.so. Not part of the public ABI.
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
// Records `message` as the calling thread's last error and returns `code`.
int32_t iree_b200_internal_set_error(int32_t code, const char* message);
// Encodes (on the host, 128 bytes into out_map) the tensor map through which the decode kernels fetch
// int4 weight tiles [N, K / 2] when K spans more than one 4096-wide slice. Returns a status code.
int32_t iree_b200_internal_encode_decode_weight_map(const void* wq, int32_t N, int32_t K, void* out_map);
#ifdef __cplusplus
}
#endif
