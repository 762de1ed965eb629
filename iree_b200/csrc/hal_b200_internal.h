// Internal glue between the translation units of libiree_b200.so. Not part of the public ABI.
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
// Records `message` as the calling thread's last error and returns `code`.
int32_t iree_b200_internal_set_error(int32_t code, const char* message);
#ifdef __cplusplus
}
#endif
