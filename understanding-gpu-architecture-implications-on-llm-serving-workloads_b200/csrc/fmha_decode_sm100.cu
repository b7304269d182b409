// placeholder translation unit, replaced by the split-KV decode kernels
#include "host_common.h"
extern "C" int b200k_fmha_decode_splitkv(const void*, const void*, const void*, void*, int, int, int, int, int, int,
                                         const int64_t*, const int64_t*, const int64_t*, const int64_t*, float,
                                         const int32_t*, int, int, void*, size_t, b200k_stream_t) {
  return B200K_EARG;
}
extern "C" size_t b200k_fmha_decode_workspace_bytes(int, int, int, int, int, int, int) { return 0; }
extern "C" int b200k_fmha_decode_auto_splits(int, int, int) { return 1; }
