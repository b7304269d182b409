// Host-side helpers shared by the entry points: tensor-map encoding through
// the driver entry point (the library does not link libcuda), the per-device
// status word, launch counting and argument checks.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/b200k.h"

namespace b200k {

// 16-bit element tensor map.  dims/strides innermost first; strides_bytes[i] is
// the byte stride of dimension i+1 (dimension 0 is contiguous).
// swizzle: 0 = none, 1 = 128-byte, 2 = 64-byte.  Returns B200K_OK / B200K_ETMAP / B200K_ECUDA.
int encode_tmap_16bit(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, int swizzle);

// Device pointer to the int[4] status word of the current device.
int* status_ptr();

void count_launch(int n = 1);

// Last CUDA error -> B200K_ECUDA (and clears it), else B200K_OK.
int check_launch();

// properties of the current device, cached per device
struct DevInfo {
  int sm_count;
  int cc_major;
  int max_smem_optin;
};
const DevInfo& dev_info();

// Skinny GEMM (M <= 128): split-K inside thread-block clusters (gemm_skinny_sm100.cu).
// epilogue: 0 none, B200K_EPI_ADD (R, ldr: the residual), B200K_EPI_SWIGLU (C is N/2 wide).
int launch_skinny(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                  bool bf16, cudaStream_t stream, int epilogue = 0, const void* R = nullptr, int64_t ldr = 0);

// Tuning overrides for experiments and tests (B200K_OPT_* in b200k.h).  Each starts from its
// environment variable, read ONCE when the first launcher asks, and can be changed afterwards with
// b200k_set_option; 0 = the library's own choice.  A launch reads an atomic, never the environment.
int tuning_option(int which);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace b200k
