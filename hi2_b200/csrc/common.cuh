// Shared definitions of the sm_100a kernels behind the C-ABI declared in include/hi2_b200.h.
//
// Arithmetic convention: the whole library is compiled with -fmad=false, so `a * b + c` is two
// roundings exactly as written (the reference path rounds every product and sum separately).
// Where a fused multiply-add is wanted it is spelled fmaf()/fma().
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../include/hi2_b200.h"

namespace hi2 {

void set_error(const char* fmt, ...);
void note_launch();  // one more kernel launch enqueued by this library (process-wide counter)

inline int fail(int code, const char* what) {
  set_error("%s", what);
  return code;
}

inline int check_launch(const char* what) {
  note_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return HI2_ERR_LAUNCH;
  }
  return HI2_OK;
}

#define HI2_REQUIRE(cond, msg)                         \
  do {                                                 \
    if (!(cond)) return ::hi2::fail(HI2_ERR_ARG, msg); \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__host__ __device__ inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// torch.clamp(lo, hi) semantics: NaN stays NaN.
__device__ __forceinline__ float clamp_keep_nan(float v, float lo, float hi) {
  v = (v < lo) ? lo : v;
  v = (v > hi) ? hi : v;
  return v;
}

__device__ __forceinline__ float round_f16(float v) { return __half2float(__float2half_rn(v)); }

}  // namespace hi2
