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

// A long chain of short kernels queued as ONE graph launch.  Between construction and finish()
// everything the calling thread launches on `stream` is captured instead of run; finish()
// instantiates the captured graph and launches it on the stream.  Why: a stream's launch queue
// holds about a thousand entries, so a chain of 1700 small kernels (the inverse factor of one
// input) throttles the host to the GPU's pace until it has drained, and the host cannot feed the
// other streams meanwhile - the chains of four inputs then run one after the other instead of
// side by side; as a graph the chain costs the host one launch and its kernels start back to back.
// A stream that is already being captured by the caller is left alone (the launches then join the
// caller's graph).  Finished graphs are destroyed on later calls, once their completion event has
// passed.
class ChainGraph {
 public:
  explicit ChainGraph(cudaStream_t stream);
  // rc: the status of the launches issued since construction.  Returns rc if it is an error (the
  // captured work is dropped), else the status of instantiating and launching the graph.
  int finish(int rc, const char* what);
  ~ChainGraph();

 private:
  cudaStream_t stream_;
  bool capturing_ = false;
};

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

// Division by a value that stays fixed over many quotients.  r is the correctly rounded
// reciprocal; `fast` is false when b is outside a comfortable normal range or its significand is
// all ones (the one case Markstein's correction step does not cover): then the IEEE division
// is used, so both helpers below return exactly what __fdiv_rn would give.
struct Recip {
  float r;
  bool fast;
};
__device__ __forceinline__ Recip make_recip(float b) {
  const float ab = fabsf(b);
  Recip rc;
  rc.fast = ab > 1e-18f && ab < 1e18f && (__float_as_uint(b) & 0x7fffffu) != 0x7fffffu;
  rc.r = __frcp_rn(b);
  return rc;
}

// rintf(__fdiv_rn(a, b)) for results that the caller clamps to [0, 255].  a * r is within 2 ulp
// of the quotient, so the two can round to different integers only when a * r lies within a
// few ulp of a half-integer; those cases (about one in 10^4) take the IEEE division.  Beyond
// 1024 a difference of one survives no clamp to a ladder of at most 256 levels.
__device__ __forceinline__ float rint_div(float a, float b, Recip rc) {
  if (!rc.fast) return rintf(__fdiv_rn(a, b));
  const float t = a * rc.r;
  float q = rintf(t);
  if (fabsf(fabsf(t - q) - 0.5f) < 2.5e-4f && fabsf(t) < 1024.0f) q = rintf(__fdiv_rn(a, b));
  return q;
}

// __fdiv_rn(a, b): q0 = a * r is a faithful quotient, one fused correction step makes it the
// correctly rounded one (Markstein).  a is assumed finite and not denormal-small.
__device__ __forceinline__ float div_by(float a, float b, Recip rc) {
  if (!rc.fast) return __fdiv_rn(a, b);
  const float q0 = a * rc.r;
  return fmaf(fmaf(-q0, b, a), rc.r, q0);
}

}  // namespace hi2
