// Order-16 Hadamard rotation of flagged column groups, fused with the load-side cast and the
// smoothing multiply (hi2/format.py:30-41, hi2/calibrate.py:243-251).
//
// Layout: the [rows, k] matrix is one flat array of 16-element groups.  A lane owns four
// consecutive elements (one 128-bit access for fp32), so four adjacent lanes own one group and a
// warp moves 512 contiguous bytes per access.  The twelve values a lane lacks arrive by warp
// shuffle.  Every output is the left-to-right sum over k = 0..15 of x_k * (+-1/4): the products
// are exact, so the result equals a row-times-matrix product accumulated in ascending k, which
// is what the reference's CPU product gives bit for bit (a radix-2 butterfly does not).
#include <type_traits>

#include "common.cuh"

namespace hi2 {
namespace {

template <typename T>
struct Quad;  // four consecutive elements of type T as the compute type C

template <>
struct Quad<float> {
  using C = float;
  static __device__ __forceinline__ void load(const float* p, C v[4]) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
  }
  static __device__ __forceinline__ void store(float* p, const C v[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Quad<double> {
  using C = double;
  static __device__ __forceinline__ void load(const double* p, C v[4]) {
    double2 a = *reinterpret_cast<const double2*>(p), b = *reinterpret_cast<const double2*>(p + 2);
    v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
  }
  static __device__ __forceinline__ void store(double* p, const C v[4]) {
    *reinterpret_cast<double2*>(p) = make_double2(v[0], v[1]);
    *reinterpret_cast<double2*>(p + 2) = make_double2(v[2], v[3]);
  }
};
template <>
struct Quad<__half> {
  using C = double;
  static __device__ __forceinline__ void load(const __half* p, C v[4]) {
    uint2 raw = *reinterpret_cast<const uint2*>(p);
    __half2 a = *reinterpret_cast<__half2*>(&raw.x), b = *reinterpret_cast<__half2*>(&raw.y);
    v[0] = (double)__low2float(a), v[1] = (double)__high2float(a);
    v[2] = (double)__low2float(b), v[3] = (double)__high2float(b);
  }
  static __device__ __forceinline__ void store(__half* p, const C v[4]) {
    __half h[4] = {__double2half(v[0]), __double2half(v[1]), __double2half(v[2]),
                   __double2half(v[3])};
    *reinterpret_cast<uint2*>(p) = *reinterpret_cast<uint2*>(h);
  }
};
template <>
struct Quad<__nv_bfloat16> {
  using C = double;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, C v[4]) {
    uint2 raw = *reinterpret_cast<const uint2*>(p);
    // a bf16 is the upper half of an fp32
    v[0] = (double)__uint_as_float(raw.x << 16), v[1] = (double)__uint_as_float(raw.x & 0xffff0000u);
    v[2] = (double)__uint_as_float(raw.y << 16), v[3] = (double)__uint_as_float(raw.y & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const C v[4]) {
    __nv_bfloat16 h[4] = {__double2bfloat16(v[0]), __double2bfloat16(v[1]), __double2bfloat16(v[2]),
                          __double2bfloat16(v[3])};
    *reinterpret_cast<uint2*>(p) = *reinterpret_cast<uint2*>(h);
  }
};

// fp32 view of four half-precision elements (exact), for the F16/BF16 -> F32 fused path.
template <typename T>
__device__ __forceinline__ void load_as_f32(const T* p, float v[4]);
template <>
__device__ __forceinline__ void load_as_f32<float>(const float* p, float v[4]) {
  Quad<float>::load(p, v);
}
template <>
__device__ __forceinline__ void load_as_f32<__half>(const __half* p, float v[4]) {
  uint2 raw = *reinterpret_cast<const uint2*>(p);
  __half2 a = *reinterpret_cast<__half2*>(&raw.x), b = *reinterpret_cast<__half2*>(&raw.y);
  v[0] = __low2float(a), v[1] = __high2float(a), v[2] = __low2float(b), v[3] = __high2float(b);
}
template <>
__device__ __forceinline__ void load_as_f32<__nv_bfloat16>(const __nv_bfloat16* p, float v[4]) {
  uint2 raw = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(raw.x << 16), v[1] = __uint_as_float(raw.x & 0xffff0000u);
  v[2] = __uint_as_float(raw.y << 16), v[3] = __uint_as_float(raw.y & 0xffff0000u);
}

__device__ __forceinline__ float fma_c(float a, float b, float c) { return fmaf(a, b, c); }
__device__ __forceinline__ double fma_c(double a, double b, double c) { return fma(a, b, c); }
__device__ __forceinline__ float shfl_c(float v, int src) { return __shfl_sync(0xffffffffu, v, src); }
__device__ __forceinline__ double shfl_c(double v, int src) {
  return __shfl_sync(0xffffffffu, v, src);
}

// The four outputs j = 4*sub + jj of one group, given the lane's own quad `mine`.
// Entry (k, j) of the matrix is (1/4) * (-1)^popcount(k & j); with k = 4*kh + kl the sign
// splits into a compile-time part popcount(kl & jj) and a per-lane part popcount(kh & sub),
// which is applied to the incoming quad by an exact negation.
template <typename C>
__device__ __forceinline__ void rotate_quad(const C mine[4], int lane, C out[4]) {
  const int sub = lane & 3, base = lane & ~3;
  C acc[4] = {C(0), C(0), C(0), C(0)};
#pragma unroll
  for (int kh = 0; kh < 4; ++kh) {
    const bool neg = __popc(kh & sub) & 1;
    C in[4];
#pragma unroll
    for (int kl = 0; kl < 4; ++kl) {
      C v = shfl_c(mine[kl], base + kh);
      in[kl] = neg ? -v : v;
    }
#pragma unroll
    for (int kl = 0; kl < 4; ++kl) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const C h = (__popc(kl & jj) & 1) ? C(-0.25) : C(0.25);
        acc[jj] = fma_c(in[kl], h, acc[jj]);
      }
    }
  }
#pragma unroll
  for (int jj = 0; jj < 4; ++jj) out[jj] = acc[jj];
}

// Tin == Tout (C = compute type of the pair) or Tin half/bf16 with Tout float.
// A lane takes UN quads per trip and issues all their loads before the first shuffle, so that
// enough bytes are in flight per SM to cover the latency of HBM (one 8- or 16-byte load per lane
// at a time left the kernel at about half of the copy bandwidth).
constexpr int ROT_UN = 4;

template <typename Tin, typename Tout, bool kSameType>
__global__ void __launch_bounds__(256)
rotate_kernel(const Tin* __restrict__ x, Tout* __restrict__ y, const uint8_t* __restrict__ flags,
              const float* __restrict__ col_scale, int64_t quads, int groups_per_row) {
  using C = typename std::conditional<kSameType, typename Quad<Tin>::C, float>::type;
  const int lane = threadIdx.x & 31;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // every lane of a warp runs the same number of iterations: quads is rounded up to a warp
  const int64_t limit = (quads + 31) & ~(int64_t)31;
  for (int64_t q0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q0 < limit; q0 += stride * ROT_UN) {
    C mine[ROT_UN][4];
    int64_t qq[ROT_UN];
    bool live[ROT_UN], on[ROT_UN];  // on: the whole warp has this trip
#pragma unroll
    for (int u = 0; u < ROT_UN; ++u) {
      const int64_t q = q0 + u * stride;
      on[u] = q < limit;
      live[u] = q < quads;
      qq[u] = live[u] ? q : quads - 1;
      if (on[u]) {
        if constexpr (kSameType) Quad<Tin>::load(x + qq[u] * 4, mine[u]);
        else load_as_f32<Tin>(x + qq[u] * 4, mine[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < ROT_UN; ++u) {
      if (!on[u]) continue;
      const int g = (int)((qq[u] >> 2) % groups_per_row);
      const bool flagged = flags[g] != 0;
      if constexpr (!kSameType || sizeof(Tin) == 4) {
        if (col_scale != nullptr) {
          float4 s = *reinterpret_cast<const float4*>(col_scale + (int64_t)g * 16 + (lane & 3) * 4);
          mine[u][0] *= s.x, mine[u][1] *= s.y, mine[u][2] *= s.z, mine[u][3] *= s.w;
        }
      }
      C out[4];
      rotate_quad<C>(mine[u], lane, out);
      if (live[u]) Quad<Tout>::store(y + qq[u] * 4, flagged ? out : mine[u]);
    }
  }
}

template <typename Tin, typename Tout, bool kSame>
int launch(const void* x, void* y, const uint8_t* flags, const float* scale, int64_t rows, int64_t k,
           cudaStream_t stream) {
  const int64_t quads = rows * k / 4;
  if (quads == 0) return HI2_OK;
  int64_t blocks = ceil_div(quads, 256);
  const int64_t cap = 148 * 8 * 4;  // a few waves of resident blocks; the loop strides the rest
  if (blocks > cap) blocks = cap;
  rotate_kernel<Tin, Tout, kSame><<<(unsigned)blocks, 256, 0, stream>>>(
      static_cast<const Tin*>(x), static_cast<Tout*>(y), flags, scale, quads, (int)(k / 16));
  return check_launch("rotate_groups");
}

}  // namespace
}  // namespace hi2

extern "C" int hi2_rotate_groups(const void* x, int in_dtype, void* y, int out_dtype,
                                 const uint8_t* flags, const float* col_scale, int64_t rows,
                                 int64_t k, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(rows >= 0 && k > 0 && k % 16 == 0, "rotate_groups: k must be a positive multiple of 16");
  if (rows == 0) return HI2_OK;
  HI2_REQUIRE(x && y && flags, "rotate_groups: null pointer");
  HI2_REQUIRE(aligned16(x) && aligned16(y), "rotate_groups: x and y must be 16-byte aligned");
  HI2_REQUIRE(col_scale == nullptr || aligned16(col_scale), "rotate_groups: col_scale alignment");
  HI2_REQUIRE(col_scale == nullptr || out_dtype == HI2_F32,
              "rotate_groups: col_scale needs an fp32 output");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (in_dtype == HI2_F32 && out_dtype == HI2_F32)
    return launch<float, float, true>(x, y, flags, col_scale, rows, k, s);
  if (in_dtype == HI2_F64 && out_dtype == HI2_F64)
    return launch<double, double, true>(x, y, flags, nullptr, rows, k, s);
  if (in_dtype == HI2_F16 && out_dtype == HI2_F16)
    return launch<__half, __half, true>(x, y, flags, nullptr, rows, k, s);
  if (in_dtype == HI2_BF16 && out_dtype == HI2_BF16)
    return launch<__nv_bfloat16, __nv_bfloat16, true>(x, y, flags, nullptr, rows, k, s);
  if (in_dtype == HI2_F16 && out_dtype == HI2_F32)
    return launch<__half, float, false>(x, y, flags, col_scale, rows, k, s);
  if (in_dtype == HI2_BF16 && out_dtype == HI2_F32)
    return launch<__nv_bfloat16, float, false>(x, y, flags, col_scale, rows, k, s);
  return fail(HI2_ERR_ARG, "rotate_groups: unsupported dtype pair");
}
