// Order-16 Hadamard rotation of flagged column groups, fused with the load-side cast and the
// smoothing multiply (hi2/format.py:30-41, hi2/calibrate.py:243-251).
//
// Layout: the [rows, k] matrix is one flat array of 16-element groups and a THREAD owns a whole
// group: 16 consecutive elements arrive as 128-bit loads (two for bf16/fp16, four for fp32), the
// 16 outputs leave the same way, and nothing is exchanged between lanes.  Adjacent lanes read
// adjacent 32- or 64-byte pieces, so a warp's accesses cover one contiguous run and every DRAM
// sector is fetched once (the second load of a lane finds the other half of its sector in L1).
// Every output is the left-to-right sum over k = 0..15 of x_k * (+-1/4) with compile-time signs:
// the products are exact, so the result equals a row-times-matrix product accumulated in ascending
// k, which is what the reference's CPU product gives bit for bit (a radix-2 butterfly does not).
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
    __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));  // written once, read much later
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

// Tin == Tout (C = compute type of the pair) or Tin half/bf16 with Tout float.
template <typename Tin, typename Tout, bool kSameType>
__global__ void __launch_bounds__(256)
rotate_kernel(const Tin* __restrict__ x, Tout* __restrict__ y, const uint8_t* __restrict__ flags,
              const float* __restrict__ col_scale, int64_t groups, int groups_per_row) {
  using C = typename std::conditional<kSameType, typename Quad<Tin>::C, float>::type;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gid < groups; gid += stride) {
    C v[16];
    if constexpr (!kSameType && sizeof(Tin) == 2) {  // 32 bytes: two 128-bit loads, unpacked from registers
      const uint4 lo = *reinterpret_cast<const uint4*>(x + gid * 16);
      const uint4 hi = *reinterpret_cast<const uint4*>(x + gid * 16 + 8);
      const uint32_t raw[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if constexpr (std::is_same<Tin, __nv_bfloat16>::value) {
          v[2 * i] = __uint_as_float(raw[i] << 16), v[2 * i + 1] = __uint_as_float(raw[i] & 0xffff0000u);
        } else {
          const __half2 h = *reinterpret_cast<const __half2*>(&raw[i]);
          v[2 * i] = __low2float(h), v[2 * i + 1] = __high2float(h);
        }
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if constexpr (kSameType) Quad<Tin>::load(x + gid * 16 + q * 4, &v[q * 4]);
        else load_as_f32<Tin>(x + gid * 16 + q * 4, &v[q * 4]);
      }
    }
    const int g = (int)(gid % groups_per_row);
    if constexpr (!kSameType || sizeof(Tin) == 4) {
      if (col_scale != nullptr) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 sc = __ldg(reinterpret_cast<const float4*>(col_scale + (int64_t)g * 16 + q * 4));
          v[q * 4] *= sc.x, v[q * 4 + 1] *= sc.y, v[q * 4 + 2] *= sc.z, v[q * 4 + 3] *= sc.w;
        }
      }
    }
    if (__ldg(flags + g) != 0) {
      // All 16 outputs of the group, each the k-ascending sum.  (Measured alternatives, all slower on
      // the 11008 x 4096 bf16 -> fp32 case at 72 us: four lanes per group with shuffles 82 us; two
      // groups per trip, 96 registers, 81 us; four outputs at a time capped at 40 registers 85 us.)
      C out[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        C acc = C(0);
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) acc = fma_c(v[kk], (__popc(kk & j) & 1) ? C(-0.25) : C(0.25), acc);
        out[j] = acc;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) Quad<Tout>::store(y + gid * 16 + q * 4, &out[q * 4]);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) Quad<Tout>::store(y + gid * 16 + q * 4, &v[q * 4]);
    }
  }
}

template <typename Tin, typename Tout, bool kSame>
int launch(const void* x, void* y, const uint8_t* flags, const float* scale, int64_t rows, int64_t k,
           cudaStream_t stream) {
  const int64_t groups = rows * k / 16;
  if (groups == 0) return HI2_OK;
  int64_t blocks = ceil_div(groups, 256);
  const int64_t cap = 148 * 8 * 4;  // a few waves of resident blocks; the loop strides the rest
  if (blocks > cap) blocks = cap;
  rotate_kernel<Tin, Tout, kSame><<<(unsigned)blocks, 256, 0, stream>>>(
      static_cast<const Tin*>(x), static_cast<Tout*>(y), flags, scale, groups, (int)(k / 16));
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
