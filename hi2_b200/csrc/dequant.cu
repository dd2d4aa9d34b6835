// The inverse path of the format (hi2/format.py:195-239 dequantize_stored, dequantize; the decode
// arithmetic of :45-69): flat per-tensor buffers -> the fp16 reconstruction of every weight, in the
// stored (rotated, smoothed) basis or back in the original one.
//
// A thread owns one 16-column group of one row: it finds the row's code width, block size and
// offsets, unpacks the group's 16 codes (one, two or four words), decodes the block's ladder
// (lo = fp16(fma_f32(u, lo_scale, lo_min)), step = fp16(u * step_scale)), forms fp16(lo + c * step)
// with the sum exact in fp64 and one rounding, and - for the original basis - applies the group's
// rotation (sums of sixteen fp16 values times 1/4: exact in fp64 in any order) and divides by the
// smoothing vector (a correctly rounded fp64 quotient).  Every step is exact or correctly rounded,
// so the fp64 output equals the reference's on any device, bit for bit.  Output is fp64 (the
// reference's type) or fp32 (the fp64 value rounded once).  Traffic: about nbits/8 bytes per weight
// in, 4 or 8 bytes out: bound by the stores.
#include "common.cuh"

namespace hi2 {
namespace {

template <typename OUT, bool ORIGINAL>
__global__ void __launch_bounds__(256)
dequant_kernel(const int32_t* __restrict__ codes, const int32_t* __restrict__ code_off,
               const uint8_t* __restrict__ blk_params, const int32_t* __restrict__ param_off,
               const uint16_t* __restrict__ row_consts, const uint8_t* __restrict__ row_nbits,
               const uint8_t* __restrict__ row_block, const uint8_t* __restrict__ had,
               const uint16_t* __restrict__ col_scale, int64_t rows, int64_t k, OUT* __restrict__ out,
               int32_t* __restrict__ bad) {
  const int64_t groups_per_row = k / 16;
  const int64_t total = rows * groups_per_row;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gid < total; gid += stride) {
    const int64_t row = gid / groups_per_row;
    const int g = (int)(gid % groups_per_row);
    const int nbits = row_nbits[row], block = row_block[row];
    if ((nbits != 2 && nbits != 4 && nbits != 8) || (block != 16 && block != 32 && block != 64)) {
      atomicOr(bad, 1);  // not a row of this format: leave the output untouched
      continue;
    }
    // the group's 16 codes: 16 * nbits bits = nbits / 2 words, starting at word g * nbits / 2
    const int32_t* wp = codes + (int64_t)code_off[row] + (int64_t)g * (nbits / 2);
    uint32_t c[16];
    if (nbits == 2) {
      const uint32_t w0 = (uint32_t)wp[0];
#pragma unroll
      for (int i = 0; i < 16; ++i) c[i] = (w0 >> (2 * i)) & 3u;
    } else if (nbits == 4) {
      const uint32_t w0 = (uint32_t)wp[0], w1 = (uint32_t)wp[1];
#pragma unroll
      for (int i = 0; i < 8; ++i) c[i] = (w0 >> (4 * i)) & 15u, c[8 + i] = (w1 >> (4 * i)) & 15u;
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t w = (uint32_t)wp[q];
#pragma unroll
        for (int i = 0; i < 4; ++i) c[4 * q + i] = (w >> (8 * i)) & 255u;
      }
    }
    // the ladder of the block this group lies in
    const int64_t blk = (int64_t)param_off[row] + (int64_t)g * 16 / block;
    const float lo_u = (float)blk_params[2 * blk], st_u = (float)blk_params[2 * blk + 1];
    const float lo_min = __half2float(__ushort_as_half(row_consts[row * 3 + 0]));
    const float lo_scale = __half2float(__ushort_as_half(row_consts[row * 3 + 1]));
    const float st_scale = __half2float(__ushort_as_half(row_consts[row * 3 + 2]));
    const double lo = (double)round_f16(fmaf(lo_u, lo_scale, lo_min));
    const double st = (double)round_f16(st_u * st_scale);
    double v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i)
      v[i] = (double)__half2float(__double2half(fma((double)c[i], st, lo)));  // exact sum, one rounding
    if (ORIGINAL) {
      if (had[g] != 0) {
        double y[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          double acc = 0.0;
#pragma unroll
          for (int i = 0; i < 16; ++i) acc += (__popc(i & j) & 1) ? -v[i] : v[i];
          y[j] = acc * 0.25;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = y[j];
      }
      if (col_scale != nullptr) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          v[j] = v[j] / (double)__half2float(__ushort_as_half(col_scale[(int64_t)g * 16 + j]));
      }
    }
    OUT* dst = out + row * k + (int64_t)g * 16;
#pragma unroll
    for (int j = 0; j < 16; ++j) dst[j] = (OUT)v[j];
  }
}

}  // namespace
}  // namespace hi2

extern "C" int hi2_dequantize(const int32_t* codes, const int32_t* code_off, const uint8_t* blk_params,
                              const int32_t* param_off, const uint16_t* row_consts,
                              const uint8_t* row_nbits, const uint8_t* row_block, const uint8_t* had,
                              const uint16_t* col_scale, int64_t rows, int64_t k, int original_basis,
                              void* out, int out_dtype, int32_t* bad, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(rows >= 0 && k > 0 && k % 64 == 0, "dequantize: k must be a positive multiple of 64");
  if (rows == 0) return HI2_OK;
  HI2_REQUIRE(codes && code_off && blk_params && param_off && row_consts && row_nbits && row_block && out && bad,
              "dequantize: null pointer");
  HI2_REQUIRE(!original_basis || had != nullptr, "dequantize: the original basis needs the rotation flags");
  HI2_REQUIRE(out_dtype == HI2_F64 || out_dtype == HI2_F32, "dequantize: output must be fp64 or fp32");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t total = rows * (k / 16);
  int64_t blocks = ceil_div(total, 256);
  if (blocks > 148 * 32) blocks = 148 * 32;
  const unsigned grid = (unsigned)blocks;
#define HI2_DEQ(T, ORIG)                                                                                   \
  dequant_kernel<T, ORIG><<<grid, 256, 0, s>>>(codes, code_off, blk_params, param_off, row_consts, row_nbits, \
                                               row_block, had, col_scale, rows, k, static_cast<T*>(out), bad)
  if (out_dtype == HI2_F64) {
    if (original_basis) HI2_DEQ(double, true);
    else HI2_DEQ(double, false);
  } else {
    if (original_basis) HI2_DEQ(float, true);
    else HI2_DEQ(float, false);
  }
#undef HI2_DEQ
  return check_launch("dequantize");
}
