// One block of columns of the +-1 refinement sweep (hi2/refine_kernel.py:51-120).
//
// Same mapping as the GPTQ block kernel: a warp per row, four consecutive columns per lane.  The
// lane's slice of g = e Hs lives in registers; the lane that owns column j decides the move
// from g_j, H_jj and the two neighbouring ladder values, one shuffle tells the warp the change
// dw, and every lane adds dw * Hs[j, q] to its columns q > j.  Rows of Hs arrive as one 128-bit
// load per lane, fetched four rows ahead.  The gain is formed exactly as the reference kernel
// does: -((2*dw)*g + (dw*dw)*H_jj), each operation rounded; ties go to +1; NaN never moves.
#include "common.cuh"

namespace hi2 {
namespace {

constexpr int LMAX = 128;
constexpr int ROWS_PER_CTA = 8;

__global__ void __launch_bounds__(ROWS_PER_CTA * 32)
refine_block_kernel(const float* __restrict__ gb, int len, float* __restrict__ c,
                    const float* __restrict__ lo, const float* __restrict__ st,
                    const float* __restrict__ top, const float* __restrict__ hs, int64_t n_rows,
                    int64_t k, int64_t b0, float* __restrict__ dwb) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * ROWS_PER_CTA + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int c0 = lane * 4;
  const bool mine = c0 < len;
  const float tp = top[row];
  const int64_t base = row * k + b0 + c0;

  float g[4] = {0.f, 0.f, 0.f, 0.f}, cj[4] = {0.f, 0.f, 0.f, 0.f}, lo_c[4] = {0.f, 0.f, 0.f, 0.f},
        st_c[4] = {0.f, 0.f, 0.f, 0.f}, dw_keep[4] = {0.f, 0.f, 0.f, 0.f};
  if (mine) {
    const float4 gv = *reinterpret_cast<const float4*>(gb + row * len + c0);
    const float4 cv = *reinterpret_cast<const float4*>(c + base);
    const float4 lv = *reinterpret_cast<const float4*>(lo + base);
    const float4 sv = *reinterpret_cast<const float4*>(st + base);
    g[0] = gv.x, g[1] = gv.y, g[2] = gv.z, g[3] = gv.w;
    cj[0] = cv.x, cj[1] = cv.y, cj[2] = cv.z, cj[3] = cv.w;
    lo_c[0] = lv.x, lo_c[1] = lv.y, lo_c[2] = lv.z, lo_c[3] = lv.w;
    st_c[0] = sv.x, st_c[1] = sv.y, st_c[2] = sv.z, st_c[3] = sv.w;
  }

  const float* hrow = hs + b0 * k + b0 + c0;  // row b0 of Hs, this lane's columns
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 ahead[4];
#pragma unroll
  for (int s = 0; s < 4; ++s)
    ahead[s] = mine ? *reinterpret_cast<const float4*>(hrow + (int64_t)s * k) : zero4;

  for (int i = 0; i < len; i += 4) {
    float4 cur[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) cur[s] = ahead[s];
    if (i + 4 < len) {
#pragma unroll
      for (int s = 0; s < 4; ++s)
        ahead[s] = mine ? *reinterpret_cast<const float4*>(hrow + (int64_t)(i + 4 + s) * k) : zero4;
    }
    const int owner = i >> 2;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int jj = i + s;
      const float hv[4] = {cur[s].x, cur[s].y, cur[s].z, cur[s].w};
      const float lo_j = lo_c[s], st_j = st_c[s], cc = cj[s], gj = g[s], hd = hv[s];
      const float now = round_f16(lo_j + cc * st_j);
      const float cp = cc + 1.0f, cm = cc - 1.0f;
      const bool okp = (cp >= 0.0f) && (cp <= tp) && (st_j > 0.0f);
      const bool okm = (cm >= 0.0f) && (cm <= tp) && (st_j > 0.0f);
      const float dwp = round_f16(lo_j + cp * st_j) - now;
      const float dwm = round_f16(lo_j + cm * st_j) - now;
      const float gp = okp ? -(((2.0f * dwp) * gj) + ((dwp * dwp) * hd)) : -INFINITY;
      const float gm = okm ? -(((2.0f * dwm) * gj) + ((dwm * dwm) * hd)) : -INFINITY;
      const bool pick_m = gm > gp;
      const float best = pick_m ? gm : gp;
      const bool take_own = best > 0.0f;
      const float dw_own = take_own ? (pick_m ? dwm : dwp) : 0.0f;
      const float dw = __shfl_sync(0xffffffffu, dw_own, owner);
      const bool take = __shfl_sync(0xffffffffu, (int)take_own, owner) != 0;
      if (lane == owner) {
        dw_keep[s] = dw_own;
        if (take_own) cj[s] = pick_m ? cm : cp;
      }
      if (take) {
#pragma unroll
        for (int t = 0; t < 4; ++t)
          if (c0 + t > jj) g[t] = g[t] + dw * hv[t];
      }
    }
  }

  if (mine) {
    *reinterpret_cast<float4*>(c + base) = make_float4(cj[0], cj[1], cj[2], cj[3]);
    *reinterpret_cast<float4*>(dwb + row * len + c0) =
        make_float4(dw_keep[0], dw_keep[1], dw_keep[2], dw_keep[3]);
  }
}

}  // namespace
}  // namespace hi2

extern "C" int hi2_refine_block(const float* gb, int len, float* c, const float* lo,
                                const float* st, const float* top, const float* hs, int64_t n_rows,
                                int64_t k, int64_t b0, float* dwb, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(k > 0 && k % 16 == 0, "refine_block: k must be a positive multiple of 16");
  HI2_REQUIRE(len > 0 && len <= LMAX && len % 16 == 0, "refine_block: block length must be 16..128");
  HI2_REQUIRE(b0 >= 0 && b0 % 16 == 0 && b0 + len <= k, "refine_block: block outside the row");
  if (n_rows == 0) return HI2_OK;
  HI2_REQUIRE(gb && c && lo && st && top && hs && dwb, "refine_block: null pointer");
  HI2_REQUIRE(aligned16(gb) && aligned16(c) && aligned16(lo) && aligned16(st) && aligned16(hs) &&
                  aligned16(dwb),
              "refine_block: buffers must be 16-byte aligned");
  const unsigned grid = (unsigned)ceil_div(n_rows, ROWS_PER_CTA);
  refine_block_kernel<<<grid, ROWS_PER_CTA * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      gb, len, c, lo, st, top, hs, n_rows, k, b0, dwb);
  return check_launch("refine_block");
}
