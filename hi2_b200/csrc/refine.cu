// One block of columns of the +-1 refinement sweep (hi2/refine_kernel.py:51-120).
//
// One LANE per row, the mapping of the GPTQ block kernel.  The row's slice of g = e Hs (up to 128
// columns) lives in registers as 64 pairs that move down by one pair every two columns, so the
// columns being decided are always the first pair and every register index is static.  The block
// Hs[b0:b0+len, b0:b0+len] is staged in shared memory with every row already shifted to the column
// its first pair starts at, where Hs[j, c] is one address for all lanes (a broadcast).  A column's
// move is decided exactly as the reference kernel decides it: gain = -((2*dw)*g + (dw*dw)*H_jj),
// each operation rounded on its own; ties go to +1; NaN never moves; a move adds dw * Hs[j, q]
// (product and sum rounded separately) to every later column q of the block, in column order.  A
// column that does not move adds dw = 0, which leaves g as it is.  Codes, ladders and the output
// dw travel as 128-bit accesses, four columns at a time, one quad ahead of their use.
// (A warp per row with four columns per lane and a shuffle per column spent 45 warp instructions
// per row and column; this mapping spends about 7.)
#include "common.cuh"

namespace hi2 {
namespace {

constexpr int LMAX = 128;
constexpr int ROWS_PER_CTA = 64;
constexpr int H_DIAG = LMAX * LMAX;        // Hs[j, j] (padded with zeros)
constexpr int H_NEXT = H_DIAG + LMAX;      // Hs[j, j+1]
constexpr int H_STAGE_FLOATS = H_NEXT + LMAX;

// pair + dw * (h0, h1), product and sum rounded separately (a packed multiply feeding scalar adds:
// a packed add would be contracted into a packed FMA by the assembler).
__device__ __forceinline__ float2 add_scaled(float2 g, float2 dw, float h0, float h1) {
  const float2 p = __fmul2_rn(dw, make_float2(h0, h1));
  return make_float2(g.x + p.x, g.y + p.y);
}

// The move of one column: the new code and the change dw of its decoded value (0 when it stays).
__device__ __forceinline__ void decide(float gj, float cc, float lo_j, float st_j, float hd, float tp,
                                       float& c_out, float& dw_out) {
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
  const bool take = best > 0.0f;
  dw_out = take ? (pick_m ? dwm : dwp) : 0.0f;
  c_out = take ? (pick_m ? cm : cp) : cc;
}

// hi = tf32(x), lo = tf32(x - hi), round-to-nearest: the operand form of the tensor-core product
// that follows the block (lazy_tc.cu).
__device__ __forceinline__ void tf32_parts(float x, float& hi, float& lo) {
  uint32_t hb, lb;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(x));
  hi = __uint_as_float(hb);
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lb) : "f"(x - hi));
  lo = __uint_as_float(lb);
}
// Four changes dw: as they are, or (dw_lo given) as their TF32 parts.
__device__ __forceinline__ void store_dw(float* dw, float* dw_lo, float a, float b, float c, float d) {
  if (dw_lo == nullptr) {
    *reinterpret_cast<float4*>(dw) = make_float4(a, b, c, d);
    return;
  }
  float h[4], l[4];
  tf32_parts(a, h[0], l[0]), tf32_parts(b, h[1], l[1]), tf32_parts(c, h[2], l[2]), tf32_parts(d, h[3], l[3]);
  *reinterpret_cast<float4*>(dw) = make_float4(h[0], h[1], h[2], h[3]);
  *reinterpret_cast<float4*>(dw_lo) = make_float4(l[0], l[1], l[2], l[3]);
}

struct Quad4 {
  float v[4];
};
__device__ __forceinline__ Quad4 load4(const float* p) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  return {{t.x, t.y, t.z, t.w}};
}

// Steps while more than W - 32 columns remain (W registers live: g[0] holds columns j, j+1).
template <int W>
__device__ __forceinline__ void run_phase(float2 (&g)[LMAX / 2], int& j, int len, float tp,
                                          const float* __restrict__ h_stage, const float* c_in,
                                          const float* lo_in, const float* st_in, Quad4& cq, Quad4& lq, Quad4& sq,
                                          bool live, float* c_out, float* dw_out, float* dw_lo_out) {
  constexpr int P = W / 2;
#pragma unroll 1
  while (len - j > W - 32 && j < len) {
    const int j0 = j;  // a multiple of 4: the quad cq/lq/sq holds columns j0 .. j0+3
    Quad4 cn = cq, ln = lq, sn = sq;
    if (j0 + 4 < len) cn = load4(c_in + j0 + 4), ln = load4(lo_in + j0 + 4), sn = load4(st_in + j0 + 4);
    float cnew[4], dws[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int ja = j0 + 2 * h;                 // even column A, odd column B = A + 1
      const float* ha = h_stage + ja * LMAX;     // ha[t] = Hs[A, A+2+t]
      const float* hb = ha + LMAX;               // hb[t] = Hs[B, A+2+t]
      float dwa, dwb;
      decide(g[0].x, cq.v[2 * h], lq.v[2 * h], sq.v[2 * h], h_stage[H_DIAG + ja], tp, cnew[2 * h], dwa);
      const float gb = g[0].y + dwa * h_stage[H_NEXT + ja];
      decide(gb, cq.v[2 * h + 1], lq.v[2 * h + 1], sq.v[2 * h + 1], h_stage[H_DIAG + ja + 1], tp, cnew[2 * h + 1], dwb);
      dws[2 * h] = dwa, dws[2 * h + 1] = dwb;
      const float2 da = make_float2(dwa, dwa), db = make_float2(dwb, dwb);
#pragma unroll
      for (int t = 0; t + 1 < P; t += 2) {
        const float4 va = *reinterpret_cast<const float4*>(ha + 2 * t);
        const float4 vb = *reinterpret_cast<const float4*>(hb + 2 * t);
        g[t] = add_scaled(add_scaled(g[t + 1], da, va.x, va.y), db, vb.x, vb.y);
        if (t + 2 < P) g[t + 1] = add_scaled(add_scaled(g[t + 2], da, va.z, va.w), db, vb.z, vb.w);
      }
      g[P - 1] = make_float2(0.0f, 0.0f);
    }
    if (live) {
      *reinterpret_cast<float4*>(c_out + j0) = make_float4(cnew[0], cnew[1], cnew[2], cnew[3]);
      store_dw(dw_out + j0, dw_lo_out ? dw_lo_out + j0 : nullptr, dws[0], dws[1], dws[2], dws[3]);
    }
    cq = cn, lq = ln, sq = sn;
    j = j0 + 4;
  }
}

__global__ void __launch_bounds__(ROWS_PER_CTA, 3)
refine_block_kernel(const float* __restrict__ gb, int64_t ldg, int len, float* __restrict__ c,
                    const float* __restrict__ lo, const float* __restrict__ st,
                    const float* __restrict__ top, const float* __restrict__ hs, int64_t n_rows,
                    int64_t k, int64_t b0, float* __restrict__ dwb, float* __restrict__ dw_lo, int64_t lddw) {
  extern __shared__ float4 h_stage4[];
  float* h_stage = reinterpret_cast<float*>(h_stage4);
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  {
    // h_stage[j][t] = Hs[b0+j, b0+first(j)+t] with first(j) = j+2 for even j and j+1 for odd j (zero
    // past the block); then the diagonal and Hs[j, j+1]
    const float* src = hs + b0 * k + b0;
    for (int idx = threadIdx.x; idx < H_STAGE_FLOATS / 4; idx += ROWS_PER_CTA) h_stage4[idx] = zero4;
    __syncthreads();
    const int quads = len / 4;
    for (int idx = threadIdx.x; idx < len * quads; idx += ROWS_PER_CTA) {
      const int j = idx / quads, cc = (idx % quads) * 4;
      const int first = j + 2 - (j & 1);
      if (cc + 3 < first) continue;
      const float4 v = *reinterpret_cast<const float4*>(src + (int64_t)j * k + cc);
      float* dst = h_stage + j * LMAX + (cc - first);
      if (cc >= first) dst[0] = v.x;
      if (cc + 1 >= first) dst[1] = v.y;
      if (cc + 2 >= first) dst[2] = v.z;
      dst[3] = v.w;
    }
    for (int idx = threadIdx.x; idx < len; idx += ROWS_PER_CTA) {
      h_stage[H_DIAG + idx] = src[(int64_t)idx * k + idx];
      h_stage[H_NEXT + idx] = idx + 1 < len ? src[(int64_t)idx * k + idx + 1] : 0.0f;
    }
  }
  __syncthreads();

  const int64_t row_raw = (int64_t)blockIdx.x * ROWS_PER_CTA + threadIdx.x;
  const bool live = row_raw < n_rows;
  const int64_t row = live ? row_raw : n_rows - 1;  // spare lanes shadow the last row and store nothing
  const float tp = top[row];
  const float* grow = gb + row * ldg;
  float* crow = c + row * k + b0;
  const float* lorow = lo + row * k + b0;
  const float* strow = st + row * k + b0;
  float* dwrow = dwb + row * lddw;
  float* dwlrow = dw_lo ? dw_lo + row * lddw : nullptr;

  float2 g[LMAX / 2];
#pragma unroll
  for (int q = 0; q < LMAX / 4; ++q) {
    const float4 v = (4 * q < len) ? *reinterpret_cast<const float4*>(grow + 4 * q) : zero4;
    g[2 * q] = make_float2(v.x, v.y), g[2 * q + 1] = make_float2(v.z, v.w);
  }
  Quad4 cq = load4(crow), lq = load4(lorow), sq = load4(strow);
  int j = 0;
  run_phase<128>(g, j, len, tp, h_stage, crow, lorow, strow, cq, lq, sq, live, crow, dwrow, dwlrow);
  run_phase<96>(g, j, len, tp, h_stage, crow, lorow, strow, cq, lq, sq, live, crow, dwrow, dwlrow);
  run_phase<64>(g, j, len, tp, h_stage, crow, lorow, strow, cq, lq, sq, live, crow, dwrow, dwlrow);
  run_phase<32>(g, j, len, tp, h_stage, crow, lorow, strow, cq, lq, sq, live, crow, dwrow, dwlrow);
}

// The same block with a WARP per row, four consecutive columns per lane: the lane that owns column j
// decides the move, one shuffle tells the warp the change dw, every lane adds dw * Hs[j, q] to its
// columns q > j; rows of Hs arrive as one 128-bit load per lane, fetched four rows ahead.  Forty-five
// warp instructions per row and column against seven for the lane-per-row kernel, but 32 times the
// parallelism: with fewer rows than fill the SMs at a lane each (148 x 64) the block is a latency
// chain either way and this mapping finishes it sooner (49 us against ~70 us at 4096 rows).
constexpr int WARP_ROWS_PER_CTA = 8;

__global__ void __launch_bounds__(WARP_ROWS_PER_CTA * 32)
refine_block_warp_kernel(const float* __restrict__ gb, int64_t ldg, int len, float* __restrict__ c,
                    const float* __restrict__ lo, const float* __restrict__ st,
                    const float* __restrict__ top, const float* __restrict__ hs, int64_t n_rows,
                    int64_t k, int64_t b0, float* __restrict__ dwb, float* __restrict__ dw_lo, int64_t lddw) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * WARP_ROWS_PER_CTA + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int c0 = lane * 4;
  const bool mine = c0 < len;
  const float tp = top[row];
  const int64_t base = row * k + b0 + c0;

  float g[4] = {0.f, 0.f, 0.f, 0.f}, cj[4] = {0.f, 0.f, 0.f, 0.f}, lo_c[4] = {0.f, 0.f, 0.f, 0.f},
        st_c[4] = {0.f, 0.f, 0.f, 0.f}, dw_keep[4] = {0.f, 0.f, 0.f, 0.f};
  if (mine) {
    const float4 gv = *reinterpret_cast<const float4*>(gb + row * ldg + c0);
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
    store_dw(dwb + row * lddw + c0, dw_lo ? dw_lo + row * lddw + c0 : nullptr, dw_keep[0], dw_keep[1], dw_keep[2],
             dw_keep[3]);
  }
}

}  // namespace
}  // namespace hi2

namespace hi2 {
namespace {
int launch_refine_block(const float* gb, int64_t ldg, int len, float* c, const float* lo, const float* st,
                        const float* top, const float* hs, int64_t n_rows, int64_t k, int64_t b0, float* dwb,
                        float* dw_lo, int64_t lddw, cudaStream_t stream) {
  if (n_rows < (int64_t)148 * ROWS_PER_CTA) {  // too few rows to fill the SMs at a lane per row
    const unsigned wgrid = (unsigned)ceil_div(n_rows, WARP_ROWS_PER_CTA);
    refine_block_warp_kernel<<<wgrid, WARP_ROWS_PER_CTA * 32, 0, stream>>>(gb, ldg, len, c, lo, st, top, hs, n_rows,
                                                                            k, b0, dwb, dw_lo, lddw);
    return check_launch("refine_block");
  }
  const unsigned grid = (unsigned)ceil_div(n_rows, ROWS_PER_CTA);
  const int smem = H_STAGE_FLOATS * (int)sizeof(float);
  if (cudaFuncSetAttribute(refine_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return fail(HI2_ERR_LAUNCH, "refine_block: cannot reserve shared memory");
  refine_block_kernel<<<grid, ROWS_PER_CTA, smem, stream>>>(gb, ldg, len, c, lo, st, top, hs, n_rows, k, b0, dwb,
                                                             dw_lo, lddw);
  return check_launch("refine_block");
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
  return launch_refine_block(gb, len, len, c, lo, st, top, hs, n_rows, k, b0, dwb, nullptr, len,
                             static_cast<cudaStream_t>(stream));
}

extern "C" int hi2_refine_block_in_place(const float* g, int len, float* c, const float* lo, const float* st,
                                         const float* top, const float* hs, int64_t n_rows, int64_t k,
                                         int64_t b0, float* dw_hi, float* dw_lo, int64_t lddw, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(k > 0 && k % 16 == 0, "refine_block_in_place: k must be a positive multiple of 16");
  HI2_REQUIRE(len > 0 && len <= LMAX && len % 16 == 0, "refine_block_in_place: block length must be 16..128");
  HI2_REQUIRE(b0 >= 0 && b0 % 16 == 0 && b0 + len <= k, "refine_block_in_place: block outside the row");
  HI2_REQUIRE(lddw >= len && lddw % 4 == 0, "refine_block_in_place: lddw must cover the block and be a multiple of 4");
  if (n_rows == 0) return HI2_OK;
  HI2_REQUIRE(g && c && lo && st && top && hs && dw_hi && dw_lo, "refine_block_in_place: null pointer");
  HI2_REQUIRE(aligned16(g) && aligned16(c) && aligned16(lo) && aligned16(st) && aligned16(hs) &&
                  aligned16(dw_hi) && aligned16(dw_lo),
              "refine_block_in_place: buffers must be 16-byte aligned");
  return launch_refine_block(g + b0, k, len, c, lo, st, top, hs, n_rows, k, b0, dw_hi, dw_lo, lddw,
                             static_cast<cudaStream_t>(stream));
}
