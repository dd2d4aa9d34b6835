// Ladder search and row quantisation (hi2/encode.py:53-173, hi2/ladder_kernel.py:44-101).
//
// fit kernel   one thread per (row, block).  The 32 lanes of a warp take 32 consecutive ROWS of
//              the same block, so the column weights d of the block are warp-uniform (one
//              broadcast load serves the warp) and the block's weights stay in registers for the
//              whole grid search and the least-squares refits.  The work is ~800 fp32
//              instructions per weight (effort "normal") against 4 bytes read: ALU-bound.
// row kernel   one thread block per row: row-wide extrema of (lo, step), the three fp16 row
//              constants, the parameter bytes, the decoded fp16 ladders, and optionally the
//              nearest codes and the weighted error of the row.  One pass over the row: HBM-bound.
#include "common.cuh"

namespace hi2 {
namespace {

struct GridSpec {
  float v[8];
  int g;
};

// Codes are rint((x - lo) / safe) with an IEEE division in the reference.  Here one correctly
// rounded reciprocal of `safe` serves the block and every quotient is finished with Markstein's
// fused correction (div_by), which yields the correctly rounded quotient itself, so rint sees the
// very number the division would give.  Divisors outside the range the correction covers
// (rc.fast false: tiny, huge, or a significand of all ones) take true divisions.
//
// WIDE (blocks of 16 and 32): the column weights d and the differences x - lo of the current grid
// row are kept in registers next to x, which removes one load and one subtraction per element
// and pass; a block of 64 has no registers to spare for that.
template <int B, bool WIDE>
struct BlockRegs {
  float x[B];
  float d[WIDE ? B : 1];
  float a[WIDE ? B : 1];  // x - lo of the current lo
};

// Block sums are formed in the order of torch's CPU reduction over a contiguous inner dimension
// (aten/src/ATen/native/cpu/SumKernel.cpp): the block is read as B/8 vectors of 8 lanes, four
// interleaved vector accumulators take vectors 0-3 and then 4-7, the accumulators are added left
// to right, and the 8 lanes of the result are added left to right.  The reference's (lo, step)
// depend on these sums to the last bit (the least-squares formulas cancel), so with this order
// the search returns the reference's ladders bit for bit; a plain left-to-right sum does not.
template <int B>
__device__ __forceinline__ float fold_lane(const float (&v)[B / 8]) {
  if constexpr (B == 16) {
    return v[0] + v[1];
  } else if constexpr (B == 32) {
    return ((v[0] + v[1]) + v[2]) + v[3];
  } else {
    return (((v[0] + v[4]) + (v[1] + v[5])) + (v[2] + v[6])) + (v[3] + v[7]);
  }
}

template <int B, bool WIDE>
__device__ __forceinline__ float block_error(const BlockRegs<B, WIDE>& r, const float* __restrict__ dd,
                                             bool a_valid, float lo, float step, float nmax) {
  const float safe = (step == 0.0f) ? 1.0f : step;
  const Recip rc = make_recip(safe);
  float err = 0.0f;
  if (rc.fast) {
#pragma unroll
    for (int l = 0; l < 8; ++l) {
      float v[B / 8];
#pragma unroll
      for (int j = 0; j < B / 8; ++j) {
        const int t = 8 * j + l;
        const float num = (WIDE && a_valid) ? r.a[t] : r.x[t] - lo;
        const float q0 = num * rc.r;
        float q = rintf(fmaf(fmaf(-q0, safe, num), rc.r, q0));
        q = fminf(fmaxf(q, 0.0f), nmax);
        const float diff = (lo + q * step) - r.x[t];
        v[j] = (WIDE ? r.d[t] : __ldg(dd + t)) * (diff * diff);
      }
      const float s = fold_lane<B>(v);
      err = (l == 0) ? s : err + s;
    }
  } else {
#pragma unroll
    for (int l = 0; l < 8; ++l) {
      float v[B / 8];
#pragma unroll
      for (int j = 0; j < B / 8; ++j) {
        const int t = 8 * j + l;
        float q = rintf(__fdiv_rn(r.x[t] - lo, safe));
        q = fminf(fmaxf(q, 0.0f), nmax);
        const float diff = (lo + q * step) - r.x[t];
        v[j] = (WIDE ? r.d[t] : __ldg(dd + t)) * (diff * diff);
      }
      const float s = fold_lane<B>(v);
      err = (l == 0) ? s : err + s;
    }
  }
  return err;
}

// Two ladders with the same lo at once (two neighbouring points of a grid row): the differences
// x - lo and the column weights are fetched once, and the two error sums are independent chains,
// which doubles the instruction-level parallelism of the loop.  Each sum is formed exactly as
// block_error forms it.
template <int B, bool WIDE>
__device__ __forceinline__ void block_error2(const BlockRegs<B, WIDE>& r, const float* __restrict__ dd, float lo,
                                             float step_a, float step_b, float nmax, float& err_a, float& err_b) {
  const float safe_a = (step_a == 0.0f) ? 1.0f : step_a, safe_b = (step_b == 0.0f) ? 1.0f : step_b;
  const Recip ra = make_recip(safe_a), rb = make_recip(safe_b);
  if (!(ra.fast && rb.fast)) {
    err_a = block_error<B, WIDE>(r, dd, true, lo, step_a, nmax);
    err_b = block_error<B, WIDE>(r, dd, true, lo, step_b, nmax);
    return;
  }
  float ea = 0.0f, eb = 0.0f;
#pragma unroll
  for (int l = 0; l < 8; ++l) {
    float va[B / 8], vb[B / 8];
#pragma unroll
    for (int j = 0; j < B / 8; ++j) {
      const int t = 8 * j + l;
      const float num = WIDE ? r.a[t] : r.x[t] - lo;
      const float dt = WIDE ? r.d[t] : __ldg(dd + t);
      const float qa0 = num * ra.r, qb0 = num * rb.r;
      float qa = rintf(fmaf(fmaf(-qa0, safe_a, num), ra.r, qa0));
      float qb = rintf(fmaf(fmaf(-qb0, safe_b, num), rb.r, qb0));
      qa = fminf(fmaxf(qa, 0.0f), nmax);
      qb = fminf(fmaxf(qb, 0.0f), nmax);
      const float da = (lo + qa * step_a) - r.x[t], db = (lo + qb * step_b) - r.x[t];
      va[j] = dt * (da * da);
      vb[j] = dt * (db * db);
    }
    const float sa = fold_lane<B>(va), sb = fold_lane<B>(vb);
    ea = (l == 0) ? sa : ea + sa;
    eb = (l == 0) ? sb : eb + sb;
  }
  err_a = ea, err_b = eb;
}

template <int B, bool WIDE>
__global__ void __launch_bounds__(256, (B == 16 ? 3 : 2))
fit_kernel(const float* __restrict__ w, int64_t ldw, const float* __restrict__ d,
           const int32_t* __restrict__ row_d, int64_t n_rows, int64_t nb, GridSpec grid, int refits, float nmax, float* __restrict__ lo_out,
           float* __restrict__ st_out, float* __restrict__ err_out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t blk = (int64_t)blockIdx.y * 8 + warp;
  if (blk >= nb) return;  // uniform over the warp
  const int64_t row = (int64_t)blockIdx.x * 32 + lane;
  const bool live = row < n_rows;
  const int64_t row_c = live ? row : n_rows - 1;
  const float* src = w + row_c * ldw + blk * B;
  // row_d given: d is [groups, k] and row r is weighted by d[row_d[r]] (tensors that read different
  // inputs, e.g. the experts of a layer, searched in one launch)
  const float* dd = d + (row_d != nullptr ? (int64_t)row_d[row_c] * (nb * B) : 0) + blk * B;

  BlockRegs<B, WIDE> r;
#pragma unroll
  for (int t = 0; t < B; t += 4) {
    const float4 v = *reinterpret_cast<const float4*>(src + t);
    r.x[t] = v.x, r.x[t + 1] = v.y, r.x[t + 2] = v.z, r.x[t + 3] = v.w;
    if (WIDE) {
      const float4 dv = __ldg(reinterpret_cast<const float4*>(dd + t));
      r.d[t] = dv.x, r.d[t + 1] = dv.y, r.d[t + 2] = dv.z, r.d[t + 3] = dv.w;
    }
  }
  float mn = r.x[0], mx = r.x[0];
#pragma unroll
  for (int t = 1; t < B; ++t) mn = fminf(mn, r.x[t]), mx = fmaxf(mx, r.x[t]);
  const float span = mx - mn;
  const Recip rc_n = make_recip(nmax);  // nmax is 3, 15 or 255: div_by is the IEEE quotient

  float best_lo = 0.0f, best_st = 0.0f, best_err = 0.0f;
  for (int gi = 0; gi < grid.g; ++gi) {
    const float lo = mn + grid.v[gi] * span;
    if (WIDE) {
#pragma unroll
      for (int t = 0; t < B; ++t) r.a[t] = r.x[t] - lo;
    }
    int gj = 0;
    // Blocks of 64 take two grid points per pass, in their order (6 % faster); the narrower blocks
    // keep x - lo and d in registers and have none left for a second chain.
    for (; !WIDE && gj + 1 < grid.g; gj += 2) {
      const float step_a = div_by((mx - grid.v[gj] * span) - lo, nmax, rc_n);
      const float step_b = div_by((mx - grid.v[gj + 1] * span) - lo, nmax, rc_n);
      float err_a, err_b;
      block_error2<B, WIDE>(r, dd, lo, step_a, step_b, nmax, err_a, err_b);
      if ((gi | gj) == 0 || err_a < best_err) best_lo = lo, best_st = step_a, best_err = err_a;
      if (err_b < best_err) best_lo = lo, best_st = step_b, best_err = err_b;
    }
    for (; gj < grid.g; ++gj) {
      const float step = div_by((mx - grid.v[gj] * span) - lo, nmax, rc_n);
      const float err = block_error<B, WIDE>(r, dd, true, lo, step, nmax);
      if ((gi | gj) == 0 || err < best_err) best_lo = lo, best_st = step, best_err = err;
    }
  }

  for (int it = 0; it < refits; ++it) {
    const float safe = (best_st == 0.0f) ? 1.0f : best_st;
    const Recip rc = make_recip(safe);
    float sd = 0.f, sc = 0.f, scc = 0.f, sw = 0.f, scw = 0.f, sum = 0.f;
#pragma unroll
    for (int l = 0; l < 8; ++l) {
      float vd[B / 8], vc[B / 8], vcc[B / 8], vw[B / 8], vcw[B / 8], vx[B / 8];
#pragma unroll
      for (int j = 0; j < B / 8; ++j) {
        const int t = 8 * j + l;
        const float num = r.x[t] - best_lo;
        float c;
        if (rc.fast) {
          const float q0 = num * rc.r;
          c = rintf(fmaf(fmaf(-q0, safe, num), rc.r, q0));
        } else {
          c = rintf(__fdiv_rn(num, safe));
        }
        c = fminf(fmaxf(c, 0.0f), nmax);
        const float dt = WIDE ? r.d[t] : __ldg(dd + t), dc = dt * c;
        vd[j] = dt, vc[j] = dc, vcc[j] = dc * c, vw[j] = dt * r.x[t], vcw[j] = dc * r.x[t], vx[j] = r.x[t];
      }
      const float fd = fold_lane<B>(vd), fc = fold_lane<B>(vc), fcc = fold_lane<B>(vcc), fw = fold_lane<B>(vw),
                  fcw = fold_lane<B>(vcw), fx = fold_lane<B>(vx);
      if (l == 0) {
        sd = fd, sc = fc, scc = fcc, sw = fw, scw = fcw, sum = fx;
      } else {
        sd += fd, sc += fc, scc += fcc, sw += fw, scw += fcw, sum += fx;
      }
    }
    const float det = sd * scc - sc * sc;
    const bool ok = fabsf(det) > 1e-20f;
    const float step = ok ? __fdiv_rn(sd * scw - sc * sw, det) : 0.0f;
    const float lo = ok ? __fdiv_rn(sw - step * sc, fmaxf(sd, 1e-20f)) : __fdiv_rn(sum, (float)B);
    const float err = block_error<B, WIDE>(r, dd, false, lo, step, nmax);
    if (err < best_err && step > 0.0f) best_lo = lo, best_st = step, best_err = err;
  }

  if (live) {
    const int64_t o = row * nb + blk;
    lo_out[o] = best_lo;
    st_out[o] = best_st;
    if (err_out != nullptr) err_out[o] = best_err;
  }
}

int launch_fit(const float* w, int64_t ldw, const float* d, const int32_t* row_d, const float* grid_host, int g,
               int refits, int n, int64_t n_rows, int64_t nb, int block, float* lo, float* st,
               float* err, cudaStream_t stream) {
  GridSpec spec;
  spec.g = g;
  for (int i = 0; i < 8; ++i) spec.v[i] = i < g ? grid_host[i] : 0.0f;
  dim3 grid((unsigned)ceil_div(n_rows, 32), (unsigned)ceil_div(nb, 8));
  const float nmax = (float)(n - 1);
#define HI2_FIT(BB)                                                                              \
  fit_kernel<BB, (BB <= 32)><<<grid, 256, 0, stream>>>(w, ldw, d, row_d, n_rows, nb, spec, refits, nmax, lo, st, err)
  if (block == 16) HI2_FIT(16);
  if (block == 32) HI2_FIT(32);
  if (block == 64) HI2_FIT(64);
#undef HI2_FIT
  return check_launch("fit_ladder");
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int ROW_THREADS = 256;
constexpr int ROW_WARPS = ROW_THREADS / 32;
constexpr int ROW_UN = 4;  // quads a lane loads before it computes

// One WARP per row: the row-wide extrema, the constants and the parameter bytes need only warp
// shuffles, so no thread block barrier sits between the phases of a row and 64 rows are in flight
// per SM.  Dynamic shared memory: per warp the decoded lo[nb], step[nb] of its row.
// CODES / ENERGY: whether code bytes are written and the row energy is summed.  The tables ask for
// neither on five of their six passes, and the pass is bound by instruction issue (73 % of the
// issue slots at a third of the copy bandwidth), so the instructions of unused outputs are compiled out.
template <int B, bool CODES, bool ENERGY>
__global__ void __launch_bounds__(ROW_THREADS, 4)
row_kernel(const float* __restrict__ lo_in, const float* __restrict__ st_in,
           const float* __restrict__ w, int64_t ldw, const float* __restrict__ d_all,
           const int32_t* __restrict__ row_d, float nmax, int64_t n_rows, int64_t k, uint8_t* __restrict__ params, uint16_t* __restrict__ consts,
           float* __restrict__ lo_d, float* __restrict__ st_d, int64_t ldp,
           uint8_t* __restrict__ codes, float* __restrict__ sse, float* __restrict__ energy) {
  extern __shared__ float dyn[];
  const int64_t nb = k / B;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* s_lo = dyn + (size_t)warp * 2 * nb;
  float* s_st = s_lo + nb;

  for (int64_t row = (int64_t)blockIdx.x * ROW_WARPS + warp; row < n_rows; row += (int64_t)gridDim.x * ROW_WARPS) {
    const float* lo_r = lo_in + row * nb;
    const float* st_r = st_in + row * nb;
    // ---- row-wide extrema -----------------------------------------------------------------
    float mxst = -INFINITY, mnlo = INFINITY, mxlo = -INFINITY;
    for (int64_t b = lane; b < nb; b += 32) {
      const float s = st_r[b], l = lo_r[b];
      mxst = fmaxf(mxst, s < 0.0f ? 0.0f : s);
      mnlo = fminf(mnlo, l);
      mxlo = fmaxf(mxlo, l);
    }
    mxst = warp_max(mxst), mnlo = warp_min(mnlo), mxlo = warp_max(mxlo);
    // ---- the three fp16 row constants -------------------------------------------------------
    const __half ss_h = __float2half_rn(__fdiv_rn(mxst, 255.0f));
    const float ss = __half2float(ss_h);
    const __half lm_h = __float2half_rn(mnlo);
    const float lm = __half2float(lm_h);
    float spread = mxlo - lm;
    spread = spread < 0.0f ? 0.0f : spread;
    const __half ls_h = __float2half_rn(__fdiv_rn(spread, 255.0f));
    const float ls = __half2float(ls_h);
    if (lane == 0 && consts != nullptr) {
      consts[row * 3 + 0] = __half_as_ushort(lm_h);
      consts[row * 3 + 1] = __half_as_ushort(ls_h);
      consts[row * 3 + 2] = __half_as_ushort(ss_h);
    }
    // ---- parameter bytes and decoded ladders ------------------------------------------------
    __syncwarp();  // the previous row's readers of s_lo / s_st are done
    for (int64_t b = lane; b < nb; b += 32) {
      float s = st_r[b];
      s = s < 0.0f ? 0.0f : s;
      float su = 0.0f, lu = 0.0f;
      if (ss > 0.0f) su = clamp_keep_nan(rintf(__fdiv_rn(s, fmaxf(ss, 1e-30f))), 0.0f, 255.0f);
      if (ls > 0.0f)
        lu = clamp_keep_nan(rintf(__fdiv_rn(lo_r[b] - lm, fmaxf(ls, 1e-30f))), 0.0f, 255.0f);
      const uint8_t su8 = (uint8_t)su, lu8 = (uint8_t)lu;
      const float lod = round_f16(fmaf((float)lu8, ls, lm));
      const float std_ = round_f16((float)su8 * ss);
      s_lo[b] = lod;
      s_st[b] = std_;
      if (params != nullptr) {
        params[(row * nb + b) * 2 + 0] = lu8;
        params[(row * nb + b) * 2 + 1] = su8;
      }
      if (lo_d != nullptr) lo_d[row * ldp + b] = lod;
      if (st_d != nullptr) st_d[row * ldp + b] = std_;
    }
    if (sse == nullptr && codes == nullptr && energy == nullptr) continue;
    __syncwarp();
    // ---- nearest codes, weighted error, energy ------------------------------------------------
    // A lane takes ROW_UN quads per trip, all loads first, to keep enough bytes in flight.  Codes are
    // rint((w - lo) / step) with an IEEE division in the reference; the quotient is formed with the
    // block's correctly rounded reciprocal and Markstein's fused correction, which gives the same
    // correctly rounded number.
    const float* wr = w + row * ldw;
    const float* d = d_all + (row_d != nullptr ? (int64_t)row_d[row] * k : 0);  // the row's own column weights
    float acc = 0.0f, en = 0.0f;
    for (int64_t j0 = (int64_t)lane * 4; j0 < k; j0 += 128 * ROW_UN) {
      float4 wq[ROW_UN], dq[ROW_UN];
#pragma unroll
      for (int u = 0; u < ROW_UN; ++u) {
        const int64_t j = j0 + u * 128;
        if (j < k) {
          wq[u] = *reinterpret_cast<const float4*>(wr + j);
          dq[u] = *reinterpret_cast<const float4*>(d + j);
        }
      }
#pragma unroll
      for (int u = 0; u < ROW_UN; ++u) {
        const int64_t j = j0 + u * 128;
        if (j >= k) break;
        const int64_t b = j / B;
        const float lod = s_lo[b], std_ = s_st[b];
        const float safe = (std_ == 0.0f) ? 1.0f : std_;
        const Recip rc = make_recip(safe);
        const float ws[4] = {wq[u].x, wq[u].y, wq[u].z, wq[u].w}, ds[4] = {dq[u].x, dq[u].y, dq[u].z, dq[u].w};
        uint8_t cs[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float num = ws[t] - lod;
          float c;
          if (rc.fast) {
            const float q0 = num * rc.r;
            c = rintf(fmaf(fmaf(-q0, safe, num), rc.r, q0));
          } else {
            c = rintf(__fdiv_rn(num, safe));
          }
          if (std_ == 0.0f) c = 0.0f;
          c = clamp_keep_nan(c, 0.0f, nmax);
          const float diff = round_f16(lod + c * std_) - ws[t];
          acc += ds[t] * (diff * diff);
          if (ENERGY) en += ds[t] * (ws[t] * ws[t]);
          if (CODES) cs[t] = (uint8_t)c;
        }
        if (CODES) *reinterpret_cast<uchar4*>(codes + row * k + j) = make_uchar4(cs[0], cs[1], cs[2], cs[3]);
      }
    }
    acc = warp_sum(acc);
    if (ENERGY) en = warp_sum(en);
    if (lane == 0) {
      if (sse != nullptr) sse[row] = acc;
      if (ENERGY) energy[row] = en;
    }
  }
}

// sse of given codes against given decoded ladders (the tail of the GPTQ path).
template <int B>
__global__ void __launch_bounds__(ROW_THREADS)
sse_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ w, int64_t ldw,
           const float* __restrict__ d, const float* __restrict__ lo, const float* __restrict__ st,
           int64_t ldp, int64_t n_rows, int64_t k, float* __restrict__ sse) {
  __shared__ float red[ROW_THREADS / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
    float acc = 0.0f;
    for (int64_t j = (int64_t)tid * 4; j < k; j += ROW_THREADS * 4) {
      const float4 wv = *reinterpret_cast<const float4*>(w + row * ldw + j);
      const float4 dv = *reinterpret_cast<const float4*>(d + j);
      const uchar4 cv = *reinterpret_cast<const uchar4*>(codes + row * k + j);
      const float lod = lo[row * ldp + j / B], std_ = st[row * ldp + j / B];
      const float ws[4] = {wv.x, wv.y, wv.z, wv.w}, ds[4] = {dv.x, dv.y, dv.z, dv.w};
      const float cs[4] = {(float)cv.x, (float)cv.y, (float)cv.z, (float)cv.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float diff = round_f16(lod + cs[t] * std_) - ws[t];
        acc += ds[t] * (diff * diff);
      }
    }
    acc = warp_sum(acc);
    __syncthreads();
    if (lane == 0) red[warp] = acc;
    __syncthreads();
    if (tid == 0) {
      float a = 0.0f;
#pragma unroll
      for (int i = 0; i < ROW_THREADS / 32; ++i) a += red[i];
      sse[row] = a;
    }
  }
}

bool block_ok(int block) { return block == 16 || block == 32 || block == 64; }

}  // namespace
}  // namespace hi2

extern "C" int hi2_ladder_grid(const float* wb, const float* db, const float* grid_host, int g,
                               int n, int64_t n_rows, int64_t nb, int block, float* lo,
                               float* step, float* err, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(block_ok(block), "ladder_grid: block must be 16, 32 or 64");
  HI2_REQUIRE(g >= 1 && g <= 8 && grid_host, "ladder_grid: the grid has 1 to 8 points");
  HI2_REQUIRE(n >= 2, "ladder_grid: n must be at least 2");
  if (n_rows == 0 || nb == 0) return HI2_OK;
  HI2_REQUIRE(wb && db && lo && step, "ladder_grid: null pointer");
  HI2_REQUIRE(aligned16(wb), "ladder_grid: wb must be 16-byte aligned");
  return launch_fit(wb, nb * block, db, nullptr, grid_host, g, 0, n, n_rows, nb, block, lo, step, err,
                    static_cast<cudaStream_t>(stream));
}

extern "C" int hi2_fit_ladder_grouped(const float* w, int64_t ldw, const float* d, const int32_t* row_d,
                                      const float* grid_host, int g, int refits, int n, int64_t n_rows,
                                      int64_t k, int block, float* lo, float* step, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(block_ok(block), "fit_ladder: block must be 16, 32 or 64");
  HI2_REQUIRE(k > 0 && k % block == 0, "fit_ladder: k must be a multiple of the block");
  HI2_REQUIRE(g >= 1 && g <= 8 && grid_host, "fit_ladder: the grid has 1 to 8 points");
  HI2_REQUIRE(n >= 2 && refits >= 0, "fit_ladder: bad n or refits");
  if (n_rows == 0) return HI2_OK;
  HI2_REQUIRE(w && d && lo && step, "fit_ladder: null pointer");
  HI2_REQUIRE(aligned16(w) && aligned16(d) && ldw % 4 == 0 && ldw >= k, "fit_ladder: w, d alignment or ldw");
  return launch_fit(w, ldw, d, row_d, grid_host, g, refits, n, n_rows, k / block, block, lo, step,
                    nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int hi2_fit_ladder(const float* w, int64_t ldw, const float* d, const float* grid_host,
                              int g, int refits, int n, int64_t n_rows, int64_t k, int block,
                              float* lo, float* step, void* stream) {
  return hi2_fit_ladder_grouped(w, ldw, d, nullptr, grid_host, g, refits, n, n_rows, k, block, lo, step, stream);
}

extern "C" int hi2_quantize_rows_grouped(const float* lo, const float* step, const float* w, int64_t ldw,
                                         const float* d, const int32_t* row_d, int nbits, int64_t n_rows,
                                         int64_t k, int block, uint8_t* params, uint16_t* consts, float* lo_d,
                                         float* step_d, int64_t ldp, uint8_t* codes, float* sse,
                                         float* energy, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(block_ok(block), "quantize_rows: block must be 16, 32 or 64");
  HI2_REQUIRE(k > 0 && k % block == 0, "quantize_rows: k must be a multiple of the block");
  HI2_REQUIRE(nbits >= 1 && nbits <= 8, "quantize_rows: nbits out of range");
  if (n_rows == 0) return HI2_OK;
  HI2_REQUIRE(lo && step, "quantize_rows: null ladders");
  const bool scan = codes || sse || energy;
  if (scan) {
    HI2_REQUIRE(w && d, "quantize_rows: codes, sse and energy need w and d");
    HI2_REQUIRE(aligned16(w) && aligned16(d) && ldw % 4 == 0 && ldw >= k,
                "quantize_rows: w, d alignment or ldw");
    HI2_REQUIRE(codes == nullptr || (reinterpret_cast<uintptr_t>(codes) & 3u) == 0,
                "quantize_rows: codes must be 4-byte aligned");
  }
  HI2_REQUIRE((lo_d == nullptr && step_d == nullptr) || ldp >= k / block, "quantize_rows: ldp");
  const int64_t nb = k / block;
  const size_t smem = (size_t)ROW_WARPS * (2 * nb) * sizeof(float);
  HI2_REQUIRE(smem <= 200 * 1024, "quantize_rows: k too large for the ladder cache");
  const int64_t want = ceil_div(n_rows, (int64_t)ROW_WARPS);
  const unsigned grid = (unsigned)(want < 148 * 8 ? want : 148 * 8);
  const float nmax = (float)((1 << nbits) - 1);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define HI2_ROW_V(BB, CC, EE)                                                                              \
  do {                                                                                                     \
    if (smem > 48 * 1024 &&                                                                                \
        cudaFuncSetAttribute(row_kernel<BB, CC, EE>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                             (int)smem) != cudaSuccess)                                                    \
      return fail(HI2_ERR_LAUNCH, "quantize_rows: cannot reserve shared memory");                          \
    row_kernel<BB, CC, EE><<<grid, ROW_THREADS, smem, s>>>(lo, step, w, ldw, d, row_d, nmax, n_rows, k,      \
                                                           params, consts, lo_d, step_d, ldp, codes, sse,    \
                                                           energy);                                          \
  } while (0)
#define HI2_ROW(BB)                                     \
  do {                                                  \
    if (codes != nullptr && energy != nullptr) HI2_ROW_V(BB, true, true);   \
    else if (codes != nullptr) HI2_ROW_V(BB, true, false);                  \
    else if (energy != nullptr) HI2_ROW_V(BB, false, true);                 \
    else HI2_ROW_V(BB, false, false);                                       \
  } while (0)
  if (block == 16) HI2_ROW(16);
  if (block == 32) HI2_ROW(32);
  if (block == 64) HI2_ROW(64);
#undef HI2_ROW
#undef HI2_ROW_V
  return check_launch("quantize_rows");
}

extern "C" int hi2_quantize_rows(const float* lo, const float* step, const float* w, int64_t ldw,
                                 const float* d, int nbits, int64_t n_rows, int64_t k, int block,
                                 uint8_t* params, uint16_t* consts, float* lo_d, float* step_d,
                                 int64_t ldp, uint8_t* codes, float* sse, float* energy,
                                 void* stream) {
  return hi2_quantize_rows_grouped(lo, step, w, ldw, d, nullptr, nbits, n_rows, k, block, params, consts, lo_d, step_d,
                                   ldp, codes, sse, energy, stream);
}

extern "C" int hi2_ladder_sse(const uint8_t* codes, const float* w, int64_t ldw, const float* d,
                              const float* lo, const float* st, int64_t ldp, int64_t n_rows,
                              int64_t k, int block, float* sse, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(block_ok(block), "ladder_sse: block must be 16, 32 or 64");
  HI2_REQUIRE(k > 0 && k % block == 0, "ladder_sse: k must be a multiple of the block");
  if (n_rows == 0) return HI2_OK;
  HI2_REQUIRE(codes && w && d && lo && st && sse, "ladder_sse: null pointer");
  HI2_REQUIRE(aligned16(w) && aligned16(d) && ldw % 4 == 0 &&
                  (reinterpret_cast<uintptr_t>(codes) & 3u) == 0,
              "ladder_sse: alignment");
  const unsigned grid = (unsigned)(n_rows < 148 * 16 ? n_rows : 148 * 16);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define HI2_SSE(BB) \
  sse_kernel<BB><<<grid, ROW_THREADS, 0, s>>>(codes, w, ldw, d, lo, st, ldp, n_rows, k, sse)
  if (block == 16) HI2_SSE(16);
  if (block == 32) HI2_SSE(32);
  if (block == 64) HI2_SSE(64);
#undef HI2_SSE
  return check_launch("ladder_sse");
}
