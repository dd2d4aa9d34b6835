// Fixed-ladder GPTQ rounding (hi2/gptq_kernel.py:59-127, hi2/hessian.py:267-315).
//
// Block kernel: one LANE per row (see gptq_block_kernel).  Each product, sum and quotient is
// rounded on its own (the library is built without FMA contraction) and wq is rounded to fp16
// before the error is formed, so given the same inputs the codes equal those of the
// column-by-column loop.
//
// Trailing update: wc[:, i2:] -= err1 @ U[i1:i2, i2:] in fp32 FMA arithmetic (gemm.cuh).
#include "gemm.cuh"

namespace hi2 {

int launch_lazy_tc(float* wc, int64_t n_rows, int64_t k, int64_t i1, const float* err_hi,
                   const float* err_lo, const float* u_hi, const float* u_lo, int* status,
                   cudaStream_t stream);
int launch_split_tf32(const float* x, float* hi, float* lo, int64_t n, cudaStream_t stream);

namespace {

constexpr int LMAX = 128;
constexpr int ROWS_PER_CTA = 64;  // one lane per row; three thread blocks (and staged factor blocks) per SM

// One LANE per row.  The row's segment of up to 128 columns lives in registers as 64 pairs and
// moves down by one pair every two steps, so the columns being rounded are always the first
// pair, every register index is static and two steps are a compact loop body.  The updates use
// a packed fp32 multiply for two columns at a time (see sub_scaled):
// new pair[t] = pair[t+1] - eA * U[j, ..] - eB * U[j+1, ..].  The block
// U[i1:i1+len, i1:i1+len] is staged in shared memory with every row already shifted to the
// column its first pair starts at, where U[j, c] is the same address for every lane (a
// broadcast), and the dependent chain of a column carries no shuffle.  The loop is
// software-pipelined: the error of column j is applied while column j+1 is rounded from the one
// value it needs, and so on, so the chains run inside the updates instead of between them.  The
// live width shrinks in four phases (128, 96, 64, 32 registers) as the columns are used up.
// Rows of one thread block that read different factors (a block that straddles two tensors) are
// served one factor after the other.
constexpr int U_DIAG = LMAX * LMAX;          // diagonal U[j, j] (padded with ones)
constexpr int U_NEXT = U_DIAG + 2 * LMAX;    // U[j, j+1]
constexpr int U_STAGE_FLOATS = U_NEXT + LMAX;

// pair - e * (u0, u1) with the product and the difference rounded separately.  The product is one
// packed multiply; the two additions stay scalar on purpose: a packed multiply feeding a packed
// add is contracted into a packed FMA by the assembler even with contraction switched off, and
// a fused update no longer gives the codes of the reference's separately rounded one.
__device__ __forceinline__ float2 sub_scaled(float2 w, float2 neg_e, float u0, float u1) {
  const float2 p = __fmul2_rn(neg_e, make_float2(u0, u1));
  return make_float2(w.x + p.x, w.y + p.y);
}

struct Ladder {
  float lo, st;
};

// Code and scaled error of one column (hi2/gptq_kernel.py:88-101): exactly the IEEE quotients
// the reference forms.  The fast path (one reciprocal product per division) is computed
// unconditionally and redone with true divisions in the rare unsafe case, so the common path is
// straight-line code.
__device__ __forceinline__ void round_column(float col, Ladder p, float ud, float nm, float& q_out, float& e_out) {
  const float safe = (p.st == 0.0f) ? 1.0f : p.st;
  const Recip rs = make_recip(safe), ru = make_recip(ud);
  const float a = col - p.lo;
  const float t = a * rs.r;
  float q = rintf(t);
  const bool near = fabsf(fabsf(t - q) - 0.5f) < 2.5e-4f && fabsf(t) < 1024.0f;
  if (!rs.fast || !ru.fast || near) {  // rare
    q = rintf(__fdiv_rn(a, safe));
    q = (q < 0.0f) ? 0.0f : q;
    q = (q > nm) ? nm : q;
    if (p.st == 0.0f) q = 0.0f;
    const float wq = round_f16(p.lo + q * p.st);
    q_out = q;
    e_out = __fdiv_rn(col - wq, ud);
    return;
  }
  q = (q < 0.0f) ? 0.0f : q;
  q = (q > nm) ? nm : q;
  if (p.st == 0.0f) q = 0.0f;
  const float wq = round_f16(p.lo + q * p.st);
  const float num = col - wq;
  const float q0 = num * ru.r;
  q_out = q;
  e_out = fmaf(fmaf(-q0, ud, num), ru.r, q0);
}

// Per-row state between steps.  Everything that a load fills is addressed by column modulo 4 with
// the step loop unrolled four times, so a value in flight is never moved: a register copy of it
// would wait for the load and put its latency back on every step.
template <bool WITH_COMP>
struct RowState {
  int j;      // the column whose error is applied next (a multiple of 4 between iterations)
  float e;    // its scaled error
  float ev[4], cv[4];  // outputs of the current quad of columns
  uint32_t qk;
  Ladder p[4];  // ladders of columns j+1 .. j+4
  int b[4];     // block indices of columns j+5 .. j+8
};

// Steps while more than W - 32 columns remain (W registers live: w[0] holds columns s.j, s.j+1).
template <int W, bool WITH_COMP>
__device__ __forceinline__ void run_phase(float2 (&w)[LMAX / 2], RowState<WITH_COMP>& s, int len, float nm,
                                          const float* __restrict__ u_stage, const int32_t* __restrict__ brow,
                                          const float* __restrict__ lorow, const float* __restrict__ strow,
                                          bool live, float* err_row, uint8_t* code_row, float* comp_row) {
  const int last = len - 1;
  constexpr int P = W / 2;  // live pairs
#pragma unroll 1
  while (len - s.j > W - 32 && s.j < len) {
    const int j0 = s.j;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int j = j0 + 2 * h;                      // even: the column whose error is known
      const float* ua = u_stage + j * LMAX;          // ua[t] = U[j, j+2+t]
      const float* ub = ua + LMAX;                   // ub[t] = U[j+1, j+2+t]
      const float ea = s.e;
      // column j+1: one scalar update, then its rounding (overlaps the packed updates below)
      const float cb = w[0].y - ea * u_stage[U_NEXT + j];
      float qb, eb;
      round_column(cb, s.p[(2 * h + 1) & 3], u_stage[U_DIAG + j + 1], nm, qb, eb);
      const float2 na = make_float2(-ea, -ea);
#pragma unroll
      for (int t = 0; t + 1 < P; t += 2) {
        const float4 v = *reinterpret_cast<const float4*>(ua + 2 * t);
        w[t] = sub_scaled(w[t + 1], na, v.x, v.y);
        if (t + 2 < P) w[t + 1] = sub_scaled(w[t + 2], na, v.z, v.w);
      }
      w[P - 1] = make_float2(0.0f, 0.0f);
      // column j+2 (ignored past the last column)
      const float4 fb = *reinterpret_cast<const float4*>(ub);
      const float ca = w[0].x - eb * fb.x;
      float qa, ea2;
      round_column(ca, s.p[(2 * h + 2) & 3], u_stage[U_DIAG + j + 2], nm, qa, ea2);
      const float2 nb = make_float2(-eb, -eb);
      w[0] = sub_scaled(w[0], nb, fb.x, fb.y);
      if (1 < P) w[1] = sub_scaled(w[1], nb, fb.z, fb.w);
#pragma unroll
      for (int t = 2; t < P; t += 2) {
        const float4 v = *reinterpret_cast<const float4*>(ub + 2 * t);
        w[t] = sub_scaled(w[t], nb, v.x, v.y);
        if (t + 1 < P) w[t + 1] = sub_scaled(w[t + 1], nb, v.z, v.w);
      }
      // outputs of columns j+1 and j+2 (slot 3 completes the quad j0 .. j0+3, slot 0 opens the next)
      const int sb = (2 * h + 1) & 3, sa = (2 * h + 2) & 3;
      s.ev[sb] = eb;
      if (WITH_COMP) s.cv[sb] = cb;
      s.qk = (s.qk >> 8) | ((uint32_t)qb << 24);
      if (sb == 3 && live) {
        *reinterpret_cast<float4*>(err_row + j0) = make_float4(s.ev[0], s.ev[1], s.ev[2], s.ev[3]);
        *reinterpret_cast<uint32_t*>(code_row + j0) = s.qk;
        if (WITH_COMP) *reinterpret_cast<float4*>(comp_row + j0) = make_float4(s.cv[0], s.cv[1], s.cv[2], s.cv[3]);
      }
      s.ev[sa] = ea2;
      if (WITH_COMP) s.cv[sa] = ca;
      s.qk = (s.qk >> 8) | ((uint32_t)qa << 24);
      // ladders of columns j+5 and j+6 into the slots just used, block indices of j+9 and j+10 behind them
      s.p[sb].lo = lorow[s.b[sb]], s.p[sb].st = strow[s.b[sb]];
      s.b[sb] = brow[min(j + 9, last)];
      s.p[sa].lo = lorow[s.b[sa]], s.p[sa].st = strow[s.b[sa]];
      s.b[sa] = brow[min(j + 10, last)];
      s.e = ea2;
    }
    s.j = j0 + 4;
  }
}

template <bool WITH_COMP>
__global__ void __launch_bounds__(ROWS_PER_CTA, 3)
gptq_block_kernel(const float* __restrict__ wc, int64_t n_rows, int64_t k, int64_t i1, int len,
                  float* __restrict__ err1, uint8_t* __restrict__ codes,
                  const float* __restrict__ lo, const float* __restrict__ st, int64_t ldp,
                  const int32_t* __restrict__ row_grp, const int64_t* __restrict__ u_ptrs,
                  const int32_t* __restrict__ blk, const float* __restrict__ nmax,
                  float* __restrict__ comp) {
  extern __shared__ float4 u_stage4[];
  float* u_stage = reinterpret_cast<float*>(u_stage4);
  __shared__ unsigned long long next_factor;

  const int64_t row_raw = (int64_t)blockIdx.x * ROWS_PER_CTA + threadIdx.x;
  const bool live = row_raw < n_rows;
  const int64_t row = live ? row_raw : n_rows - 1;  // spare lanes shadow the last row and store nothing
  const int g = row_grp[row];
  const unsigned long long my_factor = (unsigned long long)u_ptrs[g];
  const float nm = nmax[g];
  const float* wrow = wc + row * k + i1;
  const int32_t* brow = blk + (int64_t)g * k + i1;
  const float* lorow = lo + row * ldp;
  const float* strow = st + row * ldp;
  float* err_row = err1 + row * len;
  uint8_t* code_row = codes + row * k + i1;
  float* comp_row = WITH_COMP ? comp + row * k + i1 : nullptr;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  const int last = len - 1;

  bool done = false;
  while (true) {
    if (threadIdx.x == 0) next_factor = ~0ull;
    __syncthreads();
    if (!done) atomicMin(&next_factor, my_factor);
    __syncthreads();
    const unsigned long long factor = next_factor;
    if (factor == ~0ull) break;
    {
      // u_stage[j][t] = U[i1+j, i1+first(j)+t] with first(j) = j+2 for even j and j+1 for odd j (zero
      // past the segment); then the diagonal and U[j, j+1]
      const float* src = reinterpret_cast<const float*>(factor) + i1 * k + i1;
      for (int idx = threadIdx.x; idx < LMAX * LMAX / 4; idx += ROWS_PER_CTA)
        u_stage4[idx] = zero4;
      __syncthreads();
      const int quads = len / 4;
      for (int idx = threadIdx.x; idx < len * quads; idx += ROWS_PER_CTA) {
        const int j = idx / quads, c = (idx % quads) * 4;
        const int first = j + 2 - (j & 1);
        if (c + 3 < first) continue;
        const float4 v = *reinterpret_cast<const float4*>(src + j * k + c);
        float* dst = u_stage + j * LMAX + (c - first);
        if (c >= first) dst[0] = v.x;
        if (c + 1 >= first) dst[1] = v.y;
        if (c + 2 >= first) dst[2] = v.z;
        dst[3] = v.w;
      }
      for (int idx = threadIdx.x; idx < 2 * LMAX; idx += ROWS_PER_CTA)
        u_stage[U_DIAG + idx] = idx < len ? src[idx * k + idx] : 1.0f;
      for (int idx = threadIdx.x; idx < LMAX; idx += ROWS_PER_CTA)
        u_stage[U_NEXT + idx] = idx + 1 < len ? src[idx * k + idx + 1] : 0.0f;
    }
    __syncthreads();
    if (!done && my_factor == factor) {
      done = true;
      float2 w[LMAX / 2];
#pragma unroll
      for (int q = 0; q < LMAX / 4; ++q) {
        const float4 v = (4 * q < len) ? *reinterpret_cast<const float4*>(wrow + 4 * q) : zero4;
        w[2 * q] = make_float2(v.x, v.y), w[2 * q + 1] = make_float2(v.z, v.w);
      }
      RowState<WITH_COMP> s;
      s.j = 0, s.qk = 0;
      auto ladder = [&](int c) {
        const int b = brow[min(c, last)];
        Ladder p;
        p.lo = lorow[b], p.st = strow[b];
        return p;
      };
#pragma unroll
      for (int c = 1; c <= 4; ++c) s.p[c & 3] = ladder(c), s.b[c & 3] = brow[min(c + 4, last)];
      {  // column 0 opens the pipeline
        float q0, e0;
        round_column(w[0].x, ladder(0), u_stage[U_DIAG], nm, q0, e0);
        s.ev[0] = e0, s.ev[1] = s.ev[2] = s.ev[3] = 0.0f;
        s.cv[0] = w[0].x, s.cv[1] = s.cv[2] = s.cv[3] = 0.0f;
        s.qk = (uint32_t)q0 << 24;
        s.e = e0;
      }
      run_phase<128, WITH_COMP>(w, s, len, nm, u_stage, brow, lorow, strow, live, err_row, code_row, comp_row);
      run_phase<96, WITH_COMP>(w, s, len, nm, u_stage, brow, lorow, strow, live, err_row, code_row, comp_row);
      run_phase<64, WITH_COMP>(w, s, len, nm, u_stage, brow, lorow, strow, live, err_row, code_row, comp_row);
      run_phase<32, WITH_COMP>(w, s, len, nm, u_stage, brow, lorow, strow, live, err_row, code_row, comp_row);
    }
    __syncthreads();  // the staged block is replaced in the next round
  }
}

int launch_block(const float* wc, int64_t n_rows, int64_t k, int64_t i1, int len, float* err1,
                 uint8_t* codes, const float* lo, const float* st, int64_t ldp,
                 const int32_t* row_grp, const int64_t* u_ptrs, const int32_t* blk,
                 const float* nmax, float* comp, cudaStream_t stream) {
  const unsigned grid = (unsigned)ceil_div(n_rows, ROWS_PER_CTA);
  const int smem = U_STAGE_FLOATS * (int)sizeof(float);
  if (cudaFuncSetAttribute(gptq_block_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
      cudaFuncSetAttribute(gptq_block_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return fail(HI2_ERR_LAUNCH, "gptq_block: cannot reserve shared memory");
  if (comp != nullptr)
    gptq_block_kernel<true><<<grid, ROWS_PER_CTA, smem, stream>>>(wc, n_rows, k, i1, len, err1, codes, lo, st,
                                                               ldp, row_grp, u_ptrs, blk, nmax, comp);
  else
    gptq_block_kernel<false><<<grid, ROWS_PER_CTA, smem, stream>>>(wc, n_rows, k, i1, len, err1, codes, lo, st,
                                                                ldp, row_grp, u_ptrs, blk, nmax, comp);
  return check_launch("gptq_block");
}

int launch_lazy(float* wc, int64_t n_rows, int64_t k, int64_t i1, int64_t i2, const float* err1,
                const float* u, cudaStream_t stream) {
  GemmArgs<float, float, float> p;
  p.m = n_rows, p.n = k - i2, p.kk = i2 - i1;
  p.alpha = -1.0f, p.beta = 1.0f;
  p.a = err1, p.lda = i2 - i1;
  p.b = u + i1 * k + i2, p.ldb = k;
  p.c = wc + i2, p.ldc = k;
  p.flags = 0;
  return launch_gemm_async<float, 8, 8, 16>(false, false, p, stream, "gptq_lazy_update");
}

int check_block_args(const float* wc, int64_t n_rows, int64_t k, int64_t i1, int len,
                     const float* err1, const uint8_t* codes, const float* lo, const float* st,
                     int64_t ldp, const int32_t* row_grp, const int64_t* u_ptrs, const int32_t* blk,
                     const float* nmax, const float* comp) {
  HI2_REQUIRE(k > 0 && k % 16 == 0, "gptq_block: k must be a positive multiple of 16");
  HI2_REQUIRE(len > 0 && len <= LMAX && len % 16 == 0, "gptq_block: block length must be 16..128");
  HI2_REQUIRE(i1 >= 0 && i1 % 16 == 0 && i1 + len <= k, "gptq_block: block outside the row");
  HI2_REQUIRE(wc && err1 && codes && lo && st && row_grp && u_ptrs && blk && nmax,
              "gptq_block: null pointer");
  HI2_REQUIRE(aligned16(wc) && aligned16(err1) && aligned16(blk) && (comp == nullptr || aligned16(comp)),
              "gptq_block: wc, err1, blk and comp must be 16-byte aligned");
  HI2_REQUIRE((reinterpret_cast<uintptr_t>(codes) & 3u) == 0, "gptq_block: codes must be 4-byte aligned");
  HI2_REQUIRE(ldp > 0, "gptq_block: ldp");
  (void)n_rows;
  return HI2_OK;
}

}  // namespace
}  // namespace hi2

extern "C" int hi2_gptq_block(const float* wc, int64_t n_rows, int64_t k, int64_t i1, int len,
                              float* err1, uint8_t* codes, const float* lo, const float* st,
                              int64_t ldp, const int32_t* row_grp, const int64_t* u_ptrs,
                              const int32_t* blk, const float* nmax, float* comp, void* stream) {
  using namespace hi2;
  if (n_rows == 0) return HI2_OK;
  int rc = check_block_args(wc, n_rows, k, i1, len, err1, codes, lo, st, ldp, row_grp, u_ptrs, blk,
                            nmax, comp);
  if (rc != HI2_OK) return rc;
  return launch_block(wc, n_rows, k, i1, len, err1, codes, lo, st, ldp, row_grp, u_ptrs, blk, nmax,
                      comp, static_cast<cudaStream_t>(stream));
}

extern "C" int hi2_gptq_lazy_update(float* wc, int64_t n_rows, int64_t k, int64_t i1, int64_t i2,
                                    const float* err1, const float* u, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(k > 0 && 0 <= i1 && i1 < i2 && i2 <= k, "gptq_lazy_update: bad block range");
  if (n_rows == 0 || i2 == k) return HI2_OK;
  HI2_REQUIRE(wc && err1 && u, "gptq_lazy_update: null pointer");
  return launch_lazy(wc, n_rows, k, i1, i2, err1, u, static_cast<cudaStream_t>(stream));
}

extern "C" int hi2_gptq_round(float* wc, int64_t n_rows, int64_t k, float* err1, uint8_t* codes,
                              const float* lo, const float* st, int64_t ldp,
                              const int32_t* row_grp, const int64_t* u_ptrs, const int32_t* blk,
                              const float* nmax, float* comp, int n_units,
                              const int64_t* unit_rows_host, const int64_t* u_host, void* stream) {
  using namespace hi2;
  if (n_rows == 0) return HI2_OK;
  HI2_REQUIRE(n_units >= 1 && unit_rows_host && u_host, "gptq_round: unit table missing");
  HI2_REQUIRE(unit_rows_host[0] == 0 && unit_rows_host[n_units] == n_rows,
              "gptq_round: units must cover the rows");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  ChainGraph chain(s);  // the K/128 segments and their trailing updates as one graph launch
  auto enqueue = [&]() -> int {
    for (int64_t i1 = 0; i1 < k; i1 += LMAX) {
      const int64_t i2 = (i1 + LMAX < k) ? i1 + LMAX : k;
      const int len = (int)(i2 - i1);
      int rc = check_block_args(wc, n_rows, k, i1, len, err1, codes, lo, st, ldp, row_grp, u_ptrs,
                                blk, nmax, comp);
      if (rc != HI2_OK) return rc;
      rc = launch_block(wc, n_rows, k, i1, len, err1, codes, lo, st, ldp, row_grp, u_ptrs, blk, nmax,
                        comp, s);
      if (rc != HI2_OK) return rc;
      if (i2 == k) break;
      for (int un = 0; un < n_units; ++un) {
        const int64_t r0 = unit_rows_host[un], r1 = unit_rows_host[un + 1];
        if (r1 <= r0) continue;
        rc = launch_lazy(wc + r0 * k, r1 - r0, k, i1, i2, err1 + r0 * len,
                         reinterpret_cast<const float*>(u_host[un]), s);
        if (rc != HI2_OK) return rc;
      }
    }
    return HI2_OK;
  };
  return chain.finish(enqueue(), "gptq_round");
}

extern "C" int hi2_gptq_lazy_update_tc(float* wc, int64_t n_rows, int64_t k, int64_t i1,
                                       const float* err_split, const float* u_split, int32_t* status,
                                       void* stream) {
  using namespace hi2;
  HI2_REQUIRE(k > 0 && k % 4 == 0 && i1 >= 0 && i1 % 4 == 0 && i1 + LMAX <= k,
              "gptq_lazy_update_tc: bad block range");
  if (n_rows == 0 || i1 + LMAX == k) return HI2_OK;
  HI2_REQUIRE(wc && err_split && u_split && status, "gptq_lazy_update_tc: null pointer");
  HI2_REQUIRE(aligned16(wc) && aligned16(err_split) && aligned16(u_split), "gptq_lazy_update_tc: alignment");
  return launch_lazy_tc(wc, n_rows, k, i1, err_split, err_split + n_rows * LMAX, u_split, u_split + k * k,
                        reinterpret_cast<int*>(status), static_cast<cudaStream_t>(stream));
}

extern "C" int hi2_gptq_round_tc(float* wc, int64_t n_rows, int64_t k, float* err1, float* err_split,
                                 uint8_t* codes, const float* lo, const float* st, int64_t ldp,
                                 const int32_t* row_grp, const int64_t* u_ptrs, const int32_t* blk,
                                 const float* nmax, float* comp, int n_units,
                                 const int64_t* unit_rows_host, const int64_t* u_split_host,
                                 int32_t* status, void* stream) {
  using namespace hi2;
  if (n_rows == 0) return HI2_OK;
  HI2_REQUIRE(n_units >= 1 && unit_rows_host && u_split_host, "gptq_round_tc: unit table missing");
  HI2_REQUIRE(unit_rows_host[0] == 0 && unit_rows_host[n_units] == n_rows,
              "gptq_round_tc: units must cover the rows");
  HI2_REQUIRE(err_split && status && aligned16(err_split), "gptq_round_tc: scratch missing or unaligned");
  HI2_REQUIRE(k % 4 == 0, "gptq_round_tc: k must be a multiple of 4");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* err_hi = err_split;
  float* err_lo = err_split + n_rows * LMAX;
  ChainGraph chain(s);  // the K/128 segments and their trailing updates as one graph launch
  auto enqueue = [&]() -> int {
    if (cudaMemsetAsync(status, 0, sizeof(int32_t), s) != cudaSuccess)
      return fail(HI2_ERR_LAUNCH, "gptq_round_tc: memset failed");
    for (int64_t i1 = 0; i1 < k; i1 += LMAX) {
      const int64_t i2 = (i1 + LMAX < k) ? i1 + LMAX : k;
      const int len = (int)(i2 - i1);
      int rc = check_block_args(wc, n_rows, k, i1, len, err1, codes, lo, st, ldp, row_grp, u_ptrs,
                                blk, nmax, comp);
      if (rc != HI2_OK) return rc;
      rc = launch_block(wc, n_rows, k, i1, len, err1, codes, lo, st, ldp, row_grp, u_ptrs, blk, nmax,
                        comp, s);
      if (rc != HI2_OK) return rc;
      if (i2 == k) break;  // a block shorter than 128 columns is always the last one
      rc = launch_split_tf32(err1, err_hi, err_lo, n_rows * LMAX, s);
      if (rc != HI2_OK) return rc;
      for (int un = 0; un < n_units; ++un) {
        const int64_t r0 = unit_rows_host[un], r1 = unit_rows_host[un + 1];
        if (r1 <= r0) continue;
        const float* u_hi = reinterpret_cast<const float*>(u_split_host[un]);
        rc = launch_lazy_tc(wc + r0 * k, r1 - r0, k, i1, err_hi + r0 * LMAX, err_lo + r0 * LMAX, u_hi,
                            u_hi + k * k, reinterpret_cast<int*>(status), s);
        if (rc != HI2_OK) return rc;
      }
    }
    return HI2_OK;
  };
  return chain.finish(enqueue(), "gptq_round_tc");
}

extern "C" int hi2_gemm_f32(int trans_a, int trans_b, int64_t m, int64_t n, int64_t kk, float alpha,
                            const float* a, int64_t lda, const float* b, int64_t ldb, float beta,
                            float* c, int64_t ldc, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(m >= 0 && n >= 0 && kk >= 0, "gemm_f32: negative size");
  if (m == 0 || n == 0) return HI2_OK;
  HI2_REQUIRE(c && (kk == 0 || (a && b)), "gemm_f32: null pointer");
  GemmArgs<float, float, float> p;
  p.m = m, p.n = n, p.kk = kk, p.alpha = alpha, p.beta = beta;
  p.a = a, p.lda = lda, p.b = b, p.ldb = ldb, p.c = c, p.ldc = ldc, p.flags = 0;
  return launch_gemm_async<float, 8, 8, 16>(trans_a != 0, trans_b != 0, p,
                                            static_cast<cudaStream_t>(stream), "gemm_f32");
}
