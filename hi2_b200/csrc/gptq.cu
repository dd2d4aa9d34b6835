// Fixed-ladder GPTQ rounding (hi2/gptq_kernel.py:59-127, hi2/hessian.py:267-315).
//
// Block kernel: one WARP per row.  A lane keeps four consecutive columns of the row's 128-column
// segment in registers together with their ladder (lo, step).  Column i is rounded by the lane
// that owns it; its scaled error reaches the other lanes with one shuffle and every lane
// subtracts e * U[j, c] from its columns c > i.  Rows of U are read as one 128-bit load per lane
// (a contiguous 512-byte line per warp, served from L1/L2 since every warp of the same factor
// walks the same rows) and fetched two rows ahead of their use, so the dependent chain per
// column is shuffle + ~10 arithmetic instructions.  Each product, sum and quotient is rounded
// on its own (the library is built without FMA contraction) and wq is rounded to fp16 before the
// error is formed, so given the same inputs the codes equal those of the column-by-column loop.
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
constexpr int ROWS_PER_CTA = 8;

template <bool WITH_COMP>
__global__ void __launch_bounds__(ROWS_PER_CTA * 32, 3)
gptq_block_kernel(const float* __restrict__ wc, int64_t n_rows, int64_t k, int64_t i1, int len,
                  float* __restrict__ err1, uint8_t* __restrict__ codes,
                  const float* __restrict__ lo, const float* __restrict__ st, int64_t ldp,
                  const int32_t* __restrict__ row_grp, const int64_t* __restrict__ u_ptrs,
                  const int32_t* __restrict__ blk, const float* __restrict__ nmax,
                  float* __restrict__ comp) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * ROWS_PER_CTA + (threadIdx.x >> 5);
  if (row >= n_rows) return;  // whole warp
  const int c0 = lane * 4;
  const bool mine = c0 < len;  // len is a multiple of 16: a quad is entirely inside or outside
  const int g = row_grp[row];
  const float* __restrict__ u = reinterpret_cast<const float*>(u_ptrs[g]);
  const float nm = nmax[g];

  float w[4] = {0.f, 0.f, 0.f, 0.f}, lo_c[4] = {0.f, 0.f, 0.f, 0.f}, st_c[4] = {0.f, 0.f, 0.f, 0.f};
  if (mine) {
    const float4 v = *reinterpret_cast<const float4*>(wc + row * k + i1 + c0);
    w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
    const int4 b = *reinterpret_cast<const int4*>(blk + (int64_t)g * k + i1 + c0);
    const int bs[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int s = 0; s < 4; ++s) lo_c[s] = lo[row * ldp + bs[s]], st_c[s] = st[row * ldp + bs[s]];
  }
  float q_keep[4] = {0.f, 0.f, 0.f, 0.f}, e_keep[4] = {0.f, 0.f, 0.f, 0.f},
        col_keep[4] = {0.f, 0.f, 0.f, 0.f};
  // Reciprocals of the two divisors of a column, taken off the dependent chain: the ladder
  // step of the column's block and the diagonal entry of U.  rint_div / div_by give exactly the
  // IEEE quotients the reference forms.
  Recip rc_st[4], rc_u[4];
  float udiag[4];
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const int64_t j = i1 + c0 + s;
    udiag[s] = mine ? u[j * k + j] : 1.0f;
    rc_u[s] = make_recip(udiag[s]);
    rc_st[s] = make_recip((st_c[s] == 0.0f) ? 1.0f : st_c[s]);
  }

  // rows i1 .. i1+len-1 of U, this lane's four columns, held two rows ahead of their use in a
  // ring of four registers-quads: rows i, i+1 are in ring[0..1] when a group of four steps starts,
  // rows i+2, i+3 are requested then, and the first two rows of the next group as soon as steps
  // 0 and 1 have consumed theirs
  const float* urow = u + i1 * k + i1 + c0;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  auto fetch = [&](int r) {
    return (mine && r < len) ? *reinterpret_cast<const float4*>(urow + (int64_t)r * k) : zero4;
  };
  float4 ring[4];
  ring[0] = fetch(0), ring[1] = fetch(1);

  for (int i = 0; i < len; i += 4) {
    ring[2] = fetch(i + 2), ring[3] = fetch(i + 3);
    const int owner = i >> 2;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const float us[4] = {ring[s].x, ring[s].y, ring[s].z, ring[s].w};
      if (s == 2) ring[0] = fetch(i + 4), ring[1] = fetch(i + 5);
      // every lane evaluates slot s of its own quad; only the owner's result is used
      const float col = w[s], lo_j = lo_c[s], st_j = st_c[s];
      const float safe = (st_j == 0.0f) ? 1.0f : st_j;
      float q = rint_div(col - lo_j, safe, rc_st[s]);
      q = (q < 0.0f) ? 0.0f : q;
      q = (q > nm) ? nm : q;
      if (st_j == 0.0f) q = 0.0f;
      const float wq = round_f16(lo_j + q * st_j);
      const float e_own = div_by(col - wq, udiag[s], rc_u[s]);
      const float e = __shfl_sync(0xffffffffu, e_own, owner);
      if (lane == owner) {
        q_keep[s] = q, e_keep[s] = e_own;
        if (WITH_COMP) col_keep[s] = col;
      }
      // all four columns, as the reference updates w1[:, i:]: columns up to this one are never
      // read again (and U is upper triangular, so their factor entries are zero anyway)
#pragma unroll
      for (int t = 0; t < 4; ++t) w[t] = w[t] - e * us[t];
    }
  }

  if (mine) {
    *reinterpret_cast<float4*>(err1 + row * len + c0) =
        make_float4(e_keep[0], e_keep[1], e_keep[2], e_keep[3]);
    *reinterpret_cast<uchar4*>(codes + row * k + i1 + c0) =
        make_uchar4((uint8_t)q_keep[0], (uint8_t)q_keep[1], (uint8_t)q_keep[2], (uint8_t)q_keep[3]);
    if (WITH_COMP)
      *reinterpret_cast<float4*>(comp + row * k + i1 + c0) =
          make_float4(col_keep[0], col_keep[1], col_keep[2], col_keep[3]);
  }
}

int launch_block(const float* wc, int64_t n_rows, int64_t k, int64_t i1, int len, float* err1,
                 uint8_t* codes, const float* lo, const float* st, int64_t ldp,
                 const int32_t* row_grp, const int64_t* u_ptrs, const int32_t* blk,
                 const float* nmax, float* comp, cudaStream_t stream) {
  const unsigned grid = (unsigned)ceil_div(n_rows, ROWS_PER_CTA);
  if (comp != nullptr)
    gptq_block_kernel<true><<<grid, ROWS_PER_CTA * 32, 0, stream>>>(wc, n_rows, k, i1, len, err1, codes,
                                                                    lo, st, ldp, row_grp, u_ptrs, blk,
                                                                    nmax, comp);
  else
    gptq_block_kernel<false><<<grid, ROWS_PER_CTA * 32, 0, stream>>>(wc, n_rows, k, i1, len, err1, codes,
                                                                     lo, st, ldp, row_grp, u_ptrs, blk,
                                                                     nmax, comp);
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
  if (cudaMemsetAsync(status, 0, sizeof(int32_t), s) != cudaSuccess)
    return fail(HI2_ERR_LAUNCH, "gptq_round_tc: memset failed");
  float* err_hi = err_split;
  float* err_lo = err_split + n_rows * LMAX;
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
