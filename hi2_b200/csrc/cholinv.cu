// Damped inverse factor (hi2/hessian.py:71-86): the upper-triangular U with
// U^T U = (hs + lam I)^-1.
//
// The reference factorises, inverts and factorises again.  The same U has a closed form: with J
// the index reversal, J (hs + lam I) J = L L^T (L lower) gives U = J L^-1 J.  So one Cholesky
// factorisation and one triangular inverse suffice, and both come out of one recursion on the
// reversed matrix A (fp32, lower part):
//
//   F(A):  split A = [A11 . ; A21 A22]
//          (X11) = F(A11)                      X11 = L11^-1
//          W     = A21 X11^T                   (= L21)
//          A22  -= W W^T
//          T     = W X11
//          (X22) = F(A22)
//          X21   = -X22 T
//
// Every step above the 64-wide leaves is a matrix product (gemm.cuh, fp32 FMA, triangular
// operands expressed as k-ranges); a leaf factorises and inverts one 64x64 block in shared
// memory in fp64.  W is kept in the X21 slot and T in the A21 slot, so the scratch is 2 K^2 floats.
// Precision: the reference's own path is fp32 LAPACK; measured against an fp64 solution on
// calibration-like Hessians (K = 1024..2048, condition 3e3..8e4) this recursion with fp32
// products is as close to the truth as the reference is (1.0e-5 vs 1.5e-5 of max|U| at condition
// 5e3, 3e-4 vs 1.4e-3 at 8e4), and fp64 products would not bring it closer to the REFERENCE,
// whose own rounding dominates the difference either way.  A non-positive pivot does not trap:
// the leaf records its index in *info, carries on with a unit pivot, and the host retries with
// more damping.
#include "gemm.cuh"

namespace hi2 {
// lazy_tc.cu
int launch_gemm_tc(int64_t m, int64_t n, int64_t kk, const float* a_hi, const float* a_lo, const float* b_hi,
                   const float* b_lo, int64_t ldk, float* c, int64_t ldc, int flags, int* status,
                   cudaStream_t stream);
int launch_split_block(const float* x, int64_t ldx, int64_t rows, int64_t cols, float* hi, float* lo,
                       int64_t ldo, bool transposed, cudaStream_t stream);
namespace {

constexpr int NB = 64;
constexpr int LDL = NB + 1;
constexpr size_t LEAF_SMEM = 2 * NB * LDL * sizeof(double);

// A[i][j] = hs[k-1-i][k-1-j] (+ lam on the diagonal, added in fp32 as the reference does).
__global__ void __launch_bounds__(256)
reverse_damp_kernel(const float* __restrict__ hs, const float* __restrict__ lam, int64_t k,
                    float* __restrict__ a) {
  const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (idx >= k * k) return;
  const int64_t i = idx / k, j = idx % k;
  float v = hs[(k - 1 - i) * k + (k - 1 - j)];
  if (i == j) v = v + *lam;
  a[idx] = v;
}

// u[i][j] = x[k-1-i][k-1-j]
__global__ void __launch_bounds__(256)
reverse_store_kernel(const float* __restrict__ x, int64_t k, float* __restrict__ u) {
  const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (idx >= k * k) return;
  const int64_t i = idx / k, j = idx % k;
  u[idx] = x[(k - 1 - i) * k + (k - 1 - j)];
}

// 1 / sqrt(v) in fp64 from the fp32 estimate and three Newton steps (the fp64 square root and
// division are ~60-instruction sequences on the critical path of every column of a leaf; this
// is ~15).  Outside fp32's normal range the plain expression is used.
__device__ __forceinline__ double inv_sqrt(double v) {
  if (!(v > 1e-30 && v < 1e30)) return 1.0 / sqrt(v);
  double y = (double)rsqrtf((float)v);
  const double h = 0.5 * v;
#pragma unroll
  for (int it = 0; it < 3; ++it) y = fma(y, fma(-h * y, y, 0.5), y);  // y += y * (0.5 - h y^2)
  return y;
}

// 1 / v in fp64 from the fp32 estimate and three Newton steps.
__device__ __forceinline__ double recip(double v) {
  if (!(v > 1e-30 && v < 1e30)) return 1.0 / v;
  double y = (double)__frcp_rn((float)v);
#pragma unroll
  for (int it = 0; it < 3; ++it) y = fma(y, fma(-v, y, 1.0), y);  // y += y * (1 - v y)
  return y;
}

// Factorise the n x n (n <= 64) diagonal block at `off` (lower part of a, leading dim ld) and
// write its inverse, zeros above the diagonal included, to the same place of x (fp32 in memory,
// fp64 inside the block).  One thread block of 256 threads.
//
// Factorisation: right-looking with UNSCALED columns, so a column costs one barrier: after step j
// the entries below the diagonal of column j hold the Schur-updated a_ij and the true factor is
// l_ij = a_ij / sqrt(p_j) with p_j the updated pivot; the trailing update needs only
// a_ij a_cj / p_j.  The 64 square roots are taken side by side after the loop.
//
// Inverse: column c of X = L^-1 belongs to four adjacent lanes, lane `part` keeping
// X[c + part + 4 r][c], r = 0..15, in registers.  Row i = c + d of the column is
// -(sum_{q < i} L[i][q] X[q][c]) / L[i][i]; the loop over d is unrolled so every register index
// is static, the four partial sums meet by shuffle, and no barrier is needed at all.
__global__ void __launch_bounds__(256)
leaf_kernel(const float* __restrict__ a, float* __restrict__ x, int64_t ld, int64_t off, int n,
            int32_t* info) {
  extern __shared__ double leaf_smem[];
  double (*L)[LDL] = reinterpret_cast<double (*)[LDL]>(leaf_smem);
  double (*X)[LDL] = reinterpret_cast<double (*)[LDL]>(leaf_smem + NB * LDL);
  __shared__ double pivot[NB];
  __shared__ double inv_diag[NB];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const float* src = a + off * ld + off;
  for (int idx = tid; idx < NB * NB; idx += 256) {
    const int i = idx >> 6, j = idx & 63;
    L[i][j] = (i < n && j <= i) ? (double)src[(int64_t)i * ld + j] : 0.0;
    X[i][j] = 0.0;
  }
  if (tid < NB) pivot[tid] = 1.0;
  __syncthreads();
  for (int j = 0; j < n; ++j) {
    double piv = L[j][j];  // final: every update of (j, j) was followed by a barrier
    if (!(piv > 0.0)) {    // also catches NaN
      if (tid == 0) atomicCAS(info, 0, (int32_t)(off + j + 1));
      piv = 1.0;
    }
    if (tid == 0) pivot[j] = piv;
    const double rp = recip(piv);
    for (int i = j + 1 + ty; i < n; i += 16) {
      const double lij = L[i][j] * rp;
      for (int c = j + 1 + tx; c <= i; c += 16) L[i][c] = fma(-lij, L[c][j], L[i][c]);
    }
    __syncthreads();
  }
  if (tid < NB) inv_diag[tid] = tid < n ? inv_sqrt(pivot[tid]) : 0.0;
  __syncthreads();
  for (int idx = tid; idx < NB * NB; idx += 256) {  // the true factor below the diagonal
    const int i = idx >> 6, j = idx & 63;
    if (j < i) L[i][j] *= inv_diag[j];
  }
  __syncthreads();

  const int c = tid >> 2, part = tid & 3;
  double xr[16];
#pragma unroll
  for (int r = 0; r < 16; ++r) xr[r] = 0.0;
  if (part == 0) xr[0] = inv_diag[c];
#pragma unroll
  for (int d = 1; d < NB; ++d) {
    const int i = c + d;  // rows past the block read the zero padding of L and stay zero
    double acc0 = 0.0, acc1 = 0.0;
    if (i < NB) {
#pragma unroll
      for (int r = 0; r <= (d >> 2); ++r) {
        // q = c + part + 4 r < i  <=>  part + 4 r < d
        if (4 * r + 3 < d || part + 4 * r < d) {
          const double l = L[i][c + part + 4 * r];
          if (r & 1) acc1 = fma(l, xr[r], acc1);
          else acc0 = fma(l, xr[r], acc0);
        }
      }
    }
    double acc = acc0 + acc1;
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    if (part == (d & 3)) xr[d >> 2] = (i < NB) ? -acc * inv_diag[i] : 0.0;
  }
#pragma unroll
  for (int r = 0; r < 16; ++r) {
    const int i = c + part + 4 * r;
    if (i < NB) X[i][c] = xr[r];
  }
  __syncthreads();
  float* dst = x + off * ld + off;
  for (int idx = tid; idx < n * n; idx += 256) {
    const int i = idx / n, j = idx % n;
    dst[(int64_t)i * ld + j] = (float)X[i][j];
  }
}

struct Plan {
  float* a;
  float* x;
  float* split;  // TF32 parts of the operands of one tensor-core product (4 n1^2 floats)
  int* status;   // raised by a tensor-core product whose bounded wait ran out
  int64_t k;
  int32_t* info;
  cudaStream_t stream;
};

constexpr int GT_KB_LE_J = 1, GT_KB_GE_J = 2, GT_KA_LE_I = 4, GT_LOWER_OUT = 8, GT_NEGATE = 16, GT_ADD = 32;

// Products at least this large on both output sides go to the tensor cores (3xTF32, fp32-grade);
// below it a 128 x 256 tile grid no longer fills the SMs and the FMA kernel is as fast.
#ifndef HI2_FACTOR_TC_MIN
#define HI2_FACTOR_TC_MIN 1024
#endif

int64_t top_half(int64_t n) { return ((ceil_div(n, (int64_t)64) + 1) / 2) * 64; }
size_t split_floats(int64_t k) {
  const int64_t n1 = top_half(k);
  return k >= 2 * HI2_FACTOR_TC_MIN ? (size_t)(4 * n1 * n1) : 0;
}
__global__ void merge_status_kernel(const int* status, int32_t* info) {
  if (*status != 0) *info = -1;
}

// Longest fp32 accumulation chain of a product of the recursion.  Sums longer than this are formed
// window by window and the windows added (two-level summation): the recursion cancels heavily on
// the rank-deficient, damped Hessians of short calibration sets (condition 1e5), and a chain of
// thousands of sequential fp32 adds costs a decimal digit of U there (measured on a 4096-wide
// input with 2048 tokens: error against an fp64 solution 6e-5 of max|U| with one chain per dot
// product, against 9e-6 for the reference's LAPACK path).
constexpr int64_t SUM_WINDOW = 256;

int product(bool trans_b, int64_t m, int64_t n, int64_t kk, float alpha, const float* a,
            const float* b, float beta, float* c, int64_t ld, int flags, cudaStream_t stream) {
  GemmArgs<float, float, float> p;
  p.m = m, p.n = n, p.kk = kk, p.alpha = alpha, p.beta = beta;
  p.a = a, p.lda = ld, p.b = b, p.ldb = ld, p.c = c, p.ldc = ld, p.flags = flags;
  for (int64_t k0 = 0; k0 < kk || k0 == 0; k0 += SUM_WINDOW) {
    p.k_begin = k0, p.k_end = k0 + SUM_WINDOW;
    int rc = launch_gemm_async<float, 8, 8, 16>(false, trans_b, p, stream, "inverse_factor");
    if (rc != HI2_OK) return rc;
    p.beta = 1.0f;
  }
  return HI2_OK;
}

int factor(const Plan& pl, int64_t off, int64_t n) {
  const int64_t ld = pl.k;
  if (n <= NB) {
    leaf_kernel<<<1, 256, LEAF_SMEM, pl.stream>>>(pl.a, pl.x, ld, off, (int)n, pl.info);
    return check_launch("inverse_factor leaf");
  }
  const int64_t blocks = ceil_div(n, NB);
  const int64_t n1 = ((blocks + 1) / 2) * NB, n2 = n - n1;
  int rc = factor(pl, off, n1);
  if (rc != HI2_OK) return rc;
  float* a21 = pl.a + (off + n1) * ld + off;
  float* a22 = pl.a + (off + n1) * ld + off + n1;
  float* x11 = pl.x + off * ld + off;
  float* x21 = pl.x + (off + n1) * ld + off;
  float* x22 = pl.x + (off + n1) * ld + off + n1;
  if (n2 >= HI2_FACTOR_TC_MIN && pl.split != nullptr) {
    // Tensor-core path.  Operands are split into TF32 parts first (K-major; the right-hand
    // operands of T = W X11 and X21 = -X22 T are split transposed).  n1 >= n2 and n1 is a multiple
    // of 64, so four parts of n1 x n1 floats hold any pair of operands of this level; deeper
    // levels reuse the same scratch once this level's product has consumed it (one stream).
    const int64_t part = n1 * n1;
    float *ah = pl.split, *al = ah + part, *bh = al + part, *bl = bh + part;
    const int64_t l1 = n1, l2 = ceil_div(n2, (int64_t)32) * 32;  // leading dimensions for kk = n1, n2
    // W (in the X21 slot) = A21 X11^T
    if ((rc = launch_split_block(a21, ld, n2, n1, ah, al, l1, false, pl.stream)) != HI2_OK) return rc;
    if ((rc = launch_split_block(x11, ld, n1, n1, bh, bl, l1, false, pl.stream)) != HI2_OK) return rc;
    rc = launch_gemm_tc(n2, n1, n1, ah, al, bh, bl, l1, x21, ld, GT_KB_LE_J, pl.status, pl.stream);
    if (rc != HI2_OK) return rc;
    // A22 -= W W^T (lower tiles)
    if ((rc = launch_split_block(x21, ld, n2, n1, ah, al, l1, false, pl.stream)) != HI2_OK) return rc;
    rc = launch_gemm_tc(n2, n2, n1, ah, al, ah, al, l1, a22, ld, GT_LOWER_OUT | GT_NEGATE | GT_ADD, pl.status,
                        pl.stream);
    if (rc != HI2_OK) return rc;
    // T (in the A21 slot) = W X11
    if ((rc = launch_split_block(x11, ld, n1, n1, bh, bl, l1, true, pl.stream)) != HI2_OK) return rc;
    rc = launch_gemm_tc(n2, n1, n1, ah, al, bh, bl, l1, a21, ld, GT_KB_GE_J, pl.status, pl.stream);
    if (rc != HI2_OK) return rc;
    rc = factor(pl, off + n1, n2);
    if (rc != HI2_OK) return rc;
    // X21 = -X22 T
    if ((rc = launch_split_block(x22, ld, n2, n2, ah, al, l2, false, pl.stream)) != HI2_OK) return rc;
    if ((rc = launch_split_block(a21, ld, n2, n1, bh, bl, l2, true, pl.stream)) != HI2_OK) return rc;
    return launch_gemm_tc(n2, n1, n2, ah, al, bh, bl, l2, x21, ld, GT_KA_LE_I | GT_NEGATE, pl.status, pl.stream);
  }
  // W (in the X21 slot) = A21 X11^T
  rc = product(true, n2, n1, n1, 1.0f, a21, x11, 0.0f, x21, ld, GEMM_KB_LE_J, pl.stream);
  if (rc != HI2_OK) return rc;
  // A22 -= W W^T (lower tiles)
  rc = product(true, n2, n2, n1, -1.0f, x21, x21, 1.0f, a22, ld, GEMM_LOWER_OUT, pl.stream);
  if (rc != HI2_OK) return rc;
  // T (in the A21 slot) = W X11
  rc = product(false, n2, n1, n1, 1.0f, x21, x11, 0.0f, a21, ld, GEMM_KB_GE_J, pl.stream);
  if (rc != HI2_OK) return rc;
  rc = factor(pl, off + n1, n2);
  if (rc != HI2_OK) return rc;
  // X21 = -X22 T
  return product(false, n2, n1, n2, -1.0f, x22, a21, 0.0f, x21, ld, GEMM_KA_LE_I, pl.stream);
}

}  // namespace
}  // namespace hi2

extern "C" size_t hi2_inverse_factor_workspace_bytes(int64_t k) {
  if (k <= 0) return 0;
  return ((size_t)k * (size_t)k * 2 + hi2::split_floats(k)) * sizeof(float) + 256;
}

extern "C" int hi2_inverse_factor(const float* hs, const float* lam, int64_t k, float* u,
                                  void* workspace, size_t workspace_bytes, int32_t* info,
                                  void* stream) {
  using namespace hi2;
  HI2_REQUIRE(k > 0, "inverse_factor: k must be positive");
  HI2_REQUIRE(hs && lam && u && info && workspace, "inverse_factor: null pointer");
  if (workspace_bytes < hi2_inverse_factor_workspace_bytes(k))
    return fail(HI2_ERR_WORKSPACE, "inverse_factor: workspace too small");
  HI2_REQUIRE(aligned16(workspace), "inverse_factor: workspace must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  {  // per device, so not cached: a process may drive several
    if (cudaFuncSetAttribute(leaf_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)LEAF_SMEM) != cudaSuccess)
      return fail(HI2_ERR_LAUNCH, "inverse_factor: cannot reserve shared memory");
  }
  Plan pl;
  // layout: one status word (256 bytes), A, X, then the TF32 parts
  pl.status = static_cast<int*>(workspace);
  pl.a = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256);
  pl.x = pl.a + k * k;
  pl.split = split_floats(k) ? pl.x + k * k : nullptr;
  pl.k = k, pl.info = info, pl.stream = s;
  // the whole recursion (K/64 leaves and the products between them) goes to the stream as one graph
  ChainGraph chain(s);
  auto enqueue = [&]() -> int {
    if (cudaMemsetAsync(pl.status, 0, 256, s) != cudaSuccess)
      return fail(HI2_ERR_LAUNCH, "inverse_factor: memset failed");
    const unsigned grid = (unsigned)ceil_div(k * k, 256);
    reverse_damp_kernel<<<grid, 256, 0, s>>>(hs, lam, k, pl.a);
    int rc = check_launch("inverse_factor reverse");
    if (rc != HI2_OK) return rc;
    if (cudaMemsetAsync(pl.x, 0, (size_t)k * k * sizeof(float), s) != cudaSuccess)
      return fail(HI2_ERR_LAUNCH, "inverse_factor: memset failed");
    rc = factor(pl, 0, k);
    if (rc != HI2_OK) return rc;
    if (pl.split != nullptr) merge_status_kernel<<<1, 1, 0, s>>>(pl.status, info);
    reverse_store_kernel<<<grid, 256, 0, s>>>(pl.x, k, u);
    return check_launch("inverse_factor store");
  };
  return chain.finish(enqueue(), "inverse_factor");
}
