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

// Factorise the n x n (n <= 64) diagonal block at `off` (lower part of a, leading dim ld) and
// write its inverse, zeros above the diagonal included, to the same place of x (fp32 in memory,
// fp64 inside the block).  One thread block:
// 256 threads as a 16 x 16 grid for the trailing updates of the factorisation (two barriers per
// column), then as 64 columns x 4 partial sums for the row-by-row triangular inverse (the four
// partial sums of a column sit in adjacent lanes and meet by shuffle, one barrier per row).
__global__ void __launch_bounds__(256)
leaf_kernel(const float* __restrict__ a, float* __restrict__ x, int64_t ld, int64_t off, int n,
            int32_t* info) {
  extern __shared__ double leaf_smem[];
  double (*L)[LDL] = reinterpret_cast<double (*)[LDL]>(leaf_smem);
  double (*X)[LDL] = reinterpret_cast<double (*)[LDL]>(leaf_smem + NB * LDL);
  __shared__ double inv_diag[NB];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const float* src = a + off * ld + off;
  for (int idx = tid; idx < NB * NB; idx += 256) {
    const int i = idx >> 6, j = idx & 63;
    L[i][j] = (i < n && j <= i) ? (double)src[(int64_t)i * ld + j] : 0.0;
    X[i][j] = 0.0;
  }
  __syncthreads();
  for (int j = 0; j < n; ++j) {
    double piv = L[j][j];  // final: every update of (j, j) was followed by a barrier
    if (!(piv > 0.0)) {    // also catches NaN
      if (tid == 0) atomicCAS(info, 0, (int32_t)(off + j + 1));
      piv = 1.0;
    }
    const double inv = inv_sqrt(piv);  // L[j][j] itself stays un-rooted; 1/sqrt is kept instead
    if (tid == 0) inv_diag[j] = inv;
    for (int i = j + 1 + tid; i < n; i += 256) L[i][j] *= inv;
    __syncthreads();
    for (int i = j + 1 + ty; i < n; i += 16) {
      const double lij = L[i][j];
      for (int c = j + 1 + tx; c <= i; c += 16) L[i][c] = fma(-lij, L[c][j], L[i][c]);
    }
    __syncthreads();
  }
  // X = L^-1, row by row: X[i][c] = -(sum_{q=c}^{i-1} L[i][q] X[q][c]) / L[i][i], X[i][i] = 1 / L[i][i]
  const int c = tid >> 2, part = tid & 3;
  if (tid < n) X[tid][tid] = inv_diag[tid];
  __syncthreads();
  for (int i = 1; i < n; ++i) {
    double acc = 0.0;
    if (c < i)
      for (int q = c + part; q < i; q += 4) acc = fma(L[i][q], X[q][c], acc);
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    if (part == 0 && c < i) X[i][c] = -acc * inv_diag[i];
    __syncthreads();
  }
  float* dst = x + off * ld + off;
  for (int idx = tid; idx < n * n; idx += 256) {
    const int i = idx / n, j = idx % n;
    dst[(int64_t)i * ld + j] = (float)X[i][j];
  }
}

struct Plan {
  float* a;
  float* x;
  int64_t k;
  int32_t* info;
  cudaStream_t stream;
};

int product(bool trans_b, int64_t m, int64_t n, int64_t kk, float alpha, const float* a,
            const float* b, float beta, float* c, int64_t ld, int flags, cudaStream_t stream) {
  GemmArgs<float, float, float> p;
  p.m = m, p.n = n, p.kk = kk, p.alpha = alpha, p.beta = beta;
  p.a = a, p.lda = ld, p.b = b, p.ldb = ld, p.c = c, p.ldc = ld, p.flags = flags;
  return launch_gemm_async<float, 8, 8, 16>(false, trans_b, p, stream, "inverse_factor");
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
  return k > 0 ? (size_t)k * (size_t)k * 2 * sizeof(float) : 0;
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
  pl.a = static_cast<float*>(workspace);
  pl.x = pl.a + k * k;
  pl.k = k, pl.info = info, pl.stream = s;
  const unsigned grid = (unsigned)ceil_div(k * k, 256);
  reverse_damp_kernel<<<grid, 256, 0, s>>>(hs, lam, k, pl.a);
  int rc = check_launch("inverse_factor reverse");
  if (rc != HI2_OK) return rc;
  if (cudaMemsetAsync(pl.x, 0, (size_t)k * k * sizeof(float), s) != cudaSuccess)
    return fail(HI2_ERR_LAUNCH, "inverse_factor: memset failed");
  rc = factor(pl, 0, k);
  if (rc != HI2_OK) return rc;
  reverse_store_kernel<<<grid, 256, 0, s>>>(pl.x, k, u);
  return check_launch("inverse_factor store");
}
