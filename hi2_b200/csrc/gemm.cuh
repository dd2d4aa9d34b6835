// Register-tiled FMA matrix product used where the path needs full fp32 / fp64 accuracy with
// every operand in its storage precision: the lazy trailing update of GPTQ, the products of the
// refinement sweep, and the fp64 products of the blocked inverse factor.
//
//   C[m, n] = alpha * sum_k opA[m, k] * opB[k, n] + beta * C[m, n]        (row-major)
//
// 256 threads as a 16 x 16 grid; a thread owns TM x TN outputs laid out in 16-byte pieces that
// are 16 pieces apart, so the shared-memory reads of a warp are contiguous (B side) or a
// broadcast (A side).  Global tiles are fetched into registers one step ahead of the math.
// Triangular structure of an operand is expressed as a k-range per output tile.
#pragma once

#include "common.cuh"

namespace hi2 {

enum : int {
  GEMM_LOWER_OUT = 1,  // skip output tiles that lie strictly above the diagonal
  GEMM_KA_LE_I = 2,    // opA[i, k] == 0 for k > i   (A lower triangular, square with the rows)
  GEMM_KB_GE_J = 4,    // opB[k, j] == 0 for k < j   (B lower triangular, not transposed)
  GEMM_KB_LE_J = 8,    // opB[k, j] == 0 for k > j   (B = L^T with L lower triangular)
};

template <typename T, typename TA, typename TB>
struct GemmArgs {
  int64_t m, n, kk;
  T alpha, beta;
  const TA* a;
  int64_t lda;
  const TB* b;
  int64_t ldb;
  T* c;
  int64_t ldc;
  int flags;
  // reduction window: only k in [k_begin, k_end) is summed (k_begin a multiple of 16).  A caller
  // that wants a long reduction added up in pieces calls once per window with beta = 1 after the
  // first, which bounds the length of any one fp32 accumulation chain.
  int64_t k_begin = 0, k_end = INT64_MAX;
};

template <typename T>
__device__ __forceinline__ T fma_t(T a, T b, T c);
template <>
__device__ __forceinline__ float fma_t<float>(float a, float b, float c) { return fmaf(a, b, c); }
template <>
__device__ __forceinline__ double fma_t<double>(double a, double b, double c) { return fma(a, b, c); }

template <typename T, typename S>
__device__ __forceinline__ T widen(S v) { return (T)v; }
template <>
__device__ __forceinline__ float widen<float, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float widen<float, __half>(__half v) { return __half2float(v); }

template <typename T, typename TA, typename TB, int TM, int TN, int BK, bool TRANS_A, bool TRANS_B>
// fp32: two resident blocks per SM hide the barrier stalls (measured 1.3x); fp64 needs all 255
// registers for its 8 x 4 tile and gains nothing from a second block
__global__ void __launch_bounds__(256, (sizeof(T) == 4 ? 2 : 1))
gemm_kernel(const GemmArgs<T, TA, TB> p) {
  constexpr int V = 16 / sizeof(T);  // elements per 16-byte piece
  constexpr int BM = 16 * TM, BN = 16 * TN;
  constexpr int NT = 256;
  constexpr int A_PER = BM * BK / NT, B_PER = BN * BK / NT;
  static_assert(TM % V == 0 && TN % V == 0, "micro-tile must be whole 16-byte pieces");
  static_assert((BM * BK) % NT == 0 && (BN * BK) % NT == 0, "tile loads must divide evenly");

  __shared__ __align__(16) T As[BK][BM + V];
  __shared__ __align__(16) T Bs[BK][BN + V];

  const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
  if ((p.flags & GEMM_LOWER_OUT) && n0 > m0 + BM - 1) return;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;

  int64_t k_lo = 0, k_hi = p.kk;
  if (p.flags & GEMM_KA_LE_I) k_hi = min(k_hi, m0 + BM);
  if (p.flags & GEMM_KB_LE_J) k_hi = min(k_hi, n0 + BN);
  if (p.flags & GEMM_KB_GE_J) k_lo = (n0 / BK) * BK;
  k_lo = max(k_lo, p.k_begin), k_hi = min(k_hi, p.k_end);

  T acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = T(0);

  T ra[A_PER], rb[B_PER];
  auto fetch = [&](int64_t k0) {
#pragma unroll
    for (int s = 0; s < A_PER; ++s) {
      const int idx = tid + s * NT;
      const int mi = TRANS_A ? idx % BM : idx / BK, ki = TRANS_A ? idx / BM : idx % BK;
      const int64_t gm = m0 + mi, gk = k0 + ki;
      T v = T(0);
      if (gm < p.m && gk < k_hi)
        v = widen<T, TA>(TRANS_A ? p.a[gk * p.lda + gm] : p.a[gm * p.lda + gk]);
      ra[s] = v;
    }
#pragma unroll
    for (int s = 0; s < B_PER; ++s) {
      const int idx = tid + s * NT;
      const int ni = TRANS_B ? idx / BK : idx % BN, ki = TRANS_B ? idx % BK : idx / BN;
      const int64_t gn = n0 + ni, gk = k0 + ki;
      T v = T(0);
      if (gn < p.n && gk < k_hi)
        v = widen<T, TB>(TRANS_B ? p.b[gn * p.ldb + gk] : p.b[gk * p.ldb + gn]);
      rb[s] = v;
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int s = 0; s < A_PER; ++s) {
      const int idx = tid + s * NT;
      const int mi = TRANS_A ? idx % BM : idx / BK, ki = TRANS_A ? idx / BM : idx % BK;
      As[ki][mi] = ra[s];
    }
#pragma unroll
    for (int s = 0; s < B_PER; ++s) {
      const int idx = tid + s * NT;
      const int ni = TRANS_B ? idx / BK : idx % BN, ki = TRANS_B ? idx % BK : idx / BN;
      Bs[ki][ni] = rb[s];
    }
  };

  if (k_lo < k_hi) fetch(k_lo);
  for (int64_t k0 = k_lo; k0 < k_hi; k0 += BK) {
    stash();
    __syncthreads();
    if (k0 + BK < k_hi) fetch(k0 + BK);
#pragma unroll
    for (int ki = 0; ki < BK; ++ki) {
      T fa[TM], fb[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) fa[i] = As[ki][(i / V) * (16 * V) + ty * V + (i % V)];
#pragma unroll
      for (int j = 0; j < TN; ++j) fb[j] = Bs[ki][(j / V) * (16 * V) + tx * V + (j % V)];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fma_t<T>(fa[i], fb[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int64_t gm = m0 + (i / V) * (16 * V) + ty * V + (i % V);
    if (gm >= p.m) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int64_t gn = n0 + (j / V) * (16 * V) + tx * V + (j % V);
      if (gn >= p.n) continue;
      T* dst = p.c + gm * p.ldc + gn;
      T v = p.alpha * acc[i][j];
      if (p.beta != T(0)) v = v + p.beta * *dst;
      *dst = v;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// The same product for operands already in the compute type: tiles go from global to shared
// memory with cp.async (element-wise, so the k-major <-> m-major transposition and the zero fill
// of edges and triangular k-ranges happen in the copy), three stages deep, one barrier per
// k-tile and no staging registers.
// ---------------------------------------------------------------------------------------------
template <int BYTES>
__device__ __forceinline__ void cp_async_elem(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int src_bytes = valid ? BYTES : 0;  // 0: nothing is read, the destination is zero-filled
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(dst), "l"(gsrc), "n"(BYTES), "r"(src_bytes)
               : "memory");
}

template <typename T, int TM, int TN, int BK, bool TRANS_A, bool TRANS_B>
__global__ void __launch_bounds__(256, (sizeof(T) == 4 ? 2 : 1))
gemm_async_kernel(const GemmArgs<T, T, T> p) {
  constexpr int V = 16 / sizeof(T);
  constexpr int BM = 16 * TM, BN = 16 * TN, NT = 256, STAGES = 3;
  constexpr int A_PER = BM * BK / NT, B_PER = BN * BK / NT;
  constexpr int A_STAGE = BK * (BM + V), B_STAGE = BK * (BN + V);
  static_assert(TM % V == 0 && TN % V == 0, "micro-tile must be whole 16-byte pieces");
  extern __shared__ __align__(16) unsigned char gemm_smem[];
  T* As = reinterpret_cast<T*>(gemm_smem);          // [STAGES][BK][BM + V]
  T* Bs = As + STAGES * A_STAGE;                    // [STAGES][BK][BN + V]

  const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
  if ((p.flags & GEMM_LOWER_OUT) && n0 > m0 + BM - 1) return;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  int64_t k_lo = 0, k_hi = p.kk;
  if (p.flags & GEMM_KA_LE_I) k_hi = min(k_hi, m0 + BM);
  if (p.flags & GEMM_KB_LE_J) k_hi = min(k_hi, n0 + BN);
  if (p.flags & GEMM_KB_GE_J) k_lo = (n0 / BK) * BK;
  k_lo = max(k_lo, p.k_begin), k_hi = min(k_hi, p.k_end);

  auto issue = [&](int64_t k0, int slot) {
    T* as = As + slot * A_STAGE;
    T* bs = Bs + slot * B_STAGE;
#pragma unroll
    for (int s = 0; s < A_PER; ++s) {
      const int idx = tid + s * NT;
      const int mi = TRANS_A ? idx % BM : idx / BK, ki = TRANS_A ? idx / BM : idx % BK;
      const int64_t gm = m0 + mi, gk = k0 + ki;
      const bool ok = gm < p.m && gk < k_hi;
      const T* src = ok ? (TRANS_A ? p.a + gk * p.lda + gm : p.a + gm * p.lda + gk) : p.a;
      cp_async_elem<sizeof(T)>(as + ki * (BM + V) + mi, src, ok);
    }
#pragma unroll
    for (int s = 0; s < B_PER; ++s) {
      const int idx = tid + s * NT;
      const int ni = TRANS_B ? idx / BK : idx % BN, ki = TRANS_B ? idx % BK : idx / BN;
      const int64_t gn = n0 + ni, gk = k0 + ki;
      const bool ok = gn < p.n && gk < k_hi;
      const T* src = ok ? (TRANS_B ? p.b + gn * p.ldb + gk : p.b + gk * p.ldb + gn) : p.b;
      cp_async_elem<sizeof(T)>(bs + ki * (BN + V) + ni, src, ok);
    }
  };

  T acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = T(0);

  const int64_t tiles = k_hi > k_lo ? (k_hi - k_lo + BK - 1) / BK : 0;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < tiles) issue(k_lo + (int64_t)s * BK, s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int64_t t = 0; t < tiles; ++t) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();  // tile t has landed for everyone; the slot of tile t-1 is free
    if (t + STAGES - 1 < tiles) issue(k_lo + (t + STAGES - 1) * BK, (int)((t + STAGES - 1) % STAGES));
    asm volatile("cp.async.commit_group;" ::: "memory");
    const T* as = As + (int)(t % STAGES) * A_STAGE;
    const T* bs = Bs + (int)(t % STAGES) * B_STAGE;
#pragma unroll
    for (int ki = 0; ki < BK; ++ki) {
      T fa[TM], fb[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) fa[i] = as[ki * (BM + V) + (i / V) * (16 * V) + ty * V + (i % V)];
#pragma unroll
      for (int j = 0; j < TN; ++j) fb[j] = bs[ki * (BN + V) + (j / V) * (16 * V) + tx * V + (j % V)];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fma_t<T>(fa[i], fb[j], acc[i][j]);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int64_t gm = m0 + (i / V) * (16 * V) + ty * V + (i % V);
    if (gm >= p.m) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int64_t gn = n0 + (j / V) * (16 * V) + tx * V + (j % V);
      if (gn >= p.n) continue;
      T* dst = p.c + gm * p.ldc + gn;
      T v = p.alpha * acc[i][j];
      if (p.beta != T(0)) v = v + p.beta * *dst;
      *dst = v;
    }
  }
}

template <typename T, int TM, int TN, int BK>
int launch_gemm_async(bool trans_a, bool trans_b, const GemmArgs<T, T, T>& p, cudaStream_t stream,
                      const char* what) {
  if (p.m <= 0 || p.n <= 0) return HI2_OK;
  constexpr int V = 16 / sizeof(T);
  constexpr size_t smem = (size_t)3 * BK * ((16 * TM + V) + (16 * TN + V)) * sizeof(T);
  dim3 grid((unsigned)ceil_div(p.n, 16 * TN), (unsigned)ceil_div(p.m, 16 * TM));
#define HI2_GEMM_ASYNC(TA_, TB_)                                                                        \
  do {                                                                                                  \
    auto kern = gemm_async_kernel<T, TM, TN, BK, TA_, TB_>;                                             \
    static bool reserved[64] = {false}; /* per device: the attribute belongs to the context */         \
    int dev_ = 0;                                                                                       \
    cudaGetDevice(&dev_);                                                                               \
    if (smem > 48 * 1024 && !(dev_ >= 0 && dev_ < 64 && reserved[dev_])) {                              \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=         \
          cudaSuccess)                                                                                  \
        return fail(HI2_ERR_LAUNCH, "gemm: cannot reserve shared memory");                              \
      if (dev_ >= 0 && dev_ < 64) reserved[dev_] = true;                                                \
    }                                                                                                   \
    kern<<<grid, 256, smem, stream>>>(p);                                                               \
  } while (0)
  if (!trans_a && !trans_b) HI2_GEMM_ASYNC(false, false);
  else if (!trans_a && trans_b) HI2_GEMM_ASYNC(false, true);
  else if (trans_a && !trans_b) HI2_GEMM_ASYNC(true, false);
  else HI2_GEMM_ASYNC(true, true);
#undef HI2_GEMM_ASYNC
  return check_launch(what);
}

template <typename T, typename TA, typename TB, int TM, int TN, int BK>
int launch_gemm(bool trans_a, bool trans_b, const GemmArgs<T, TA, TB>& p, cudaStream_t stream,
                const char* what) {
  if (p.m <= 0 || p.n <= 0) return HI2_OK;
  dim3 grid((unsigned)ceil_div(p.n, 16 * TN), (unsigned)ceil_div(p.m, 16 * TM));
  if (!trans_a && !trans_b)
    gemm_kernel<T, TA, TB, TM, TN, BK, false, false><<<grid, 256, 0, stream>>>(p);
  else if (!trans_a && trans_b)
    gemm_kernel<T, TA, TB, TM, TN, BK, false, true><<<grid, 256, 0, stream>>>(p);
  else if (trans_a && !trans_b)
    gemm_kernel<T, TA, TB, TM, TN, BK, true, false><<<grid, 256, 0, stream>>>(p);
  else
    gemm_kernel<T, TA, TB, TM, TN, BK, true, true><<<grid, 256, 0, stream>>>(p);
  return check_launch(what);
}

}  // namespace hi2
