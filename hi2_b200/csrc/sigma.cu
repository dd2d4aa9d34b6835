// Hessian basis change (hi2/hessian.py:50-68) and the 16x16 group moments (hi2/stats.py:27-33).
//
// transform_sigma is a tile-local operation because the rotation is block diagonal with 16-wide
// blocks: hs = sym(M (D s D) M^T) only mixes entries inside one 16x16 cell.  A thread block takes
// the pair of 64x64 tiles (bi, bj) and (bj, bi), applies scale, left and right products to both
// in shared memory, averages them and writes both, so sigma is read once and hs written once
// (8 K^2 bytes in all): bound by HBM.
#include "common.cuh"

namespace hi2 {
namespace {

constexpr int TS = 64;      // tile side
constexpr int LD = TS + 1;  // odd stride: rows and columns of a tile are both conflict-free

// y = H x for the normalised order-16 Sylvester matrix, in place: four butterfly stages (64
// additions) and one exact scaling by 1/4 instead of 256 multiply-adds.  The basis change is
// compared with the reference by tolerance (its own product runs in a BLAS), so the order of the
// additions is free here; the weight rotation, which must match bit for bit, keeps the plain sum.
__device__ __forceinline__ void wht16(float (&v)[16]) {
#pragma unroll
  for (int h = 1; h < 16; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if ((i & h) == 0) {
        const float a = v[i], b = v[i + h];
        v[i] = a + b;
        v[i + h] = a - b;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] *= 0.25f;
}

// The thread's four quads of tile (tr, tc) of sigma: 128-bit loads, all in flight at once (a scalar
// load per trip of a rolled loop left a few KB in flight per SM and the kernel at a fifth of the
// copy bandwidth).  k is a multiple of 16, so a quad never straddles the edge.
__device__ __forceinline__ void load_tile(float4 (&quad)[4], const float* __restrict__ sigma, int64_t k,
                                          int64_t tr, int64_t tc) {
  const int tid = threadIdx.x;
  const int64_t r0 = tr * TS, c0 = tc * TS;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int idx = tid + q * 256, i = idx >> 4, j = (idx & 15) * 4;
    const int64_t gr = r0 + i, gc = c0 + j;
    quad[q] = (gr < k && gc < k) ? __ldg(reinterpret_cast<const float4*>(sigma + gr * k + gc))
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// Tile (tr, tc) of sigma/denom (already in `quad`) scaled by inv[row]*inv[col], then M . M^T on
// flagged groups.
__device__ void transform_tile(float (*tile)[LD], const float4 (&quad)[4], float denom,
                               const float* __restrict__ inv_s, const uint8_t* __restrict__ had,
                               int64_t k, int64_t tr, int64_t tc) {
  const int tid = threadIdx.x;
  const int64_t r0 = tr * TS, c0 = tc * TS;
  const Recip rc = make_recip(denom);  // sigma / n with the IEEE quotient, as the reference's mean()
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int idx = tid + q * 256, i = idx >> 4, j = (idx & 15) * 4;
    float v[4] = {quad[q].x, quad[q].y, quad[q].z, quad[q].w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      if (denom != 1.0f) v[t] = div_by(v[t], denom, rc);
      if (inv_s != nullptr) v[t] = (v[t] * inv_s[i]) * inv_s[TS + j + t];
      tile[i][j + t] = v[t];
    }
  }
  __syncthreads();
  {  // left product: thread = (column c, row group gi)
    const int c = tid & 63, gi = tid >> 6;
    const int64_t grp = (r0 >> 4) + gi;
    if (grp * 16 < k && had[grp]) {
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = tile[gi * 16 + j][c];
      wht16(v);
#pragma unroll
      for (int i = 0; i < 16; ++i) tile[gi * 16 + i][c] = v[i];
    }
  }
  __syncthreads();
  {  // right product: thread = (row i, column group gj)
    const int i = tid & 63, gj = tid >> 6;
    const int64_t grp = (c0 >> 4) + gj;
    if (grp * 16 < k && had[grp]) {
      float v[16];
#pragma unroll
      for (int q = 0; q < 16; ++q) v[q] = tile[i][gj * 16 + q];
      wht16(v);
#pragma unroll
      for (int l = 0; l < 16; ++l) tile[i][gj * 16 + l] = v[l];
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(256)
transform_sigma_kernel(const float* __restrict__ sigma, float denom,
                       const uint16_t* __restrict__ col_scale, const uint8_t* __restrict__ had,
                       int64_t k, float* __restrict__ hs, float* __restrict__ diag) {
  const int64_t bi = blockIdx.y, bj = blockIdx.x;
  if (bi > bj) return;
  __shared__ float P[TS][LD];
  __shared__ float Q[TS][LD];
  __shared__ float inv_rc[2 * TS];  // 1/s of the rows of tile (bi, .) then of (bj, .)
  const int tid = threadIdx.x;
  const bool scaled = col_scale != nullptr;
  if (scaled && tid < 2 * TS) {
    const int64_t idx = (tid < TS ? bi * TS + tid : bj * TS + (tid - TS));
    float v = 1.0f;
    if (idx < k) v = __fdiv_rn(1.0f, __half2float(__ushort_as_half(col_scale[idx])));
    inv_rc[tid] = v;
  }
  __syncthreads();
  // both tiles' loads go out before anything is computed: 128 bytes in flight per thread
  float4 quad_p[4], quad_q[4];
  load_tile(quad_p, sigma, k, bi, bj);
  if (bi != bj) load_tile(quad_q, sigma, k, bj, bi);
  // tile (bi, bj): rows scaled by inv[bi-range], columns by inv[bj-range]
  transform_tile(P, quad_p, denom, scaled ? inv_rc : nullptr, had, k, bi, bj);
  if (bi != bj) {
    // tile (bj, bi) wants the two halves of inv_rc swapped
    __shared__ float inv_cr[2 * TS];
    if (scaled && tid < 2 * TS) inv_cr[tid] = inv_rc[(tid + TS) % (2 * TS)];
    __syncthreads();
    transform_tile(Q, quad_q, denom, scaled ? inv_cr : nullptr, had, k, bj, bi);
  }
  const int64_t r0 = bi * TS, c0 = bj * TS;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int idx = tid + q * 256, i = idx >> 4, j = (idx & 15) * 4;
    // upper tile (bi, bj), element (i, j) = 0.5 * (P[i][j] + Q[j][i])
    if (r0 + i < k && c0 + j < k) {
      float o[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) o[t] = 0.5f * (P[i][j + t] + ((bi == bj) ? P[j + t][i] : Q[j + t][i]));
      *reinterpret_cast<float4*>(hs + (r0 + i) * k + c0 + j) = make_float4(o[0], o[1], o[2], o[3]);
    }
    // lower tile (bj, bi), element (i, j) = 0.5 * (Q[i][j] + P[j][i]): the same sum, mirrored
    if (bi != bj && c0 + i < k && r0 + j < k) {
      float o[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) o[t] = 0.5f * (P[j + t][i] + Q[i][j + t]);
      *reinterpret_cast<float4*>(hs + (c0 + i) * k + r0 + j) = make_float4(o[0], o[1], o[2], o[3]);
    }
  }
  if (bi == bj && diag != nullptr && tid < TS && r0 + tid < k)
    diag[r0 + tid] = 0.5f * (P[tid][tid] + P[tid][tid]);
}

__global__ void __launch_bounds__(256)
group_moments_kernel(const float* __restrict__ s, int64_t k, double* __restrict__ g) {
  const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;  // (group, i, j)
  if (idx >= k * 16) return;
  const int64_t grp = idx >> 8;
  const int i = (int)(idx >> 4) & 15, j = (int)idx & 15;
  g[idx] += (double)s[(grp * 16 + i) * k + grp * 16 + j];
}

// Group moments straight from activations (hi2/stats.py:27-33): a thread block takes a slab of
// up to 4096 tokens (the reference's chunk) and 8 groups (128 columns); the slab passes through
// shared memory 64 tokens at a time, lane l of warp g owns row l/2 and eight columns of group g's
// 16 x 16 block.  Products are summed in fp32 over 64 tokens, the partial sums in fp64, and the slab's
// sum is added to the fp64 total with one atomic per entry (the reference sums 4096 tokens in fp32
// with a blocked einsum before widening; a serial fp32 sum that long would lose two more digits).
template <typename TX>
__global__ void __launch_bounds__(256)
group_moments_update_kernel(const TX* __restrict__ x, int64_t tokens, int64_t k, double* __restrict__ g) {
  __shared__ float xs[64][128 + 4];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t col0 = (int64_t)blockIdx.x * 128;
  const int64_t t_begin = (int64_t)blockIdx.y * 4096;
  const int64_t t_end = t_begin + 4096 < tokens ? t_begin + 4096 : tokens;
  const int row_i = lane >> 1, j0 = (lane & 1) * 8;
  double total[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) total[j] = 0.0;
  for (int64_t t0 = t_begin; t0 < t_end; t0 += 64) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
    for (int idx = tid; idx < 64 * 128; idx += 256) {
      const int tt = idx >> 7, c = idx & 127;
      float v = 0.0f;
      if (t0 + tt < t_end && col0 + c < k) v = (float)x[(t0 + tt) * k + col0 + c];
      xs[tt][c] = v;
    }
    __syncthreads();
#pragma unroll 8
    for (int tt = 0; tt < 64; ++tt) {
      const float a = xs[tt][warp * 16 + row_i];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(a, xs[tt][warp * 16 + j0 + j], acc[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) total[j] += (double)acc[j];
    __syncthreads();
  }
  const int64_t grp = (col0 >> 4) + warp;
  if (grp * 16 < k) {
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(g + grp * 256 + row_i * 16 + j0 + j, total[j]);
  }
}

}  // namespace
}  // namespace hi2

extern "C" int hi2_group_moments_update(const void* x, int dtype, int64_t tokens, int64_t k, double* g,
                                        void* stream) {
  using namespace hi2;
  HI2_REQUIRE(k > 0 && k % 16 == 0, "group_moments_update: k must be a positive multiple of 16");
  HI2_REQUIRE(tokens >= 0, "group_moments_update: negative token count");
  if (tokens == 0) return HI2_OK;
  HI2_REQUIRE(x && g, "group_moments_update: null pointer");
  dim3 grid((unsigned)ceil_div(k, 128), (unsigned)ceil_div(tokens, 4096));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == HI2_BF16)
    group_moments_update_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), tokens, k, g);
  else if (dtype == HI2_F16)
    group_moments_update_kernel<<<grid, 256, 0, s>>>(static_cast<const __half*>(x), tokens, k, g);
  else if (dtype == HI2_F32)
    group_moments_update_kernel<<<grid, 256, 0, s>>>(static_cast<const float*>(x), tokens, k, g);
  else
    return fail(HI2_ERR_ARG, "group_moments_update: dtype must be F16, BF16 or F32");
  return check_launch("group_moments_update");
}

extern "C" int hi2_transform_sigma(const float* sigma, float denom, const uint16_t* col_scale,
                                   const uint8_t* had, int64_t k, float* hs, float* diag,
                                   void* stream) {
  using namespace hi2;
  HI2_REQUIRE(k > 0 && k % 16 == 0, "transform_sigma: k must be a positive multiple of 16");
  HI2_REQUIRE(sigma && had && hs, "transform_sigma: null pointer");
  HI2_REQUIRE(sigma != hs, "transform_sigma: in-place operation is not supported");
  HI2_REQUIRE(denom > 0.0f, "transform_sigma: denom must be positive");
  const unsigned nt = (unsigned)ceil_div(k, TS);
  transform_sigma_kernel<<<dim3(nt, nt), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      sigma, denom, col_scale, had, k, hs, diag);
  return check_launch("transform_sigma");
}

extern "C" int hi2_group_moments(const float* s, int64_t k, double* g, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(k > 0 && k % 16 == 0, "group_moments: k must be a positive multiple of 16");
  HI2_REQUIRE(s && g, "group_moments: null pointer");
  group_moments_kernel<<<(unsigned)ceil_div(k * 16, 256), 256, 0,
                         static_cast<cudaStream_t>(stream)>>>(s, k, g);
  return check_launch("group_moments");
}
