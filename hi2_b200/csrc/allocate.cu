// One multiplier of the global allocation (hi2/allocate.py:88-137): every row takes the first
// candidate that minimises cost + lam * bits, in fp64 with the product and the sum rounded
// separately (a fused multiply-add would move ties).  The picked bits are whole numbers, so their
// sum is exact in any order and one atomic per thread block is enough.
#include "common.cuh"

namespace hi2 {
namespace {

__global__ void __launch_bounds__(256)
solve_kernel(const double* __restrict__ cost, const double* __restrict__ bits, int n_cand,
             int64_t n_rows, double lam, int64_t* __restrict__ picks, double* picked_bits) {
  __shared__ double red[8];
  const int64_t r = (int64_t)blockIdx.x * 256 + threadIdx.x;
  double mine = 0.0;
  if (r < n_rows) {
    double best = __dadd_rn(cost[r], __dmul_rn(lam, bits[r]));
    int idx = 0;
    for (int c = 1; c < n_cand; ++c) {
      const double v = __dadd_rn(cost[(int64_t)c * n_rows + r], __dmul_rn(lam, bits[(int64_t)c * n_rows + r]));
      if (v < best) best = v, idx = c;
    }
    picks[r] = idx;
    mine = bits[(int64_t)idx * n_rows + r];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < 8; ++i) t += red[i];
    atomicAdd(picked_bits, t);
  }
}

constexpr int MAX_LAMS = 32;
struct Lams {
  double v[MAX_LAMS];
  int n;
};

// Picked bits under several multipliers at once (no picks written): lets the host take five
// bisection steps per round trip by evaluating the 31 multipliers the next five steps can reach.
__global__ void __launch_bounds__(256)
solve_many_kernel(const double* __restrict__ cost, const double* __restrict__ bits, int n_cand,
                  int64_t n_rows, Lams lams, double* totals) {
  __shared__ double red[MAX_LAMS][8];
  const int64_t r = (int64_t)blockIdx.x * 256 + threadIdx.x;
  double mine[MAX_LAMS];
#pragma unroll
  for (int l = 0; l < MAX_LAMS; ++l) mine[l] = 0.0;
  if (r < n_rows) {
#pragma unroll
    for (int l = 0; l < MAX_LAMS; ++l) {
      if (l >= lams.n) break;
      double best = __dadd_rn(cost[r], __dmul_rn(lams.v[l], bits[r]));
      double picked = bits[r];
      for (int c = 1; c < n_cand; ++c) {
        const double b = bits[(int64_t)c * n_rows + r];
        const double v = __dadd_rn(cost[(int64_t)c * n_rows + r], __dmul_rn(lams.v[l], b));
        if (v < best) best = v, picked = b;
      }
      mine[l] = picked;
    }
  }
#pragma unroll
  for (int l = 0; l < MAX_LAMS; ++l) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine[l] += __shfl_xor_sync(0xffffffffu, mine[l], o);
    if ((threadIdx.x & 31) == 0) red[l][threadIdx.x >> 5] = mine[l];
  }
  __syncthreads();
  if (threadIdx.x < lams.n) {
    double t = 0.0;
    for (int i = 0; i < 8; ++i) t += red[threadIdx.x][i];
    atomicAdd(totals + threadIdx.x, t);
  }
}

}  // namespace
}  // namespace hi2

extern "C" int hi2_allocate_bits(const double* cost, const double* bits, int n_cand, int64_t n_rows,
                                 const double* lams_host, int n_lams, double* totals, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(n_cand >= 1 && n_rows >= 0, "allocate_bits: bad sizes");
  HI2_REQUIRE(n_lams >= 1 && n_lams <= MAX_LAMS && lams_host, "allocate_bits: 1 to 32 multipliers");
  if (n_rows == 0) return HI2_OK;
  HI2_REQUIRE(cost && bits && totals, "allocate_bits: null pointer");
  Lams l;
  l.n = n_lams;
  for (int i = 0; i < MAX_LAMS; ++i) l.v[i] = i < n_lams ? lams_host[i] : 0.0;
  solve_many_kernel<<<(unsigned)ceil_div(n_rows, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      cost, bits, n_cand, n_rows, l, totals);
  return check_launch("allocate_bits");
}

extern "C" int hi2_allocate_solve(const double* cost, const double* bits, int n_cand, int64_t n_rows,
                                  double lam, int64_t* picks, double* picked_bits, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(n_cand >= 1 && n_rows >= 0, "allocate_solve: bad sizes");
  if (n_rows == 0) return HI2_OK;
  HI2_REQUIRE(cost && bits && picks && picked_bits, "allocate_solve: null pointer");
  solve_kernel<<<(unsigned)ceil_div(n_rows, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      cost, bits, n_cand, n_rows, lam, picks, picked_bits);
  return check_launch("allocate_solve");
}
