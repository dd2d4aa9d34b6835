// Bit packing of codes and the scatter of one candidate group into the flat per-tensor buffers
// (hi2/format.py:73-85 pack_codes, :158-171 assemble).  Integer work, bound by HBM traffic:
// a thread reads the 16 / 8 / 4 code bytes of one output word with one vector load and writes
// one int32; neighbouring threads touch neighbouring addresses on both sides, and four words are
// in flight per thread.
#include "common.cuh"

namespace hi2 {
namespace {

// The `per = 32 / nbits` consecutive code bytes of one output word (p is per-byte aligned).
template <int NBITS>
struct Raw {
  uint32_t v[(32 / NBITS) / 4];
};
template <int NBITS>
__device__ __forceinline__ Raw<NBITS> load_raw(const uint8_t* __restrict__ p) {
  constexpr int PER = 32 / NBITS;
  Raw<NBITS> r;
  if constexpr (PER == 16) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    r.v[0] = v.x, r.v[1] = v.y, r.v[2] = v.z, r.v[3] = v.w;
  } else if constexpr (PER == 8) {
    uint2 v = *reinterpret_cast<const uint2*>(p);
    r.v[0] = v.x, r.v[1] = v.y;
  } else {
    r.v[0] = *reinterpret_cast<const uint32_t*>(p);
  }
  return r;
}
// One packed word; *bad is raised when a code does not fit nbits.
template <int NBITS>
__device__ __forceinline__ uint32_t pack_raw(const Raw<NBITS>& r, int32_t* bad) {
  constexpr int PER = 32 / NBITS;
  uint32_t word = 0, over = 0;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const uint32_t c = (r.v[i >> 2] >> (8 * (i & 3))) & 0xffu;
    over |= c >> NBITS;
    word |= (c & ((1u << NBITS) - 1u)) << (NBITS * i);
  }
  if (over != 0 && NBITS < 8) atomicOr(bad, 1);
  return word;
}

// A thread takes PACK_UN words per trip and issues all their loads first: one 16-byte load in
// flight per thread does not cover the latency of HBM.
constexpr int PACK_UN = 4;

template <int NBITS>
__global__ void __launch_bounds__(256)
pack_kernel(const uint8_t* __restrict__ codes, int32_t* __restrict__ words, int64_t n_words,
            int32_t* bad) {
  constexpr int PER = 32 / NBITS;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < n_words; i0 += stride * PACK_UN) {
    Raw<NBITS> raw[PACK_UN];
#pragma unroll
    for (int u = 0; u < PACK_UN; ++u)
      if (i0 + u * stride < n_words) raw[u] = load_raw<NBITS>(codes + (i0 + u * stride) * PER);
#pragma unroll
    for (int u = 0; u < PACK_UN; ++u)
      if (i0 + u * stride < n_words) words[i0 + u * stride] = (int32_t)pack_raw<NBITS>(raw[u], bad);
  }
}

// grid.x strides the words of a row, grid.y the rows of the piece.
template <int NBITS>
__global__ void __launch_bounds__(256)
assemble_kernel(const int64_t* __restrict__ rows, int64_t n_rows, const uint8_t* __restrict__ codes,
                const uint8_t* __restrict__ params, const uint16_t* __restrict__ consts, int64_t k,
                int64_t words_per_row, int64_t param_bytes_per_row,
                const int64_t* __restrict__ code_off, const int64_t* __restrict__ param_off,
                int32_t* __restrict__ out_codes, uint8_t* __restrict__ out_params,
                uint16_t* __restrict__ out_consts, int32_t* bad) {
  constexpr int PER = 32 / NBITS;
  for (int64_t r = blockIdx.y; r < n_rows; r += gridDim.y) {
    const int64_t row = rows[r];
    const int64_t cbase = code_off[row], pbase = 2 * param_off[row];
    const uint8_t* src = codes + r * k;
    const int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t w0 = t0; w0 < words_per_row; w0 += step * PACK_UN) {
      Raw<NBITS> raw[PACK_UN];
#pragma unroll
      for (int u = 0; u < PACK_UN; ++u)
        if (w0 + u * step < words_per_row) raw[u] = load_raw<NBITS>(src + (w0 + u * step) * PER);
#pragma unroll
      for (int u = 0; u < PACK_UN; ++u)
        if (w0 + u * step < words_per_row)
          out_codes[cbase + w0 + u * step] = (int32_t)pack_raw<NBITS>(raw[u], bad);
    }
    for (int64_t b = t0; b < param_bytes_per_row; b += step)
      out_params[pbase + b] = params[r * param_bytes_per_row + b];
    if (t0 < 3) out_consts[row * 3 + t0] = consts[r * 3 + t0];
  }
}

}  // namespace
}  // namespace hi2

extern "C" int hi2_pack_codes(const uint8_t* codes, int32_t* words, int64_t rows, int64_t n,
                              int nbits, int32_t* bad, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(nbits == 2 || nbits == 4 || nbits == 8, "pack_codes: nbits must be 2, 4 or 8");
  HI2_REQUIRE(rows >= 0 && n >= 0 && n % (32 / nbits) == 0,
              "pack_codes: the code count is not a multiple of the codes per word");
  const int64_t n_words = rows * (n * nbits / 32);
  if (n_words == 0) return HI2_OK;
  HI2_REQUIRE(codes && words && bad, "pack_codes: null pointer");
  HI2_REQUIRE(aligned16(codes), "pack_codes: codes must be 16-byte aligned");
  int64_t blocks = ceil_div(n_words, 256);
  if (blocks > 148 * 32) blocks = 148 * 32;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (nbits == 2) pack_kernel<2><<<(unsigned)blocks, 256, 0, s>>>(codes, words, n_words, bad);
  if (nbits == 4) pack_kernel<4><<<(unsigned)blocks, 256, 0, s>>>(codes, words, n_words, bad);
  if (nbits == 8) pack_kernel<8><<<(unsigned)blocks, 256, 0, s>>>(codes, words, n_words, bad);
  return check_launch("pack_codes");
}

extern "C" int hi2_assemble_piece(const int64_t* rows, int64_t n_rows, const uint8_t* codes,
                                  const uint8_t* params, const uint16_t* consts, int64_t k,
                                  int nbits, int block, const int64_t* code_off,
                                  const int64_t* param_off, int32_t* out_codes,
                                  uint8_t* out_params, uint16_t* out_consts, int32_t* bad,
                                  void* stream) {
  using namespace hi2;
  HI2_REQUIRE(nbits == 2 || nbits == 4 || nbits == 8, "assemble_piece: nbits must be 2, 4 or 8");
  HI2_REQUIRE(block == 16 || block == 32 || block == 64, "assemble_piece: block must be 16, 32 or 64");
  HI2_REQUIRE(k > 0 && k % 16 == 0 && (k * nbits) % 32 == 0 && k % block == 0,
              "assemble_piece: k does not fit the word or block size");
  if (n_rows == 0) return HI2_OK;
  HI2_REQUIRE(rows && codes && params && consts && code_off && param_off && out_codes &&
                  out_params && out_consts && bad,
              "assemble_piece: null pointer");
  HI2_REQUIRE(aligned16(codes), "assemble_piece: codes must be 16-byte aligned");
  const int64_t words_per_row = k * nbits / 32, pbytes = 2 * (k / block);
  dim3 grid((unsigned)ceil_div(words_per_row > pbytes ? words_per_row : pbytes, 256),
            (unsigned)(n_rows < 32768 ? n_rows : 32768));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define HI2_ASM(NB)                                                                         \
  assemble_kernel<NB><<<grid, 256, 0, s>>>(rows, n_rows, codes, params, consts, k,          \
                                           words_per_row, pbytes, code_off, param_off,      \
                                           out_codes, out_params, out_consts, bad)
  if (nbits == 2) HI2_ASM(2);
  if (nbits == 4) HI2_ASM(4);
  if (nbits == 8) HI2_ASM(8);
#undef HI2_ASM
  return check_launch("assemble_piece");
}
