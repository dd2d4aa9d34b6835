// Calibration second moment S += X^T X (hi2/hessian.py:35-40).
//
// 16-bit activations (bf16 / fp16; their products are exact in fp32) go through a TMA-fed
// tcgen05 kernel with fp32 accumulation in tensor memory:
//
//   * X is [tokens, k] row-major, so both operands of X^T X are "MN-major": the reduction index
//     (token) is the slow one.  One TMA box is 64 columns x 64 tokens (128-byte rows, 128-byte
//     swizzle); an A tile is two boxes (128 columns), a B tile four (256 columns), a pipeline
//     stage 48 KiB, four stages.  The MMA is 128 x 256 x 16 (cta_group::1, kind::f16), four per
//     stage, descriptors advanced by 2 KiB per 16 tokens.
//   * Only tiles that touch the upper triangle are computed; the strict lower triangle is
//     mirrored afterwards, so S is exactly symmetric.
//   * A work item is (tile, token split).  Items are ordered split-major, and inside a split in
//     bands of 16 row blocks (decode_tile), so the CTAs resident at one time read the same token
//     range of a few thousand columns and X streams through L2 about once per wave.
//   * Tensor-memory accumulation runs over 1024 tokens at a time into one of two 256-column
//     buffers; eight epilogue warps drain a finished buffer into fp32 REGISTER accumulators
//     (round-to-nearest adds) while the next 1024 tokens accumulate in the other buffer.  This
//     bounds whatever rounding the tensor-core accumulator applies to 64 steps.
//   * A finished item is written to caller scratch; a second kernel adds the splits in a fixed
//     order into S and mirrors.  No atomics: the result does not depend on scheduling.
//   * Every mbarrier wait is bounded by a clock limit; on expiry the CTA raises *status, stops
//     issuing work, frees its tensor memory and returns.
//
// fp32 activations (whose products are not exact in 16-bit operands) and small problems take the
// fp32 FMA product of gemm.cuh.
#include <cuda.h>

#include <mutex>

#include "gemm.cuh"

namespace hi2 {

// hessian2.cu: the same product on pairs of thread blocks (256 x 256 tiles, cta_group::2)
size_t pair_workspace_bytes(int64_t tokens, int64_t k);
int accumulate_pair(const void* x, int dtype, int64_t tokens, int64_t k, float* s, void* workspace,
                    size_t workspace_bytes, cudaStream_t stream);

namespace {

constexpr int BM = 128;       // output rows per tile (columns of X on the A side)
constexpr int BN = 256;       // output columns per tile
constexpr int BKT = 64;       // tokens per pipeline stage
constexpr int STAGES = 4;
constexpr int CHUNK_KB = 16;  // stages per tensor-memory accumulation (1024 tokens)
constexpr int BOX_BYTES = 64 * BKT * 2;
constexpr int A_BYTES = (BM / 64) * BOX_BYTES;
constexpr int STAGE_BYTES = A_BYTES + (BN / 64) * BOX_BYTES;
constexpr int TC_THREADS = 320;  // warps 0..7 epilogue, warp 8 TMA, warp 9 MMA
constexpr int TILE_ELEMS = BM * BN;
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;  // about one second

struct Control {
  unsigned long long full[STAGES];
  unsigned long long empty[STAGES];
  unsigned long long acc_full[2];
  unsigned long long acc_empty[2];
  unsigned int tmem_base;
  volatile unsigned int abort;
};

constexpr size_t TC_SMEM = (size_t)STAGES * STAGE_BYTES + sizeof(Control) + 1024;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(unsigned long long* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  False when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, uint32_t parity, Control* ctl,
                                          int* status) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try(bar, parity)) return true;
    if (ctl->abort) return false;
    if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
      ctl->abort = 1;
      atomicExch(status, HI2_ERR_TIMEOUT);
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map,
                                            unsigned long long* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory matrix descriptor of an MN-major, 128-byte-swizzled operand: 64-element (128 B)
// pieces along M/N are BOX_BYTES apart (leading offset), groups of 8 tokens 1024 B apart (stride
// offset); descriptor version 1, layout type 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t operand_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)(BOX_BYTES >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor, kind::f16: D fp32 (1 << 4), A/B format (0 fp16, 1 bf16) at bits 7 and
// 10, A and B MN-major (bits 15, 16), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t instr_desc(int fmt) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | (1u << 15) | (1u << 16) |
         ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_load16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

struct TcParams {
  float* scratch;   // [splits][tiles][BM][BN]
  int* status;      // device int, raised on a wait that ran out
  int64_t k;        // columns of X
  int64_t kblocks;  // ceil(tokens / BKT)
  int splits;
  int tiles;
  int nib;          // row blocks: ceil(k / BM)
  int njb;          // column blocks: ceil(k / BN)
  int fmt;          // 0 fp16, 1 bf16
};

// Scratch slot of tile (row block ib, column block jb) over the tiles that touch the upper
// triangle, row-major: row block ib owns column blocks floor(ib / 2) .. njb - 1.
__host__ __device__ __forceinline__ int tile_slot(int ib, int jb, int njb) {
  const int half = ib >> 1;
  return ib * njb - (half * (half - 1) + ((ib & 1) ? half : 0)) + (jb - half);
}

// Schedule position -> (row block, column block).  Tiles are visited in bands of BAND row blocks,
// column block by column block inside a band, so that the ~148 tiles in flight at any moment
// cover about BAND x 128 + (148 / BAND) x 256 columns of X instead of all of them: with K = 11008
// a token of X is 22 KB, and the CTAs' token positions drift apart by thousands of tokens, so the
// row-major order overflowed L2 and ran at the speed of HBM.
#ifndef HI2_HESSIAN_BAND
#define HI2_HESSIAN_BAND 16
#endif
constexpr int BAND = HI2_HESSIAN_BAND;
__device__ __forceinline__ void decode_tile(int pos, int nib, int njb, int& ib, int& jb) {
  for (int i0 = 0; i0 < nib; i0 += BAND) {
    const int rows = (nib - i0 < BAND) ? nib - i0 : BAND;
    for (int j = i0 >> 1; j < njb; ++j) {
      // row blocks of the band with floor(ib / 2) <= j, i.e. ib <= 2 j + 1
      int cnt = 2 * j + 2 - i0;
      if (cnt > rows) cnt = rows;
      if (pos < cnt) {
        ib = i0 + pos;
        jb = j;
        return;
      }
      pos -= cnt;
    }
  }
  ib = 0, jb = 0;  // not reached: pos < tiles
}

// Ten warps: the register file is four partitions of 16384, so two partitions hold three warps
// and a thread gets at most 16384 / (3 * 32) -> 168 registers (128 of them accumulators).
__global__ void __launch_bounds__(TC_THREADS, 1)
hessian_tc_kernel(const __grid_constant__ CUtensorMap map, const TcParams p) {
  extern __shared__ uint8_t raw_smem[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                             ~(uintptr_t)1023);
  Control* ctl = reinterpret_cast<Control*>(smem + (size_t)STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(&ctl->full[s], 1), mbar_init(&ctl->empty[s], 1);
    for (int b = 0; b < 2; ++b) mbar_init(&ctl->acc_full[b], 1), mbar_init(&ctl->acc_empty[b], 8);
    ctl->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&ctl->tmem_base)),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const int items = p.tiles * p.splits;

  if (warp == 8 && lane == 0) {
    // ---------------------------------------------------------------- TMA producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const int split = item / p.tiles;
      int ib, jb;
      decode_tile(item % p.tiles, p.nib, p.njb, ib, jb);
      const int64_t kb0 = p.kblocks * split / p.splits, kb1 = p.kblocks * (split + 1) / p.splits;
      for (int64_t kb = kb0; kb < kb1; ++kb) {
        if (!(ok = mbar_wait(&ctl->empty[stage], phase ^ 1, ctl, p.status))) break;
        mbar_expect_tx(&ctl->full[stage], STAGE_BYTES);
        uint8_t* dst = smem + (size_t)stage * STAGE_BYTES;
        const int y = (int)(kb * BKT);
#pragma unroll
        for (int c = 0; c < BM / 64; ++c)
          tma_load_2d(dst + c * BOX_BYTES, &map, &ctl->full[stage], ib * BM + c * 64, y);
#pragma unroll
        for (int c = 0; c < BN / 64; ++c)
          tma_load_2d(dst + A_BYTES + c * BOX_BYTES, &map, &ctl->full[stage], jb * BN + c * 64, y);
        if (++stage == STAGES) stage = 0, phase ^= 1;
      }
    }
    if (!ok) {
      // copies already issued still land in this CTA's shared memory: give them time
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000LL) {
      }
    }
  } else if (warp == 9 && lane == 0) {
    // ---------------------------------------------------------------- MMA issuer
    const uint32_t idesc = instr_desc(p.fmt);
    int stage = 0;
    uint32_t phase = 0, chunk_no = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const int split = item / p.tiles;
      const int64_t kb0 = p.kblocks * split / p.splits, kb1 = p.kblocks * (split + 1) / p.splits;
      for (int64_t c0 = kb0; c0 < kb1 && ok; c0 += CHUNK_KB, ++chunk_no) {
        const int buf = chunk_no & 1;
        if (!(ok = mbar_wait(&ctl->acc_empty[buf], ((chunk_no >> 1) & 1) ^ 1, ctl, p.status))) break;
        tc_fence_after();
        const int64_t c1 = (c0 + CHUNK_KB < kb1) ? c0 + CHUNK_KB : kb1;
        for (int64_t kb = c0; kb < c1; ++kb) {
          if (!(ok = mbar_wait(&ctl->full[stage], phase, ctl, p.status))) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + (size_t)stage * STAGE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BKT / 16; ++kk) {
            const uint64_t da = operand_desc(sa + kk * 2048);
            const uint64_t db = operand_desc(sa + A_BYTES + kk * 2048);
            mma_f16(tmem_base + buf * BN, da, db, idesc, (kb > c0 || kk > 0) ? 1u : 0u);
          }
          mma_commit(&ctl->empty[stage]);  // frees the stage once these MMAs have read it
          if (++stage == STAGES) stage = 0, phase ^= 1;
        }
        if (ok) mma_commit(&ctl->acc_full[buf]);
      }
    }
  } else if (warp < 8) {
    // ---------------------------------------------------------------- epilogue
    // a warp may only touch the 32 tensor-memory lanes of its index modulo 4
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;
    uint32_t chunk_no = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const int split = item / p.tiles;
      const int64_t kb0 = p.kblocks * split / p.splits, kb1 = p.kblocks * (split + 1) / p.splits;
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
      for (int64_t c0 = kb0; c0 < kb1 && ok; c0 += CHUNK_KB, ++chunk_no) {
        const int buf = chunk_no & 1;
        if (!(ok = mbar_wait(&ctl->acc_full[buf], (chunk_no >> 1) & 1, ctl, p.status))) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + half * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float v[16];
          tmem_load16(taddr + c * 16, v);
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[c * 16 + i] += v[i];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
      }
      if (ok) {
        int ib, jb;
        decode_tile(item % p.tiles, p.nib, p.njb, ib, jb);
        const size_t slot = (size_t)split * p.tiles + tile_slot(ib, jb, p.njb);
        float* dst = p.scratch + slot * TILE_ELEMS + (size_t)row * BN + half * 128;
#pragma unroll
        for (int i = 0; i < 128; i += 4)
          *reinterpret_cast<float4*>(dst + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512)
                 : "memory");
  }
}

// S[i][j] += sum over splits (ascending) of the item tiles, for i <= j; S[j][i] = S[i][j].
__global__ void __launch_bounds__(256)
hessian_reduce_kernel(const float* __restrict__ scratch, int splits, int tiles, int njb, int64_t k,
                      float* __restrict__ s, const int* __restrict__ status) {
  // a product that gave up on a bounded wait left stale or partial tiles: S stays as it was and the
  // caller sees the status word
  if (*status != 0) return;
  const int64_t j = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t i = blockIdx.y;
  if (j >= k || j < i) return;
  const int ib = (int)(i / BM), jb = (int)(j / BN);
  const int tile = tile_slot(ib, jb, njb);
  const size_t off = (size_t)tile * TILE_ELEMS + (size_t)(i % BM) * BN + (size_t)(j % BN);
  float sum = 0.0f;
  for (int sp = 0; sp < splits; ++sp) sum += scratch[(size_t)sp * tiles * TILE_ELEMS + off];
  const float v = s[i * k + j] + sum;
  s[i * k + j] = v;
  if (i != j) s[j * k + i] = v;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

struct TcPlan {
  int tiles, njb, splits;
  int64_t kblocks;
  size_t scratch_bytes;
};

TcPlan plan_tc(int64_t tokens, int64_t k) {
  TcPlan pl;
  const int nib = (int)ceil_div(k, BM);
  pl.njb = (int)ceil_div(k, BN);
  int tiles = 0;
  for (int ib = 0; ib < nib; ++ib) tiles += pl.njb - (ib >> 1);
  pl.tiles = tiles;
  pl.kblocks = ceil_div(tokens, BKT);
  // enough items for a few waves of 148 CTAs, but at least 64 stages (4096 tokens) per item
  int64_t want = ceil_div((int64_t)148 * 6, tiles);
  int64_t cap = pl.kblocks / 64;
  if (cap < 1) cap = 1;
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  pl.splits = (int)want;
  pl.scratch_bytes = (size_t)pl.splits * tiles * TILE_ELEMS * sizeof(float);
  return pl;
}

bool use_tc(int dtype, int64_t tokens, int64_t k) {
  return (dtype == HI2_BF16 || dtype == HI2_F16) && k >= 256 && tokens >= 256;
}
// Large problems go to the pair kernel: its 256 x 256 tiles want a few tiles per SM pair and
// thousands of tokens per item.  Beyond K = 8192 the 74 tiles in flight cover so many columns
// that they fall out of step in L2 (DRAM reads of 10.9 x X at K = 11008 against 6.2 x for 148
// one-block tiles, same time, less stable), so the widest inputs stay with the one-block kernel.
bool use_pair(int dtype, int64_t tokens, int64_t k) {
  return use_tc(dtype, tokens, k) && k >= 1024 && k <= 8192 && tokens >= 8192;
}

int accumulate_tc(const void* x, int dtype, int64_t tokens, int64_t k, float* s, void* workspace,
                  size_t workspace_bytes, cudaStream_t stream) {
  const TcPlan pl = plan_tc(tokens, k);
  const size_t need = pl.scratch_bytes + 256;
  if (workspace == nullptr || workspace_bytes < need)
    return fail(HI2_ERR_WORKSPACE, "hessian_accumulate: workspace too small");
  EncodeTiledFn enc = encode_tiled();
  if (enc == nullptr) return fail(HI2_ERR_DRIVER, "hessian_accumulate: cuTensorMapEncodeTiled unavailable");
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)tokens};
  const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
  const cuuint32_t box[2] = {64, BKT};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&map, dtype == HI2_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                   2, const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("hessian_accumulate: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return HI2_ERR_DRIVER;
  }
  {  // per device, so not cached: a process may drive several
    if (cudaFuncSetAttribute(hessian_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)TC_SMEM) != cudaSuccess)
      return fail(HI2_ERR_LAUNCH, "hessian_accumulate: cannot reserve shared memory");
  }
  // first 256 bytes of the workspace: the status word; the item tiles follow
  int* status = static_cast<int*>(workspace);
  float* scratch = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256);
  if (cudaMemsetAsync(status, 0, sizeof(int), stream) != cudaSuccess)
    return fail(HI2_ERR_LAUNCH, "hessian_accumulate: memset failed");
  TcParams p;
  p.scratch = scratch, p.status = status, p.k = k, p.kblocks = pl.kblocks;
  p.splits = pl.splits, p.tiles = pl.tiles, p.njb = pl.njb, p.nib = (int)ceil_div(k, BM), p.fmt = dtype == HI2_BF16 ? 1 : 0;
  const int items = pl.tiles * pl.splits;
  int device = 0, sms = 148;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int grid = items < sms ? items : sms;
  hessian_tc_kernel<<<grid, TC_THREADS, TC_SMEM, stream>>>(map, p);
  int rc = check_launch("hessian_accumulate (tcgen05)");
  if (rc != HI2_OK) return rc;
  dim3 rgrid((unsigned)ceil_div(k, 256), (unsigned)k);
  hessian_reduce_kernel<<<rgrid, 256, 0, stream>>>(scratch, pl.splits, pl.tiles, pl.njb, k, s, status);
  return check_launch("hessian_accumulate (reduce)");
}

template <typename TX>
int accumulate_fma(const void* x, int64_t tokens, int64_t k, float* s, cudaStream_t stream) {
  GemmArgs<float, TX, TX> p;
  p.m = k, p.n = k, p.kk = tokens, p.alpha = 1.0f, p.beta = 1.0f;
  p.a = static_cast<const TX*>(x), p.lda = k, p.b = static_cast<const TX*>(x), p.ldb = k;
  p.c = s, p.ldc = k, p.flags = 0;
  return launch_gemm<float, TX, TX, 8, 8, 8>(true, false, p, stream, "hessian_accumulate (fma)");
}

}  // namespace
}  // namespace hi2

extern "C" size_t hi2_hessian_workspace_bytes(int64_t tokens, int64_t k, int dtype) {
  using namespace hi2;
  if (tokens <= 0 || k <= 0 || !use_tc(dtype, tokens, k)) return 0;
  if (use_pair(dtype, tokens, k)) return pair_workspace_bytes(tokens, k);
  return plan_tc(tokens, k).scratch_bytes + 256;
}

extern "C" int hi2_hessian_status(const void* workspace, int* status_host) {
  // Reads the status word a tcgen05 launch left in its workspace (synchronises the device).
  using namespace hi2;
  HI2_REQUIRE(workspace && status_host, "hessian_status: null pointer");
  if (cudaMemcpy(status_host, workspace, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return fail(HI2_ERR_LAUNCH, "hessian_status: copy failed");
  return HI2_OK;
}

extern "C" int hi2_hessian_accumulate(const void* x, int dtype, int64_t tokens, int64_t k, float* s,
                                      void* workspace, size_t workspace_bytes, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(k > 0 && k % 16 == 0, "hessian_accumulate: k must be a positive multiple of 16");
  HI2_REQUIRE(tokens >= 0, "hessian_accumulate: negative token count");
  if (tokens == 0) return HI2_OK;
  HI2_REQUIRE(x && s, "hessian_accumulate: null pointer");
  HI2_REQUIRE(aligned16(x) && aligned16(s), "hessian_accumulate: x and s must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (use_pair(dtype, tokens, k)) return accumulate_pair(x, dtype, tokens, k, s, workspace, workspace_bytes, st);
  if (use_tc(dtype, tokens, k))
    return accumulate_tc(x, dtype, tokens, k, s, workspace, workspace_bytes, st);
  if (dtype == HI2_BF16) return accumulate_fma<__nv_bfloat16>(x, tokens, k, s, st);
  if (dtype == HI2_F16) return accumulate_fma<__half>(x, tokens, k, s, st);
  if (dtype == HI2_F32) return accumulate_fma<float>(x, tokens, k, s, st);
  return fail(HI2_ERR_ARG, "hessian_accumulate: dtype must be F16, BF16 or F32");
}

// --------------------------------------------------------------------------------------------
// Second moment without any allocation: the item tiles live in a fixed device array.
//
// Some callers cannot allocate device memory at the point where calibration statistics are
// taken: a forward hook that runs while another framework's caching allocator owns the device
// (an allocation there can synchronise or fragment the host framework's pool), a thread that
// must not call into the CUDA allocator because a stream capture is in progress elsewhere in
// the process, or an embedding whose memory budget was fixed up front.  For them the item tiles
// of the tensor-core kernel are kept in g_static_tiles below: 64 MiB that every GPU loading the
// library holds until the process exits.  That bounds the problem: tiles(k) * 128 KiB must fit,
// which admits K up to 5632 (K = 4096 needs 34 MiB); the token split is reduced until the items
// fit, so very few tokens per item are never needed.
//
// g_static_tiles is a device symbol: in host code its name is only a handle.  The address the
// kernels receive comes from cudaGetSymbolAddress, looked up once per device with that device
// current (first call on the device; make that call before any stream capture begins).  Every
// call shares the array and the array keeps the previous call's tiles: each call overwrites all
// tiles it later reads, and clears the caller's status word.  Two calls that overlap on the GPU
// (different streams, or different host threads on one device) race on the array.
// --------------------------------------------------------------------------------------------
namespace hi2 {
namespace {

constexpr size_t STATIC_TILE_BYTES = (size_t)64 << 20;
constexpr int STATIC_MAX_TILES = (int)(STATIC_TILE_BYTES / (TILE_ELEMS * sizeof(float)));  // 512
constexpr int MAX_DEVICES = 64;

static __device__ __align__(256) float g_static_tiles[STATIC_TILE_BYTES / sizeof(float)];

float* static_tiles_address(int device) {
  static float* cache[MAX_DEVICES] = {nullptr};
  static std::mutex lock;
  if (device < 0 || device >= MAX_DEVICES) return nullptr;
  std::lock_guard<std::mutex> guard(lock);
  if (cache[device] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_tiles) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    cache[device] = p;
  }
  return cache[device];
}

}  // namespace
}  // namespace hi2

extern "C" int hi2_hessian_accumulate_noalloc(const void* x, int dtype, int64_t tokens, int64_t k,
                                              float* s, int32_t* status, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(k > 0 && k % 16 == 0, "hessian_accumulate_noalloc: k must be a positive multiple of 16");
  HI2_REQUIRE(dtype == HI2_BF16 || dtype == HI2_F16,
              "hessian_accumulate_noalloc: activations must be bf16 or fp16");
  HI2_REQUIRE(tokens >= 256 && k >= 256,
              "hessian_accumulate_noalloc: needs at least 256 tokens and 256 columns");
  HI2_REQUIRE(x && s && status, "hessian_accumulate_noalloc: null pointer");
  HI2_REQUIRE(aligned16(x) && aligned16(s), "hessian_accumulate_noalloc: x and s must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  TcPlan pl = plan_tc(tokens, k);
  if (pl.tiles > STATIC_MAX_TILES) {
    set_error("hessian_accumulate_noalloc: k = %lld needs %d tiles of 128 KiB, the fixed scratch holds %d "
              "(k <= 5632); use hi2_hessian_accumulate with a workspace",
              (long long)k, pl.tiles, STATIC_MAX_TILES);
    return HI2_ERR_WORKSPACE;
  }
  if (pl.splits > STATIC_MAX_TILES / pl.tiles) pl.splits = STATIC_MAX_TILES / pl.tiles;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return fail(HI2_ERR_LAUNCH, "hessian_accumulate_noalloc: no device");
  float* tiles = static_tiles_address(device);
  if (tiles == nullptr)
    return fail(HI2_ERR_LAUNCH, "hessian_accumulate_noalloc: cudaGetSymbolAddress failed for the scratch array");
  EncodeTiledFn enc = encode_tiled();
  if (enc == nullptr)
    return fail(HI2_ERR_DRIVER, "hessian_accumulate_noalloc: cuTensorMapEncodeTiled unavailable");
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)tokens};
  const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
  const cuuint32_t box[2] = {64, BKT};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&map, dtype == HI2_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                   2, const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("hessian_accumulate_noalloc: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return HI2_ERR_DRIVER;
  }
  if (cudaFuncSetAttribute(hessian_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM) !=
      cudaSuccess)
    return fail(HI2_ERR_LAUNCH, "hessian_accumulate_noalloc: cannot reserve shared memory");
  if (cudaMemsetAsync(status, 0, sizeof(int32_t), st) != cudaSuccess)  // must start at zero
    return fail(HI2_ERR_LAUNCH, "hessian_accumulate_noalloc: memset failed");
  TcParams p;
  p.scratch = tiles, p.status = reinterpret_cast<int*>(status), p.k = k, p.kblocks = pl.kblocks;
  p.splits = pl.splits, p.tiles = pl.tiles, p.njb = pl.njb, p.nib = (int)ceil_div(k, BM), p.fmt = dtype == HI2_BF16 ? 1 : 0;
  const int items = pl.tiles * pl.splits;
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  hessian_tc_kernel<<<items < sms ? items : sms, TC_THREADS, TC_SMEM, st>>>(map, p);
  int rc = check_launch("hessian_accumulate_noalloc (tcgen05)");
  if (rc != HI2_OK) return rc;
  dim3 rgrid((unsigned)ceil_div(k, 256), (unsigned)k);
  hessian_reduce_kernel<<<rgrid, 256, 0, st>>>(tiles, pl.splits, pl.tiles, pl.njb, k, s,
                                               reinterpret_cast<const int*>(status));
  return check_launch("hessian_accumulate_noalloc (reduce)");
}
