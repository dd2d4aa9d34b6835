// Second moment S += X^T X on CTA PAIRS (hi2/hessian.py:36-43): the tcgen05 kernel of hessian.cu
// with cta_group::2.
//
// A pair of thread blocks on the two SMs of a TPC computes one 256 x 256 tile of S.  Each block
// loads 128 columns of X for the A side and 128 columns for the B side per 64-token stage (32 KiB
// instead of the 48 KiB a 128 x 256 tile needs for half the flops), so a tensor pipe running at
// full rate asks L2 for 64 instead of 96 bytes per clock and SM, which is what kept the one-block
// kernel at ~3/4 of the pipe.  The leader block issues tcgen05.mma.cta_group::2 (M = 256: rows
// 0..127 accumulate in its tensor memory, rows 128..255 in its peer's; each block supplies its
// half of the N = 256 columns of B), both blocks drain their halves exactly as the one-block
// kernel does (two 256-column accumulators, a drain into fp32 registers every 1024 tokens).
//
// Synchronisation: both producers send their TMA transactions to the LEADER's full barrier (the
// leader posts the expected bytes of both); the MMA thread's commits are multicast to the empty
// and accumulator-full barriers of both blocks; the epilogue warps of both blocks arrive on the
// leader's accumulator-empty barrier.  Every wait is bounded by a clock limit and raises *status;
// a cluster barrier before exit keeps a block's shared memory alive while its peer may still
// signal it.  The loads carry no multicast.
#include <cuda.h>

#include "common.cuh"

namespace hi2 {
namespace {

constexpr int T2 = 256;        // tile side
constexpr int HALF = 128;      // columns of X per block and operand
constexpr int BKT = 64;        // tokens per pipeline stage
constexpr int STAGES = 6;
constexpr int CHUNK_KB = 16;   // stages per tensor-memory accumulation (1024 tokens)
constexpr int BOX_BYTES = 64 * BKT * 2;
constexpr int OP_BYTES = (HALF / 64) * BOX_BYTES;  // 16 KiB
constexpr int STAGE_BYTES = 2 * OP_BYTES;          // 32 KiB
constexpr int THREADS = 320;   // warps 0..7 epilogue, warp 8 TMA, warp 9 MMA
constexpr int TILE_ELEMS = T2 * T2;
constexpr int BAND = 8;        // row blocks per band of the tile schedule
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;  // about one second

struct Control {
  unsigned long long full[STAGES];
  unsigned long long empty[STAGES];
  unsigned long long acc_full[2];
  unsigned long long acc_empty[2];
  unsigned int tmem_base;
  volatile unsigned int abort;
};
constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + sizeof(Control) + 1024;

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address of the same shared-memory object in block `rank` of the cluster.
__device__ __forceinline__ uint32_t in_rank(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void bar_init(unsigned long long* b, uint32_t n) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(b)), "r"(n));
}
__device__ __forceinline__ void bar_expect(unsigned long long* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool bar_try(unsigned long long* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(s32(b)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  False when the limit ran out or another role of this block already gave up.
__device__ __forceinline__ bool bar_wait(unsigned long long* b, uint32_t parity, Control* ctl, int* status) {
  if (bar_try(b, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (bar_try(b, parity)) return true;
    if (ctl->abort) return false;
    if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
      ctl->abort = 1;
      atomicExch(status, HI2_ERR_TIMEOUT);
      return false;
    }
  }
}
// One box into this block's shared memory; the transaction bytes go to the barrier at
// `bar_cluster_addr`, which may belong to the peer block of the pair.
__device__ __forceinline__ void tma_load_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x,
                                              int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(s32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
// MN-major, 128-byte-swizzled operand: 64-element (128 B) pieces along M/N are BOX_BYTES apart
// (leading offset), groups of 8 tokens 1024 B apart (stride offset); version 1, SWIZZLE_128B.
__device__ __forceinline__ uint64_t operand_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)(BOX_BYTES >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16: D fp32 (1 << 4), A/B format (0 fp16, 1 bf16) at bits 7 and 10, A and B MN-major
// (bits 15, 16), N >> 3 at bit 17, M >> 4 at bit 24; M = N = 256 for the pair.
__host__ __device__ constexpr uint32_t instr_desc(int fmt) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | (1u << 15) | (1u << 16) |
         ((uint32_t)(T2 >> 3) << 17) | ((uint32_t)(T2 >> 4) << 24);
}
__device__ __forceinline__ void mma_pair(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(da), "l"(db), "r"(idesc), "r"(acc)
      : "memory");
}
// Arrives on the barrier at this offset in BOTH blocks once the MMAs issued so far have finished.
__device__ __forceinline__ void commit_both(unsigned long long* b) {
  const unsigned short mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          s32(b)),
      "h"(mask)
      : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
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

struct Params {
  float* scratch;   // [splits][tiles][256][256]
  int* status;      // device int, raised on a wait that ran out
  int64_t kblocks;  // ceil(tokens / BKT)
  int splits;
  int tiles;
  int nb;           // 256-wide blocks of S per side
  int fmt;          // 0 fp16, 1 bf16
};

// Scratch slot of tile (I, J), I <= J, row-major over the upper triangle.
__host__ __device__ __forceinline__ int tile_slot(int i, int j, int nb) { return i * nb - i * (i - 1) / 2 + (j - i); }

// Schedule position -> (I, J): bands of BAND row blocks, column block by column block inside a
// band, so the tiles in flight at one time share a few thousand columns of X in L2.
__device__ __forceinline__ void decode_tile(int pos, int nb, int& ti, int& tj) {
  for (int i0 = 0; i0 < nb; i0 += BAND) {
    const int rows = (nb - i0 < BAND) ? nb - i0 : BAND;
    for (int j = i0; j < nb; ++j) {
      int cnt = j - i0 + 1;
      if (cnt > rows) cnt = rows;
      if (pos < cnt) {
        ti = i0 + pos, tj = j;
        return;
      }
      pos -= cnt;
    }
  }
  ti = 0, tj = 0;  // not reached: pos < tiles
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
hessian_pair_kernel(const __grid_constant__ CUtensorMap map, const Params p) {
  extern __shared__ uint8_t raw_smem[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~(uintptr_t)1023);
  Control* ctl = reinterpret_cast<Control*>(smem + (size_t)STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cta_rank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) bar_init(&ctl->full[s], 1), bar_init(&ctl->empty[s], 1);
    for (int b = 0; b < 2; ++b) bar_init(&ctl->acc_full[b], 1), bar_init(&ctl->acc_empty[b], 16);
    ctl->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&ctl->tmem_base)),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  cluster_sync();  // the peer's barriers exist before anything signals them
  fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const int items = p.tiles * p.splits;

  if (warp == 8 && lane == 0) {
    // ---------------------------------------------------------------- TMA producer (both blocks)
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int item = pair; item < items && ok; item += pairs) {
      const int split = item / p.tiles;
      int ti, tj;
      decode_tile(item % p.tiles, p.nb, ti, tj);
      const int xa = ti * T2 + (int)rank * HALF, xb = tj * T2 + (int)rank * HALF;
      const int64_t kb0 = p.kblocks * split / p.splits, kb1 = p.kblocks * (split + 1) / p.splits;
      for (int64_t kb = kb0; kb < kb1; ++kb) {
        if (!(ok = bar_wait(&ctl->empty[stage], phase ^ 1, ctl, p.status))) break;
        if (rank == 0) bar_expect(&ctl->full[stage], 2 * STAGE_BYTES);  // both blocks' bytes
        const uint32_t full = in_rank(s32(&ctl->full[stage]), 0);
        uint8_t* dst = smem + (size_t)stage * STAGE_BYTES;
        const int y = (int)(kb * BKT);
#pragma unroll
        for (int c = 0; c < HALF / 64; ++c) {
          tma_load_pair(dst + c * BOX_BYTES, &map, full, xa + c * 64, y);
          tma_load_pair(dst + OP_BYTES + c * BOX_BYTES, &map, full, xb + c * 64, y);
        }
        if (++stage == STAGES) stage = 0, phase ^= 1;
      }
    }
    if (!ok) {
      // copies already issued still land in this block's shared memory: give them time
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000LL) {
      }
    }
  } else if (warp == 9 && lane == 0 && rank == 0) {
    // ---------------------------------------------------------------- MMA issuer (leader only)
    const uint32_t idesc = instr_desc(p.fmt);
    int stage = 0;
    uint32_t phase = 0, chunk_no = 0;
    bool ok = true;
    for (int item = pair; item < items && ok; item += pairs) {
      const int split = item / p.tiles;
      const int64_t kb0 = p.kblocks * split / p.splits, kb1 = p.kblocks * (split + 1) / p.splits;
      for (int64_t c0 = kb0; c0 < kb1 && ok; c0 += CHUNK_KB, ++chunk_no) {
        const int buf = chunk_no & 1;
        if (!(ok = bar_wait(&ctl->acc_empty[buf], ((chunk_no >> 1) & 1) ^ 1, ctl, p.status))) break;
        fence_after();
        const int64_t c1 = (c0 + CHUNK_KB < kb1) ? c0 + CHUNK_KB : kb1;
        for (int64_t kb = c0; kb < c1; ++kb) {
          if (!(ok = bar_wait(&ctl->full[stage], phase, ctl, p.status))) break;
          fence_after();
          const uint32_t sa = s32(smem + (size_t)stage * STAGE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BKT / 16; ++kk) {
            const uint64_t da = operand_desc(sa + kk * 2048);
            const uint64_t db = operand_desc(sa + OP_BYTES + kk * 2048);
            mma_pair(tmem_base + buf * T2, da, db, idesc, (kb > c0 || kk > 0) ? 1u : 0u);
          }
          commit_both(&ctl->empty[stage]);  // frees the stage in both blocks once these MMAs have read it
          if (++stage == STAGES) stage = 0, phase ^= 1;
        }
        if (ok) commit_both(&ctl->acc_full[buf]);
      }
    }
  } else if (warp < 8) {
    // ---------------------------------------------------------------- epilogue (both blocks)
    // a warp may only touch the 32 tensor-memory lanes of its index modulo 4
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;
    uint32_t chunk_no = 0;
    bool ok = true;
    for (int item = pair; item < items && ok; item += pairs) {
      const int split = item / p.tiles;
      const int64_t kb0 = p.kblocks * split / p.splits, kb1 = p.kblocks * (split + 1) / p.splits;
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
      for (int64_t c0 = kb0; c0 < kb1 && ok; c0 += CHUNK_KB, ++chunk_no) {
        const int buf = chunk_no & 1;
        if (!(ok = bar_wait(&ctl->acc_full[buf], (chunk_no >> 1) & 1, ctl, p.status))) break;
        fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * T2 + half * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float v[16];
          tmem_load16(taddr + c * 16, v);
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[c * 16 + i] += v[i];
        }
        fence_before();
        __syncwarp();
        if (lane == 0) bar_arrive_cluster(in_rank(s32(&ctl->acc_empty[buf]), 0));
      }
      if (ok) {
        int ti, tj;
        decode_tile(item % p.tiles, p.nb, ti, tj);
        const size_t slot = (size_t)split * p.tiles + tile_slot(ti, tj, p.nb);
        float* dst = p.scratch + slot * TILE_ELEMS + (size_t)(rank * HALF + row) * T2 + half * 128;
#pragma unroll
        for (int i = 0; i < 128; i += 4)
          *reinterpret_cast<float4*>(dst + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
      }
    }
  }

  fence_before();
  __syncthreads();
  cluster_sync();  // neither block leaves while its peer may still signal it or read its operands
  if (warp == 9) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// S[i][j] += sum over splits (ascending) of the item tiles, for i <= j; S[j][i] = S[i][j].
__global__ void __launch_bounds__(256)
pair_reduce_kernel(const float* __restrict__ scratch, int splits, int tiles, int nb, int64_t k,
                   float* __restrict__ s, const int* __restrict__ status) {
  // a product that gave up on a bounded wait left stale or partial tiles: S stays as it was and the
  // caller sees the status word
  if (*status != 0) return;
  const int64_t j = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t i = blockIdx.y;
  if (j >= k || j < i) return;
  const int tile = tile_slot((int)(i / T2), (int)(j / T2), nb);
  const size_t off = (size_t)tile * TILE_ELEMS + (size_t)(i % T2) * T2 + (size_t)(j % T2);
  float sum = 0.0f;
  for (int sp = 0; sp < splits; ++sp) sum += scratch[(size_t)sp * tiles * TILE_ELEMS + off];
  const float v = s[i * k + j] + sum;
  s[i * k + j] = v;
  if (i != j) s[j * k + i] = v;
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encoder() {
  static EncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(ptr);
  }
  return fn;
}

struct Plan {
  int tiles, nb, splits;
  int64_t kblocks;
  size_t scratch_bytes;
};

// Token splits: the number s that minimises the waves per split, ceil(tiles * s / pairs) / s, with
// at least 4096 tokens per item and at most 512 MiB of item tiles.
Plan plan(int64_t tokens, int64_t k, int pairs) {
  Plan pl;
  pl.nb = (int)ceil_div(k, (int64_t)T2);
  pl.tiles = pl.nb * (pl.nb + 1) / 2;
  pl.kblocks = ceil_div(tokens, (int64_t)BKT);
  int64_t cap = pl.kblocks / 64;
  if (cap < 1) cap = 1;
  const size_t tile_bytes = (size_t)TILE_ELEMS * sizeof(float);
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= 16 && s <= cap; ++s) {
    if (s > 1 && (size_t)s * pl.tiles * tile_bytes > ((size_t)512 << 20)) break;
    const double cost = (double)ceil_div((int64_t)pl.tiles * s, (int64_t)pairs) / s;
    if (cost < best_cost * 0.995) best_cost = cost, best = s;
  }
  pl.splits = best;
  pl.scratch_bytes = (size_t)pl.splits * pl.tiles * tile_bytes;
  return pl;
}

int pair_count() {
  int device = 0, sms = 148;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  return sms / 2;
}

}  // namespace

// Used by hessian.cu.
size_t pair_workspace_bytes(int64_t tokens, int64_t k) { return plan(tokens, k, pair_count()).scratch_bytes + 256; }

int accumulate_pair(const void* x, int dtype, int64_t tokens, int64_t k, float* s, void* workspace,
                    size_t workspace_bytes, cudaStream_t stream) {
  const int pairs = pair_count();
  const Plan pl = plan(tokens, k, pairs);
  if (workspace == nullptr || workspace_bytes < pl.scratch_bytes + 256)
    return fail(HI2_ERR_WORKSPACE, "hessian_accumulate: workspace too small");
  EncodeFn enc = encoder();
  if (enc == nullptr) return fail(HI2_ERR_DRIVER, "hessian_accumulate: cuTensorMapEncodeTiled unavailable");
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)tokens};
  const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)BKT};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&map, dtype == HI2_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                   const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("hessian_accumulate: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return HI2_ERR_DRIVER;
  }
  if (cudaFuncSetAttribute(hessian_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) !=
      cudaSuccess)
    return fail(HI2_ERR_LAUNCH, "hessian_accumulate: cannot reserve shared memory");
  int* status = static_cast<int*>(workspace);
  float* scratch = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256);
  if (cudaMemsetAsync(status, 0, sizeof(int), stream) != cudaSuccess)
    return fail(HI2_ERR_LAUNCH, "hessian_accumulate: memset failed");
  Params p;
  p.scratch = scratch, p.status = status, p.kblocks = pl.kblocks;
  p.splits = pl.splits, p.tiles = pl.tiles, p.nb = pl.nb, p.fmt = dtype == HI2_BF16 ? 1 : 0;
  const int items = pl.tiles * pl.splits;
  const int grid = 2 * (items < pairs ? items : pairs);
  hessian_pair_kernel<<<grid, THREADS, SMEM, stream>>>(map, p);
  int rc = check_launch("hessian_accumulate (tcgen05 pair)");
  if (rc != HI2_OK) return rc;
  dim3 rgrid((unsigned)ceil_div(k, (int64_t)256), (unsigned)k);
  pair_reduce_kernel<<<rgrid, 256, 0, stream>>>(scratch, pl.splits, pl.tiles, pl.nb, k, s, status);
  return check_launch("hessian_accumulate (reduce)");
}

}  // namespace hi2
