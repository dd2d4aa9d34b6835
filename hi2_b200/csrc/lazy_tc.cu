// GPTQ trailing update on the tensor cores with fp32-grade accuracy (hi2/hessian.py:310-312):
//
//     wc[r0:r1, i2:] -= err1[r0:r1, 0:128] @ U[i1:i1+128, i2:]
//
// fp32 operands do not fit the tensor cores, TF32 alone (10-bit significand) is far too coarse
// for this path (a 1e-4 relative error in the update already moves 0.1 % of the codes), so each
// operand is split once into two TF32 numbers, x = hi + lo with hi = tf32(x), lo = tf32(x - hi),
// both rounded to nearest, and the product is formed as hi*hi + lo*hi + hi*lo with fp32
// accumulation in tensor memory: the dropped terms are below 3 * 2^-22 of |a||b|, the size of the
// rounding of an fp32 FMA chain of this length.  U is split once per factor, err1 once per block.
//
// Kernel: persistent CTAs over 128 x 256 output tiles.  Warp 4 feeds a two-stage TMA pipeline
// (per stage 32 of the 128 reduction steps: err hi/lo as 128-row and U^T hi/lo as 256-row
// K-major boxes, 96 KiB; U is stored transposed when it is split), warp 5 issues twelve tcgen05.mma kind::tf32
// (128 x 256 x 8, A negated in the instruction descriptor so the accumulator holds -err U) per
// stage into one of two 256-column accumulators, warps 0-3 each move their 32 rows of a finished
// accumulator through swizzled 32 x 32 staging boxes into wc with TMA reduce-add, so the
// read-modify-write of wc happens in L2 with full-line accesses and no warp waits on another.
// Every mbarrier wait is clock-bounded.
#include <cuda.h>

#include "common.cuh"

namespace hi2 {
namespace {

constexpr int LM = 128, LN = 256, LK = 128, KSTAGE = 32, LSTAGES = 2;
constexpr int A_BOX = LM * KSTAGE * 4;      // 16 KiB: 128 rows x 128 B
constexpr int B_PART = LN * KSTAGE * 4;     // 32 KiB: 256 output columns x 128 B, hi or lo of a stage
constexpr int LSTAGE_BYTES = 2 * A_BOX + 2 * B_PART;  // 96 KiB
constexpr int C_BOX = LM * 32 * 4;          // 16 KiB staging of 32 output columns
constexpr int L_THREADS = 192;
constexpr long long L_WAIT_CYCLES = 2000000000LL;

struct LControl {
  unsigned long long full[LSTAGES], empty[LSTAGES], acc_full[2], acc_empty[2];
  unsigned int tmem_base;
  volatile unsigned int abort;
};
constexpr size_t L_SMEM = (size_t)LSTAGES * LSTAGE_BYTES + 2 * C_BOX + sizeof(LControl) + 1024;

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(unsigned long long* b, uint32_t n) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(b)), "r"(n));
}
__device__ __forceinline__ void bar_expect(unsigned long long* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(unsigned long long* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(b)) : "memory");
}
__device__ __forceinline__ bool bar_try(unsigned long long* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(s32(b)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool bar_wait(unsigned long long* b, uint32_t parity, LControl* ctl, int* status) {
  if (bar_try(b, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (bar_try(b, parity)) return true;
    if (ctl->abort) return false;
    if (clock64() - t0 > L_WAIT_CYCLES) {
      ctl->abort = 1;
      atomicExch(status, HI2_ERR_TIMEOUT);
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load(void* dst, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(s32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(s32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_reduce_add(const CUtensorMap* map, const void* src, int x, int y) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(s32(src)), "r"(x), "r"(y) : "memory");
}
// K-major 128-byte-swizzled operand (rows of 128 B, 8-row groups 1024 B apart)
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::tf32: D fp32, A and B TF32 (format 2), A negated, both operands K-major, N = 256, M = 128.
// (With a plain 128-byte swizzle an MN-major TF32 operand reads as zeros on this hardware, which
// is why U is kept transposed rather than addressed MN-major as the second moment does for bf16.)
constexpr uint32_t L_IDESC = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 13) |
                             ((uint32_t)(LN >> 3) << 17) | ((uint32_t)(LM >> 4) << 24);

__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(da), "l"(db), "r"(L_IDESC), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void commit_to(unsigned long long* b) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(b)) : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct LParams {
  int* status;
  int row_tiles, col_tiles;
  int k0;    // first reduction row of U (i1)
  int col0;  // first output column (i2)
};

__global__ void __launch_bounds__(L_THREADS, 1)
lazy_tc_kernel(const __grid_constant__ CUtensorMap map_ahi, const __grid_constant__ CUtensorMap map_alo,
               const __grid_constant__ CUtensorMap map_bhi, const __grid_constant__ CUtensorMap map_blo,
               const __grid_constant__ CUtensorMap map_c, const LParams p) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_c = smem + (size_t)LSTAGES * LSTAGE_BYTES;
  LControl* ctl = reinterpret_cast<LControl*>(stage_c + 2 * C_BOX);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < LSTAGES; ++s) bar_init(&ctl->full[s], 1), bar_init(&ctl->empty[s], 1);
    for (int b = 0; b < 2; ++b) bar_init(&ctl->acc_full[b], 1), bar_init(&ctl->acc_empty[b], 4);
    ctl->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&ctl->tmem_base)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const int tiles = p.row_tiles * p.col_tiles;

  if (warp == 4 && lane == 0) {
    // ------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
      const int tr = tile % p.row_tiles, tc = tile / p.row_tiles;  // neighbours share the U tile
      const int row = tr * LM, col = p.col0 + tc * LN;
      for (int ks = 0; ks < LK / KSTAGE; ++ks) {
        if (!(ok = bar_wait(&ctl->empty[stage], phase ^ 1, ctl, p.status))) break;
        bar_expect(&ctl->full[stage], LSTAGE_BYTES);
        uint8_t* dst = smem + (size_t)stage * LSTAGE_BYTES;
        tma_load(dst, &map_ahi, &ctl->full[stage], ks * KSTAGE, row);
        tma_load(dst + A_BOX, &map_alo, &ctl->full[stage], ks * KSTAGE, row);
        tma_load(dst + 2 * A_BOX, &map_bhi, &ctl->full[stage], p.k0 + ks * KSTAGE, col);
        tma_load(dst + 2 * A_BOX + B_PART, &map_blo, &ctl->full[stage], p.k0 + ks * KSTAGE, col);
        if (++stage == LSTAGES) stage = 0, phase ^= 1;
      }
    }
    if (!ok) {
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000LL) {
      }
    }
  } else if (warp == 5 && lane == 0) {
    // ------------------------------------------------------------ MMA issuer
    int stage = 0;
    uint32_t phase = 0, n = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++n) {
      const int buf = n & 1;
      if (!(ok = bar_wait(&ctl->acc_empty[buf], ((n >> 1) & 1) ^ 1, ctl, p.status))) break;
      fence_after();
      const uint32_t d_tmem = tmem_base + buf * LN;
      for (int ks = 0; ks < LK / KSTAGE && ok; ++ks) {
        if (!(ok = bar_wait(&ctl->full[stage], phase, ctl, p.status))) break;
        fence_after();
        const uint32_t sa = s32(smem + (size_t)stage * LSTAGE_BYTES);
#pragma unroll
        for (int kk = 0; kk < KSTAGE / 8; ++kk) {
          const uint64_t ahi = desc_kmajor(sa + kk * 32), alo = desc_kmajor(sa + A_BOX + kk * 32);
          const uint64_t bhi = desc_kmajor(sa + 2 * A_BOX + kk * 32);
          const uint64_t blo = desc_kmajor(sa + 2 * A_BOX + B_PART + kk * 32);
          mma_tf32(d_tmem, ahi, bhi, (ks > 0 || kk > 0) ? 1u : 0u);
          mma_tf32(d_tmem, alo, bhi, 1u);
          mma_tf32(d_tmem, ahi, blo, 1u);
        }
        commit_to(&ctl->empty[stage]);
        if (++stage == LSTAGES) stage = 0, phase ^= 1;
      }
      if (ok) commit_to(&ctl->acc_full[buf]);
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------ epilogue: wc += (-err U)
    // Each warp owns the 32 rows of its tensor-memory lane quarter end to end (its own staging
    // boxes, its own reduce operations), so the four warps never wait on one another.
    uint32_t n = 0, chunk_no = 0;
    bool ok = true;
    uint8_t* my_boxes = stage_c + warp * (2 * C_BOX / 4);  // two 4 KiB boxes per warp
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++n) {
      const int tr = tile % p.row_tiles, tc = tile / p.row_tiles;
      const int buf = n & 1;
      if (!(ok = bar_wait(&ctl->acc_full[buf], (n >> 1) & 1, ctl, p.status))) break;
      fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + buf * LN;
      for (int c = 0; c < LN / 32; ++c, ++chunk_no) {
        uint32_t v[32];
        tmem_ld32(taddr + c * 32, v);
        uint8_t* box = my_boxes + (chunk_no & 1) * (C_BOX / 4);
        // the reduce issued two chunks ago has finished reading this box
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        __syncwarp();
        uint8_t* rowp = box + lane * 128;
#pragma unroll
        for (int q = 0; q < 8; ++q)  // 16-byte piece q of a row sits at piece q ^ (row % 8)
          *reinterpret_cast<uint4*>(rowp + ((q ^ (lane & 7)) << 4)) =
              make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          tma_reduce_add(&map_c, box, p.col0 + tc * LN + c * 32, tr * LM + warp * 32);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      fence_before();
      __syncwarp();
      if (lane == 0) bar_arrive(&ctl->acc_empty[buf]);
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  fence_before();
  __syncthreads();
  if (warp == 5) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// General product on the same pipeline, for the inverse factor's large steps:
//
//     C[m, n] (+)= (+-) A[m, kk] . Bt[n, kk]^T
//
// A and Bt are given as their TF32 parts (K-major, leading dimension ldk), C is fp32 with its own
// leading dimension.  Triangular operands are expressed as reduction ranges per tile (the same
// flags as gemm.cuh): the skipped range holds exact zeros, so taking whole 32-wide stages of it
// changes nothing.  The reduction of a tile is cut into windows of G_WINDOW stages (64 values of
// k): each window is accumulated in its own TMEM buffer and added, round-to-nearest, into fp32
// registers of the eight epilogue warps while the next window accumulates in the other buffer;
// the finished tile is ADDED to C by TMA once.  The tensor core's own accumulator truncates, so a
// chain of thousands of accumulation steps loses a decimal digit that the heavy cancellation of
// the factor recursion then exposes.  Measured on a rank-deficient 4096-wide Hessian (2048 tokens,
// condition 1e5), error of U against an fp64 solution over max|U|: one chain per tile 4.4e-4,
// windows of 256 4.1e-5, of 128 2.0e-5, of 64 1.2e-5 (the reference's fp32 LAPACK path: 8e-6).
// C always receives adds: for a plain store the launcher zeroes C first.  TMA clips the boxes at
// the edge of C, so m and n need no alignment.
constexpr int GT_KB_LE_J = 1, GT_KB_GE_J = 2, GT_KA_LE_I = 4, GT_LOWER_OUT = 8, GT_NEGATE = 16, GT_ADD = 32;

struct GParams {
  int* status;
  int row_tiles, col_tiles;
  int kk;
  int flags;
};

__device__ __forceinline__ void mma_tf32_d(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// Reduction stages [s0, s1) of tile (tr, tc), or s0 >= s1 for a tile that is not computed.
__device__ __forceinline__ void tile_range(const GParams& p, int tr, int tc, int& s0, int& s1) {
  int k0 = 0, k1 = p.kk;
  if (p.flags & GT_KB_LE_J) k1 = min(k1, (tc + 1) * LN);
  if (p.flags & GT_KA_LE_I) k1 = min(k1, (tr + 1) * LM);
  if (p.flags & GT_KB_GE_J) k0 = tc * LN;
  s0 = k0 / KSTAGE;
  s1 = (k1 + KSTAGE - 1) / KSTAGE;
  if (s1 < s0) s1 = s0;  // an empty range adds nothing: the tile of C keeps its (zeroed) content
  if ((p.flags & GT_LOWER_OUT) && tc * LN > tr * LM + LM - 1) s1 = s0;
}
constexpr int G_WINDOW = 2;     // stages per accumulation window
constexpr int G_THREADS = 320;  // warps 0..7 epilogue, warp 8 TMA, warp 9 MMA

__global__ void __launch_bounds__(G_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_ahi, const __grid_constant__ CUtensorMap map_alo,
               const __grid_constant__ CUtensorMap map_bhi, const __grid_constant__ CUtensorMap map_blo,
               const __grid_constant__ CUtensorMap map_c, const GParams p) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_c = smem + (size_t)LSTAGES * LSTAGE_BYTES;
  LControl* ctl = reinterpret_cast<LControl*>(stage_c + 2 * C_BOX);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < LSTAGES; ++s) bar_init(&ctl->full[s], 1), bar_init(&ctl->empty[s], 1);
    for (int b = 0; b < 2; ++b) bar_init(&ctl->acc_full[b], 1), bar_init(&ctl->acc_empty[b], 8);
    ctl->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&ctl->tmem_base)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const int tiles = p.row_tiles * p.col_tiles;

  if (warp == 8 && lane == 0) {
    // ------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
      const int tr = tile % p.row_tiles, tc = tile / p.row_tiles;  // neighbours share the B tile
      int s0, s1;
      tile_range(p, tr, tc, s0, s1);
      for (int ks = s0; ks < s1; ++ks) {
        if (!(ok = bar_wait(&ctl->empty[stage], phase ^ 1, ctl, p.status))) break;
        bar_expect(&ctl->full[stage], LSTAGE_BYTES);
        uint8_t* dst = smem + (size_t)stage * LSTAGE_BYTES;
        tma_load(dst, &map_ahi, &ctl->full[stage], ks * KSTAGE, tr * LM);
        tma_load(dst + A_BOX, &map_alo, &ctl->full[stage], ks * KSTAGE, tr * LM);
        tma_load(dst + 2 * A_BOX, &map_bhi, &ctl->full[stage], ks * KSTAGE, tc * LN);
        tma_load(dst + 2 * A_BOX + B_PART, &map_blo, &ctl->full[stage], ks * KSTAGE, tc * LN);
        if (++stage == LSTAGES) stage = 0, phase ^= 1;
      }
    }
    if (!ok) {
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000LL) {
      }
    }
  } else if (warp == 9 && lane == 0) {
    // ------------------------------------------------------------ MMA issuer
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((p.flags & GT_NEGATE) ? (1u << 13) : 0u) |
                           ((uint32_t)(LN >> 3) << 17) | ((uint32_t)(LM >> 4) << 24);
    int stage = 0;
    uint32_t phase = 0, n = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
      const int tr = tile % p.row_tiles, tc = tile / p.row_tiles;
      int s0, s1;
      tile_range(p, tr, tc, s0, s1);
      for (int w0 = s0; w0 < s1 && ok; w0 += G_WINDOW) {  // one TMEM buffer per window
        const int w1 = min(w0 + G_WINDOW, s1);
        const int buf = n & 1;
        if (!(ok = bar_wait(&ctl->acc_empty[buf], ((n >> 1) & 1) ^ 1, ctl, p.status))) break;
        fence_after();
        const uint32_t d_tmem = tmem_base + buf * LN;
        for (int ks = w0; ks < w1 && ok; ++ks) {
          if (!(ok = bar_wait(&ctl->full[stage], phase, ctl, p.status))) break;
          fence_after();
          const uint32_t sa = s32(smem + (size_t)stage * LSTAGE_BYTES);
#pragma unroll
          for (int kk = 0; kk < KSTAGE / 8; ++kk) {
            const uint64_t ahi = desc_kmajor(sa + kk * 32), alo = desc_kmajor(sa + A_BOX + kk * 32);
            const uint64_t bhi = desc_kmajor(sa + 2 * A_BOX + kk * 32);
            const uint64_t blo = desc_kmajor(sa + 2 * A_BOX + B_PART + kk * 32);
            mma_tf32_d(d_tmem, ahi, bhi, idesc, (ks > w0 || kk > 0) ? 1u : 0u);
            mma_tf32_d(d_tmem, alo, bhi, idesc, 1u);
            mma_tf32_d(d_tmem, ahi, blo, idesc, 1u);
          }
          commit_to(&ctl->empty[stage]);
          if (++stage == LSTAGES) stage = 0, phase ^= 1;
        }
        if (ok) commit_to(&ctl->acc_full[buf]);
        ++n;
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------ epilogue
    // Warp w owns tensor-memory lanes 32 (w mod 4) .. +31 (the rows of the tile) and columns
    // 128 (w / 4) .. +127.  A finished window is added into fp32 registers (round-to-nearest), so
    // the tensor-memory accumulator, which truncates, never carries more than G_WINDOW stages, and
    // C sees one add per element and tile.
    const int quarter = warp & 3, half = warp >> 2;
    uint32_t n = 0;
    bool ok = true;
    uint8_t* box = stage_c + warp * (C_BOX / 4);  // one 32 x 32 staging box per warp
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
      const int tr = tile % p.row_tiles, tc = tile / p.row_tiles;
      int s0, s1;
      tile_range(p, tr, tc, s0, s1);
      if (s1 <= s0) continue;
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
      for (int w0 = s0; w0 < s1 && ok; w0 += G_WINDOW) {
        const int buf = n & 1;
        if (!(ok = bar_wait(&ctl->acc_full[buf], (n >> 1) & 1, ctl, p.status))) break;
        fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * LN + half * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld32(taddr + c * 32, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c * 32 + i] += __uint_as_float(v[i]);
        }
        fence_before();
        __syncwarp();
        if (lane == 0) bar_arrive(&ctl->acc_empty[buf]);
        ++n;
      }
      if (!ok) break;
      uint8_t* rowp = box + lane * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the box is free again
        __syncwarp();
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<float4*>(rowp + ((q ^ (lane & 7)) << 4)) =
              make_float4(acc[c * 32 + 4 * q], acc[c * 32 + 4 * q + 1], acc[c * 32 + 4 * q + 2], acc[c * 32 + 4 * q + 3]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          tma_reduce_add(&map_c, box, tc * LN + half * 128 + c * 32, tr * LM + quarter * 32);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  fence_before();
  __syncthreads();
  if (warp == 9) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// TF32 parts of a [rows, cols] block with leading dimension ldx, written with leading dimension ldo.
__global__ void __launch_bounds__(256)
split_block_kernel(const float* __restrict__ x, int64_t ldx, int64_t rows, int64_t cols,
                   float* __restrict__ hi, float* __restrict__ lo, int64_t ldo) {
  const int64_t c4 = cols / 4;  // cols is a multiple of 4
  const int64_t total = rows * c4, stride = (int64_t)gridDim.x * 256;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / c4, c = (i % c4) * 4;
    const float4 v = *reinterpret_cast<const float4*>(x + r * ldx + c);
    const float in[4] = {v.x, v.y, v.z, v.w};
    float h[4], l[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      uint32_t hb, lb;
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(in[t]));
      h[t] = __uint_as_float(hb);
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lb) : "f"(in[t] - h[t]));
      l[t] = __uint_as_float(lb);
    }
    *reinterpret_cast<float4*>(hi + r * ldo + c) = make_float4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<float4*>(lo + r * ldo + c) = make_float4(l[0], l[1], l[2], l[3]);
  }
}

// The same for the transpose: x [rows, cols] (ldx) -> hi, lo [cols, rows] (ldo).
__global__ void __launch_bounds__(256)
split_block_transposed_kernel(const float* __restrict__ x, int64_t ldx, int64_t rows, int64_t cols,
                              float* __restrict__ hi, float* __restrict__ lo, int64_t ldo) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
  for (int i = ty; i < 32; i += 8)
    tile[i][tx] = (r0 + i < rows && c0 + tx < cols) ? x[(r0 + i) * ldx + c0 + tx] : 0.0f;
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    if (c0 + i < cols && r0 + tx < rows) {
      const float v = tile[tx][i];
      uint32_t hb, lb;
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(v));
      const float h = __uint_as_float(hb);
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lb) : "f"(v - h));
      hi[(c0 + i) * ldo + r0 + tx] = h;
      lo[(c0 + i) * ldo + r0 + tx] = __uint_as_float(lb);
    }
  }
}

// hi = tf32(x), lo = tf32(x - hi), both round-to-nearest (ties away): x = hi + lo + O(2^-22 |x|)
__global__ void __launch_bounds__(256)
split_tf32_kernel(const float* __restrict__ x, float* __restrict__ hi, float* __restrict__ lo, int64_t n4) {
  const int64_t stride = (int64_t)gridDim.x * 256;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += stride) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    const float in[4] = {v.x, v.y, v.z, v.w};
    float h[4], l[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      uint32_t hb, lb;
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(in[t]));
      h[t] = __uint_as_float(hb);
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lb) : "f"(in[t] - h[t]));
      l[t] = __uint_as_float(lb);
    }
    reinterpret_cast<float4*>(hi)[i] = make_float4(h[0], h[1], h[2], h[3]);
    reinterpret_cast<float4*>(lo)[i] = make_float4(l[0], l[1], l[2], l[3]);
  }
}

// hi/lo parts of x^T: x [rows, cols] -> hi, lo [cols, rows]; 32 x 32 tiles through shared memory
__global__ void __launch_bounds__(256)
split_tf32_transposed_kernel(const float* __restrict__ x, float* __restrict__ hi, float* __restrict__ lo,
                             int64_t rows, int64_t cols) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
  for (int i = ty; i < 32; i += 8)
    tile[i][tx] = (r0 + i < rows && c0 + tx < cols) ? x[(r0 + i) * cols + c0 + tx] : 0.0f;
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    if (c0 + i < cols && r0 + tx < rows) {
      const float v = tile[tx][i];
      uint32_t hb, lb;
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(v));
      const float h = __uint_as_float(hb);
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lb) : "f"(v - h));
      hi[(c0 + i) * rows + r0 + tx] = h;
      lo[(c0 + i) * rows + r0 + tx] = __uint_as_float(lb);
    }
  }
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

bool make_map(CUtensorMap* map, const float* base, int64_t inner, int64_t outer, int64_t ld, int box_in,
              int box_out) {
  const cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  const cuuint32_t box[2] = {(cuuint32_t)box_in, (cuuint32_t)box_out};
  const cuuint32_t es[2] = {1, 1};
  return encoder()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Used by gptq.cu.  err_hi/err_lo [n_rows, 128], ut_hi/ut_lo [k, k] = the TF32 parts of U^T,
// wc [n_rows, k]; i2 = i1 + 128.
int launch_lazy_tc(float* wc, int64_t n_rows, int64_t k, int64_t i1, const float* err_hi,
                   const float* err_lo, const float* ut_hi, const float* ut_lo, int* status,
                   cudaStream_t stream) {
  const int64_t i2 = i1 + LK;
  if (n_rows <= 0 || i2 >= k) return HI2_OK;
  if (encoder() == nullptr) return fail(HI2_ERR_DRIVER, "gptq_lazy_update: cuTensorMapEncodeTiled unavailable");
  CUtensorMap mah, mal, mbh, mbl, mc;
  if (!make_map(&mah, err_hi, LK, n_rows, LK, 32, LM) || !make_map(&mal, err_lo, LK, n_rows, LK, 32, LM) ||
      !make_map(&mbh, ut_hi, k, k, k, 32, LN) || !make_map(&mbl, ut_lo, k, k, k, 32, LN) ||
      !make_map(&mc, wc, k, n_rows, k, 32, 32))
    return fail(HI2_ERR_DRIVER, "gptq_lazy_update: cuTensorMapEncodeTiled failed");
  if (cudaFuncSetAttribute(lazy_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L_SMEM) != cudaSuccess)
    return fail(HI2_ERR_LAUNCH, "gptq_lazy_update: cannot reserve shared memory");
  LParams p;
  p.status = status;
  p.row_tiles = (int)ceil_div(n_rows, LM);
  p.col_tiles = (int)ceil_div(k - i2, LN);
  p.k0 = (int)i1, p.col0 = (int)i2;
  const int tiles = p.row_tiles * p.col_tiles;
  int device = 0, sms = 148;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  lazy_tc_kernel<<<tiles < sms ? tiles : sms, L_THREADS, L_SMEM, stream>>>(mah, mal, mbh, mbl, mc, p);
  return check_launch("gptq_lazy_update (tcgen05)");
}

// C[m, n] (ldc) = or += (+-) A . Bt^T with A = a_hi + a_lo [m, kk], Bt = b_hi + b_lo [n, kk], both with
// leading dimension ldk (a multiple of 4 floats).  flags: GT_* above.  All bases 16-byte aligned.
int launch_gemm_tc2(int64_t m, int64_t n, int64_t kk, const float* a_hi, const float* a_lo, int64_t lda,
                    const float* b_hi, const float* b_lo, int64_t ldb, float* c, int64_t ldc, int flags,
                    int* status, cudaStream_t stream);

int launch_gemm_tc(int64_t m, int64_t n, int64_t kk, const float* a_hi, const float* a_lo, const float* b_hi,
                   const float* b_lo, int64_t ldk, float* c, int64_t ldc, int flags, int* status,
                   cudaStream_t stream) {
  return launch_gemm_tc2(m, n, kk, a_hi, a_lo, ldk, b_hi, b_lo, ldk, c, ldc, flags, status, stream);
}

// The same with a leading dimension per operand (A [m, kk] with lda, Bt [n, kk] with ldb).
int launch_gemm_tc2(int64_t m, int64_t n, int64_t kk, const float* a_hi, const float* a_lo, int64_t lda,
                    const float* b_hi, const float* b_lo, int64_t ldb, float* c, int64_t ldc, int flags,
                    int* status, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || kk <= 0) return HI2_OK;
  if (encoder() == nullptr) return fail(HI2_ERR_DRIVER, "gemm_tc: cuTensorMapEncodeTiled unavailable");
  CUtensorMap mah, mal, mbh, mbl, mc;
  if (!make_map(&mah, a_hi, kk, m, lda, 32, LM) || !make_map(&mal, a_lo, kk, m, lda, 32, LM) ||
      !make_map(&mbh, b_hi, kk, n, ldb, 32, LN) || !make_map(&mbl, b_lo, kk, n, ldb, 32, LN) ||
      !make_map(&mc, c, n, m, ldc, 32, 32))
    return fail(HI2_ERR_DRIVER, "gemm_tc: cuTensorMapEncodeTiled failed");
  if (cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L_SMEM) != cudaSuccess)
    return fail(HI2_ERR_LAUNCH, "gemm_tc: cannot reserve shared memory");
  if (!(flags & GT_ADD) &&  // the kernel only adds: a plain store starts from zeros
      cudaMemset2DAsync(c, (size_t)ldc * sizeof(float), 0, (size_t)n * sizeof(float), (size_t)m, stream) != cudaSuccess)
    return fail(HI2_ERR_LAUNCH, "gemm_tc: memset failed");
  GParams p;
  p.status = status;
  p.row_tiles = (int)ceil_div(m, LM);
  p.col_tiles = (int)ceil_div(n, LN);
  p.kk = (int)kk, p.flags = flags | GT_ADD;
  const int tiles = p.row_tiles * p.col_tiles;
  int device = 0, sms = 148;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  gemm_tc_kernel<<<tiles < sms ? tiles : sms, G_THREADS, L_SMEM, stream>>>(mah, mal, mbh, mbl, mc, p);
  return check_launch("gemm_tc");
}

int launch_split_block(const float* x, int64_t ldx, int64_t rows, int64_t cols, float* hi, float* lo,
                       int64_t ldo, bool transposed, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return HI2_OK;
  if (transposed) {
    dim3 grid((unsigned)ceil_div(cols, 32), (unsigned)ceil_div(rows, 32));
    split_block_transposed_kernel<<<grid, 256, 0, stream>>>(x, ldx, rows, cols, hi, lo, ldo);
  } else {
    int64_t blocks = ceil_div(rows * (cols / 4), 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    split_block_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, ldx, rows, cols, hi, lo, ldo);
  }
  return check_launch("split_block");
}

int launch_split_tf32(const float* x, float* hi, float* lo, int64_t n, cudaStream_t stream) {
  if (n <= 0) return HI2_OK;
  int64_t blocks = ceil_div(n / 4, 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  split_tf32_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, hi, lo, n / 4);
  return check_launch("split_tf32");
}

int launch_split_tf32_transposed(const float* x, float* hi, float* lo, int64_t rows, int64_t cols,
                                 cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return HI2_OK;
  dim3 grid((unsigned)ceil_div(cols, 32), (unsigned)ceil_div(rows, 32));
  split_tf32_transposed_kernel<<<grid, 256, 0, stream>>>(x, hi, lo, rows, cols);
  return check_launch("split_tf32_transposed");
}

}  // namespace hi2

extern "C" int hi2_split_tf32_transposed(const float* x, float* hi, float* lo, int64_t rows, int64_t cols,
                                         void* stream) {
  using namespace hi2;
  HI2_REQUIRE(rows >= 0 && cols >= 0, "split_tf32_transposed: negative size");
  if (rows == 0 || cols == 0) return HI2_OK;
  HI2_REQUIRE(x && hi && lo, "split_tf32_transposed: null pointer");
  return launch_split_tf32_transposed(x, hi, lo, rows, cols, static_cast<cudaStream_t>(stream));
}

extern "C" int hi2_gemm_tf32x3(int64_t m, int64_t n, int64_t kk, const float* a_hi, const float* a_lo, int64_t lda,
                               const float* bt_hi, const float* bt_lo, int64_t ldb, float* c, int64_t ldc,
                               int accumulate, int32_t* status, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(m >= 0 && n >= 0 && kk >= 0, "gemm_tf32x3: negative size");
  if (m == 0 || n == 0) return HI2_OK;
  HI2_REQUIRE(kk > 0 && a_hi && a_lo && bt_hi && bt_lo && c && status, "gemm_tf32x3: null pointer or empty reduction");
  HI2_REQUIRE(aligned16(a_hi) && aligned16(a_lo) && aligned16(bt_hi) && aligned16(bt_lo) && aligned16(c),
              "gemm_tf32x3: operands must be 16-byte aligned");
  HI2_REQUIRE(lda % 4 == 0 && ldb % 4 == 0 && ldc % 4 == 0 && lda >= kk && ldb >= kk && ldc >= n,
              "gemm_tf32x3: leading dimensions must be multiples of 4 floats and cover the rows");
  return launch_gemm_tc2(m, n, kk, a_hi, a_lo, lda, bt_hi, bt_lo, ldb, c, ldc, accumulate ? GT_ADD : 0,
                         reinterpret_cast<int*>(status), static_cast<cudaStream_t>(stream));
}

extern "C" int hi2_split_tf32(const float* x, float* hi, float* lo, int64_t n, void* stream) {
  using namespace hi2;
  HI2_REQUIRE(n >= 0 && n % 4 == 0, "split_tf32: the element count must be a multiple of 4");
  if (n == 0) return HI2_OK;
  HI2_REQUIRE(x && hi && lo, "split_tf32: null pointer");
  HI2_REQUIRE(aligned16(x) && aligned16(hi) && aligned16(lo), "split_tf32: buffers must be 16-byte aligned");
  return launch_split_tf32(x, hi, lo, n, static_cast<cudaStream_t>(stream));
}
