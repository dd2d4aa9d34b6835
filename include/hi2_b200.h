/* C-ABI of libhi2_b200.so: the sm_100a kernels of the per-layer PTQ encode path of hi2.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in _host;
 *   - matrices are row-major and contiguous unless a leading dimension is passed;
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, nothing
 *     synchronises unless stated;
 *   - the caller owns every buffer, outputs included; the library allocates nothing
 *     except where a function says so;
 *   - the return value is 0 on success, else one of the HI2_ERR_* codes below;
 *     hi2_last_error() gives the text for the calling thread.
 *
 * Each declaration names the interface of the reference (path inside the hi2 project) that it
 * stands in for.
 */
#ifndef HI2_B200_H
#define HI2_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  HI2_OK = 0,
  HI2_ERR_ARG = 1,        /* bad shape, dtype, alignment or null pointer */
  HI2_ERR_LAUNCH = 2,     /* the CUDA runtime refused a launch or a copy */
  HI2_ERR_NOT_PD = 3,     /* factorisation met a non-positive pivot */
  HI2_ERR_TIMEOUT = 4,    /* a bounded device-side wait ran out */
  HI2_ERR_CODE_RANGE = 5, /* a code outside its ladder reached the packer */
  HI2_ERR_WORKSPACE = 6,  /* workspace too small */
  HI2_ERR_DRIVER = 7      /* a driver entry point (tensor maps) is unavailable */
};

enum { HI2_F32 = 0, HI2_F64 = 1, HI2_F16 = 2, HI2_BF16 = 3 };

int hi2_abi_version(void);
const char* hi2_last_error(void);
/* Kernel launches this library has enqueued in the process so far (all threads).  No counterpart
 * in the reference; benchmarks difference it around a timed region. */
long long hi2_launch_count(void);
/* Chains of short kernels (the inverse factor, the GPTQ column loop) that this library has sent
 * to a stream as one CUDA graph launch each, in the process so far.  No counterpart in the
 * reference. */
long long hi2_graph_launch_count(void);

/* ---- rotation ------------------------------------------------------------------------------
 * hi2/format.py:30-41 fwht_groups, fused with the cast and smoothing multiply of
 * hi2/calibrate.py:243-251.  y[r, :] = rotate(flags, x[r, :] * col_scale).  Allowed
 * (in, out) dtypes: equal types, or F16/BF16 -> F32.  col_scale (fp32 [k], may be null) needs an
 * F32 output.  fp32/fp64 are transformed in their own precision with the 16 products of an
 * output summed in ascending k; half types in fp64 with one final rounding. */
int hi2_rotate_groups(const void* x, int in_dtype, void* y, int out_dtype, const uint8_t* flags,
                      const float* col_scale, int64_t rows, int64_t k, void* stream);

/* ---- packing -------------------------------------------------------------------------------
 * hi2/format.py:73-85 pack_codes: n codes per row -> n*nbits/32 int32 words, first code in the
 * low bits.  *bad (device int, caller zeroes it) is set non-zero when a code >= 2^nbits. */
int hi2_pack_codes(const uint8_t* codes, int32_t* words, int64_t rows, int64_t n, int nbits,
                   int32_t* bad, void* stream);

/* hi2/format.py:158-171 (the loop body of assemble): scatter one piece (rows sharing one
 * (nbits, block)) into the flat buffers.  rows[n_rows] are tensor row indices; code_off /
 * param_off are the int64 [R+1] prefix sums (words / blocks). */
int hi2_assemble_piece(const int64_t* rows, int64_t n_rows, const uint8_t* codes,
                       const uint8_t* params, const uint16_t* consts, int64_t k, int nbits,
                       int block, const int64_t* code_off, const int64_t* param_off,
                       int32_t* out_codes, uint8_t* out_params, uint16_t* out_consts,
                       int32_t* bad, void* stream);

/* hi2/format.py:195-239 dequantize_stored / dequantize: the fp16 reconstruction of every weight of
 * a packed tensor (the flat buffers of hi2_assemble_piece), as fp64 (the reference's type; equal
 * bit for bit on any device, every step being exact or correctly rounded) or fp32 [rows, k].
 * original_basis = 0: the stored basis; 1: rotated back (had [k/16]) and divided by the smoothing
 * vector (col_scale fp16 [k], may be null).  *bad (device int, caller zeroes it) is raised by a row
 * whose code width or block size is not one of the format's. */
int hi2_dequantize(const int32_t* codes, const int32_t* code_off, const uint8_t* blk_params,
                   const int32_t* param_off, const uint16_t* row_consts, const uint8_t* row_nbits,
                   const uint8_t* row_block, const uint8_t* had, const uint16_t* col_scale, int64_t rows,
                   int64_t k, int original_basis, void* out, int out_dtype, int32_t* bad, void* stream);

/* ---- ladder search -------------------------------------------------------------------------
 * hi2/ladder_kernel.py:44-101 ladder_grid: wb [n_rows, nb, block] fp32, db [nb, block],
 * grid_host[g] (host floats, g <= 8), n = number of codes.  Outputs [n_rows, nb] fp32. */
int hi2_ladder_grid(const float* wb, const float* db, const float* grid_host, int g, int n,
                    int64_t n_rows, int64_t nb, int block, float* lo, float* step, float* err,
                    void* stream);

/* hi2/encode.py:53-92 fit_ladder: grid search plus `refits` weighted least-squares refits.
 * w is [n_rows, k] with leading dimension ldw; outputs [n_rows, k/block]. */
int hi2_fit_ladder(const float* w, int64_t ldw, const float* d, const float* grid_host, int g,
                   int refits, int n, int64_t n_rows, int64_t k, int block, float* lo,
                   float* step, void* stream);

/* hi2/encode.py:95-119 quantize_params + hi2/format.py:45-60 decode_params + the code
 * assignment and error of hi2/encode.py:146-157, one row per thread block.
 * Inputs lo/step [n_rows, k/block].  Outputs (each may be null): params u8 [n_rows, nb, 2],
 * consts fp16 [n_rows, 3], lo_d/step_d fp32 decoded ladders with leading dimension ldp,
 * codes u8 [n_rows, k], sse fp32 [n_rows], energy fp32 [n_rows] = sum d*w^2.
 * w and d may be null when codes, sse and energy are. */
int hi2_quantize_rows(const float* lo, const float* step, const float* w, int64_t ldw,
                      const float* d, int nbits, int64_t n_rows, int64_t k, int block,
                      uint8_t* params, uint16_t* consts, float* lo_d, float* step_d, int64_t ldp,
                      uint8_t* codes, float* sse, float* energy, void* stream);
/* The same two with column weights per row: d is [groups, k] and row r is weighted by d[row_d[r]]
 * (row_d int32 [n_rows] on the device; null: one d for all rows, as above).  Rows of tensors that
 * read different inputs (the experts of a layer, hi2/layerwise.py:636-672) are searched and
 * quantised in one launch this way; per row the arithmetic is the one above.  No counterpart in the
 * reference. */
int hi2_fit_ladder_grouped(const float* w, int64_t ldw, const float* d, const int32_t* row_d,
                           const float* grid_host, int g, int refits, int n, int64_t n_rows,
                           int64_t k, int block, float* lo, float* step, void* stream);
int hi2_quantize_rows_grouped(const float* lo, const float* step, const float* w, int64_t ldw,
                              const float* d, const int32_t* row_d, int nbits, int64_t n_rows,
                              int64_t k, int block, uint8_t* params, uint16_t* consts, float* lo_d,
                              float* step_d, int64_t ldp, uint8_t* codes, float* sse, float* energy,
                              void* stream);

/* ---- GPTQ ----------------------------------------------------------------------------------
 * hi2/gptq_kernel.py:59-127 gptq_block: one lazy block [i1, i1+len) for every row.
 * wc [n_rows, k] fp32 (read), err1 [n_rows, len], codes u8 [n_rows, k], lo/st [n_rows, ldp],
 * row_grp int32 [n_rows], u_ptrs int64 [groups] (device addresses of [k, k] fp32 factors),
 * blk int32 [groups, k], nmax fp32 [groups], comp fp32 [n_rows, k] or null. */
int hi2_gptq_block(const float* wc, int64_t n_rows, int64_t k, int64_t i1, int len, float* err1,
                   uint8_t* codes, const float* lo, const float* st, int64_t ldp,
                   const int32_t* row_grp, const int64_t* u_ptrs, const int32_t* blk,
                   const float* nmax, float* comp, void* stream);

/* hi2/hessian.py:310-312: wc[:, i2:] -= err1 @ u[i1:i2, i2:] for one unit (n_rows rows). */
int hi2_gptq_lazy_update(float* wc, int64_t n_rows, int64_t k, int64_t i1, int64_t i2,
                         const float* err1, const float* u, void* stream);

/* hi2/hessian.py:267-315 _round_kernel, the whole column loop: block kernel and trailing update
 * for every lazy block, no host synchronisation.  Units are consecutive row ranges
 * unit_rows_host[u] .. unit_rows_host[u+1] whose factor is u_host[u] (device address).
 * err1 is caller scratch [n_rows, 128]. */
int hi2_gptq_round(float* wc, int64_t n_rows, int64_t k, float* err1, uint8_t* codes,
                   const float* lo, const float* st, int64_t ldp, const int32_t* row_grp,
                   const int64_t* u_ptrs, const int32_t* blk, const float* nmax, float* comp,
                   int n_units, const int64_t* unit_rows_host, const int64_t* u_host,
                   void* stream);

/* The same column loop with the trailing update on the tensor cores: every operand split into
 * two TF32 numbers (hi + lo), three tcgen05 products with fp32 accumulation, accuracy of an fp32
 * FMA chain.  u_split_host[u] is the device address of a [2, k, k] fp32 array holding the hi and
 * lo parts of the TRANSPOSE of unit u's factor (hi2_split_tf32_transposed); err_split is caller scratch [2, n_rows, 128];
 * *status (device int32) is cleared and receives HI2_ERR_TIMEOUT if a bounded wait ran out. */
int hi2_gptq_round_tc(float* wc, int64_t n_rows, int64_t k, float* err1, float* err_split,
                      uint8_t* codes, const float* lo, const float* st, int64_t ldp,
                      const int32_t* row_grp, const int64_t* u_ptrs, const int32_t* blk,
                      const float* nmax, float* comp, int n_units, const int64_t* unit_rows_host,
                      const int64_t* u_split_host, int32_t* status, void* stream);

/* One trailing update on the tensor cores: wc[:, i1+128:] -= err @ u[i1:i1+128, i1+128:] with
 * err_split [2, n_rows, 128] the TF32 parts of err and u_split [2, k, k] those of u^T.  *status is NOT
 * cleared here (the caller zeroes it once). */
int hi2_gptq_lazy_update_tc(float* wc, int64_t n_rows, int64_t k, int64_t i1, const float* err_split,
                            const float* u_split, int32_t* status, void* stream);

/* x = hi + lo with hi = tf32(x), lo = tf32(x - hi), round to nearest; n a multiple of 4.  Prepares
 * the operands of hi2_gptq_round_tc.  No counterpart in the reference. */
int hi2_split_tf32(const float* x, float* hi, float* lo, int64_t n, void* stream);
/* The same split of x^T: x [rows, cols] -> hi, lo [cols, rows] (the factor operand of the
 * tensor-core trailing update is kept transposed so that both operands are K-major). */
int hi2_split_tf32_transposed(const float* x, float* hi, float* lo, int64_t rows, int64_t cols,
                              void* stream);

/* c[m, n] (ldc) = or += a . bt^T in fp32-grade arithmetic on the tensor cores: both operands as
 * their TF32 parts from hi2_split_tf32 (a [m, kk] with leading dimension lda, bt [n, kk] with ldb,
 * both K-major), three tcgen05 TF32 products per tile accumulated in windows of 64 values of k.
 * Replaces the fp32 library products of the refinement, g = e @ Hs and g += dw @ Hs[b0:b1]
 * (hi2/refine.py:64, :83, :103; Hs is symmetric, so its rows serve as bt).  *status (device int,
 * caller zeroes it) is raised by a bounded wait that ran out. */
int hi2_gemm_tf32x3(int64_t m, int64_t n, int64_t kk, const float* a_hi, const float* a_lo, int64_t lda,
                    const float* bt_hi, const float* bt_lo, int64_t ldb, float* c, int64_t ldc, int accumulate,
                    int32_t* status, void* stream);

/* hi2/hessian.py:331-338 (_finish): sse[r] = sum_j d[j] * (fp16(lo + code*step) - w[r, j])^2
 * with the decoded ladders lo/st [n_rows, ldp] of block size `block`. */
int hi2_ladder_sse(const uint8_t* codes, const float* w, int64_t ldw, const float* d,
                   const float* lo, const float* st, int64_t ldp, int64_t n_rows, int64_t k,
                   int block, float* sse, void* stream);

/* ---- refinement ----------------------------------------------------------------------------
 * hi2/refine_kernel.py:51-120 refine_block: gb [n_rows, len] (read), c [n_rows, k] fp32 codes
 * (in/out), lo/st [n_rows, k] per-column ladders, top [n_rows], hs [k, k], dwb [n_rows, len]
 * (out; every entry is written, 0 where the code stayed). */
int hi2_refine_block(const float* gb, int len, float* c, const float* lo, const float* st,
                     const float* top, const float* hs, int64_t n_rows, int64_t k, int64_t b0,
                     float* dwb, void* stream);
/* The same block for the sweep of hi2/refine.py:60-84 with two copies folded in: the block's slice
 * of g is read where it lies (g [n_rows, k], columns b0 .. b0+len), and the changes are written as
 * the two TF32 parts dw_hi/dw_lo (rows of len floats, lddw floats apart: the parts of several
 * blocks can lie side by side) that hi2_gemm_tf32x3 takes for g += dw Hs[b0:b0+len] (dw_hi + dw_lo
 * differs from dw by at most 2^-22 |dw|).  Same decisions as hi2_refine_block. */
int hi2_refine_block_in_place(const float* g, int len, float* c, const float* lo, const float* st,
                              const float* top, const float* hs, int64_t n_rows, int64_t k,
                              int64_t b0, float* dw_hi, float* dw_lo, int64_t lddw, void* stream);

/* ---- dense helpers of the path -------------------------------------------------------------
 * C = alpha * op(A) op(B) + beta * C in fp32 (fused multiply-add accumulation, fp32 operands):
 * the products hi2/hessian.py:312, hi2/refine.py:64,83,103 hand to the BLAS.  Row-major;
 * trans_a: A is stored [kk, m]; trans_b: B is stored [n, kk]. */
int hi2_gemm_f32(int trans_a, int trans_b, int64_t m, int64_t n, int64_t kk, float alpha,
                 const float* a, int64_t lda, const float* b, int64_t ldb, float beta, float* c,
                 int64_t ldc, void* stream);

/* ---- Hessian -------------------------------------------------------------------------------
 * hi2/hessian.py:35-40 HessianStats.update: S += x^T x, x [tokens, k] of dtype F16/BF16/F32,
 * S [k, k] fp32 (both triangles are written and are exact mirrors of each other).
 * workspace: hi2_hessian_workspace_bytes(tokens, k) bytes of caller scratch (may be null when
 * that is 0). */
size_t hi2_hessian_workspace_bytes(int64_t tokens, int64_t k, int dtype);
int hi2_hessian_accumulate(const void* x, int dtype, int64_t tokens, int64_t k, float* s,
                           void* workspace, size_t workspace_bytes, void* stream);
/* The tensor-core kernel bounds every device-side wait; a wait that ran out leaves
 * HI2_ERR_TIMEOUT in the first word of the workspace instead of hanging.  This copies that word
 * to *status_host (synchronises with the device).  No counterpart in the reference. */
int hi2_hessian_status(const void* workspace, int* status_host);

/* No counterpart in the reference.  The second moment for callers that cannot allocate device
 * memory where statistics are taken (a hook running inside another framework's allocator, a
 * process with a stream capture in flight, a fixed memory budget): same result as
 * hi2_hessian_accumulate on the tensor-core path, but the item tiles live in a 64 MiB device
 * array inside the library instead of a caller workspace, and nothing is allocated or freed.
 * Limits: dtype F16/BF16, tokens >= 256, 256 <= k <= 5632 (more returns HI2_ERR_WORKSPACE).
 * *status (device int32, caller-owned output) is cleared by the call and receives
 * HI2_ERR_TIMEOUT if a bounded device-side wait ran out.  The first call on a device looks up
 * the array's address (cudaGetSymbolAddress): make it before any stream capture.  All calls
 * share the array, so calls that overlap on the GPU race. */
int hi2_hessian_accumulate_noalloc(const void* x, int dtype, int64_t tokens, int64_t k, float* s,
                                   int32_t* status, void* stream);

/* hi2/stats.py:27-33 ColumnStats.update, taken from the second moment: g [k/16, 16, 16] fp64
 * += the 16x16 diagonal blocks of s. */
int hi2_group_moments(const float* s, int64_t k, double* g, void* stream);
/* The same blocks accumulated straight from activations x [tokens, k] (F16/BF16/F32): fp32 sums
 * per run of 4096 tokens, fp64 total, as hi2/stats.py:27-33 does. */
int hi2_group_moments_update(const void* x, int dtype, int64_t tokens, int64_t k, double* g,
                             void* stream);

/* hi2/hessian.py:50-68 transform_sigma: hs = sym(T (sigma/denom) T^T), T = R diag(1/col_scale).
 * col_scale fp16 [k] or null, had u8 [k/16], diag (fp32 [k], may be null) receives diag(hs). */
int hi2_transform_sigma(const float* sigma, float denom, const uint16_t* col_scale,
                        const uint8_t* had, int64_t k, float* hs, float* diag, void* stream);

/* hi2/hessian.py:71-86 inverse_factor, one damping attempt: u = upper Cholesky factor of
 * (hs + *lam * I)^-1 with lam a device fp32 scalar.  *info (device int, caller zeroes it) is
 * set to 1 + index of the first non-positive pivot, or to -1 when a bounded device-side wait of
 * the tensor-core products ran out; u is then unspecified.  Workspace:
 * hi2_inverse_factor_workspace_bytes(k) bytes, 16-byte aligned (8 k^2 for the two fp32 work
 * matrices, plus about 4 k^2 for the TF32 operand parts when k >= 2048). */
size_t hi2_inverse_factor_workspace_bytes(int64_t k);
int hi2_inverse_factor(const float* hs, const float* lam, int64_t k, float* u, void* workspace,
                       size_t workspace_bytes, int32_t* info, void* stream);

/* ---- allocation ----------------------------------------------------------------------------
 * hi2/allocate.py:88-137 (_argmin0 and _Flat.solve) for one multiplier: picks[r] = first
 * candidate minimising cost[c, r] + lam * bits[c, r] (fp64, product and sum rounded
 * separately); *picked_bits (device double, caller zeroes it) += the bits of the picks (whole
 * numbers, so the sum is exact in any order).  cost and bits are [n_cand, n_rows]. */
int hi2_allocate_solve(const double* cost, const double* bits, int n_cand, int64_t n_rows,
                       double lam, int64_t* picks, double* picked_bits, void* stream);

/* The picked-bit totals of up to 32 multipliers in one launch (same arithmetic, no picks written):
 * totals[i] (device doubles, caller zeroes them) += bits picked under lams_host[i].  Lets the host
 * take five steps of the reference's bisection per round trip (the 31 midpoints they can reach). */
int hi2_allocate_bits(const double* cost, const double* bits, int n_cand, int64_t n_rows,
                      const double* lams_host, int n_lams, double* totals, void* stream);

#ifdef __cplusplus
}
#endif
#endif
