/* train_gpt_b200 -- C ABI of the B200 (sm_100a) kernels behind train-gpt's FP8
 * hot path.  Every entry point takes plain device pointers, sizes and a CUDA
 * stream (passed as void*; NULL = the legacy default stream), launches
 * asynchronously on that stream and returns an int status:
 *
 *     0  TG_OK
 *    -1  TG_ERR_SHAPE      a size or stride the kernel cannot take (see each call)
 *    -2  TG_ERR_ALIGN      a pointer or row pitch is not 16-byte aligned
 *    -3  TG_ERR_ARCH       the current device is not compute capability 10.x
 *    -4  TG_ERR_CUDA       a CUDA runtime/driver call failed (see tg_last_cuda_error)
 *    -5  TG_ERR_TOO_LARGE  a size beyond a stated fixed maximum
 *
 * The caller owns every buffer, including scratch.  No entry point allocates
 * device memory, synchronises the device, or throws across the boundary.  All
 * matrices are row-major and dense unless a leading dimension is passed.
 *
 * "e4m3" is float8_e4m3fn (1-4-3, bias 7, max 448, no infinities), one byte per
 * element.  Scales are float32 and always equal max(amax/448, 1e-30) of their
 * tile, with amax taken over |x| after the upcast of the bf16 input to float32,
 * and q = RNE_e4m3(x / scale) with a true (IEEE) division -- train-gpt fp8.py:39-47.
 *
 * "Reference" below is ammar1510/train-gpt; citations are file:line in that tree.
 */
#ifndef TRAIN_GPT_B200_H_
#define TRAIN_GPT_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TG_OK 0
#define TG_ERR_SHAPE (-1)
#define TG_ERR_ALIGN (-2)
#define TG_ERR_ARCH (-3)
#define TG_ERR_CUDA (-4)
#define TG_ERR_TOO_LARGE (-5)

/* Library version (major*100 + minor). */
int tg_version(void);

/* No counterpart in the reference.  The GEMM is a persistent kernel: one 200 KB thread block per SM
 * for as long as the launch lasts.  A collective that should run BESIDE it (the data-parallel
 * gradient all-reduce overlapping the rest of the backward pass) finds no SM to start on until a
 * GEMM ends, and a GEMM launched after it finds some SMs taken and runs a ragged second wave.
 * Reserving n SMs makes every later GEMM launch of this process use at most (SM count - n) thread
 * blocks.  0 (the default) uses them all; n is clamped to 0 .. 64.  Returns the previous value.
 * Process-wide, host-side only, thread-safe; takes effect at the next launch.                  */
int tg_set_gemm_reserved_sms(int n);

/* Text of the last CUDA error a launcher of this library saw on the calling thread
 * ("" if none).  The pointer stays valid until the next failing call on that thread. */
const char* tg_last_cuda_error(void);

/* ---- quantisers ------------------------------------------------------------------- */

/* Replaces `_quantize_to_fp8(x_f32, 128)` as called on the activation at fp8.py:66
 * (body fp8.py:39-47): tiles of 1 x 128 along the last axis.
 *   x       [rows, cols] bf16          cols % 128 == 0
 *   q       [rows, cols] e4m3
 *   scales  [rows, cols/128] float32                                                  */
int tg_quantize_rowwise(const void* x, void* q, float* scales,
                        int64_t rows, int64_t cols, void* stream);

/* Replaces `_quantize_to_fp8(b.T, 128)` at fp8.py:68 without materialising b.T: tiles
 * of 128 rows x 1 column of x as stored.  q keeps x's layout; the scales come out
 * as [ceil(rows/128), cols] (the transpose of the reference's (N, K/128) array).  A
 * ragged last row block takes amax over the rows that exist.
 *   x [rows, cols] bf16, cols % 8 == 0;  q [rows, cols] e4m3;
 *   scales [ceil(rows/128), cols] float32                                             */
int tg_quantize_colwise(const void* x, void* q, float* scales,
                        int64_t rows, int64_t cols, void* stream);

/* Both of the above in one pass over x, for a tensor that two GEMMs contract along different
 * axes (the upstream gradient g of fp8.py:85-98: along N for dgrad, along the tokens for
 * wgrad): x is read from HBM once.  Outputs are bit-identical to tg_quantize_rowwise and
 * tg_quantize_colwise.
 *   x [rows, cols] bf16, cols % 128 == 0
 *   q_row [rows, cols] e4m3, s_row [rows, cols/128];  q_col [rows, cols] e4m3, s_col [ceil(rows/128), cols] */
int tg_quantize_rowcol(const void* x, void* q_row, float* s_row, void* q_col, float* s_col,
                       int64_t rows, int64_t cols, void* stream);

/* tg_quantize_rowcol with row pitches for all four outputs: row r of q_row starts q_row_ld bytes after
 * row r-1 (>= cols, a multiple of 16), row r of s_row s_row_ld floats after row r-1 (>= cols/128); likewise
 * q_col_ld (bytes, >= cols, multiple of 16) and s_col_ld (floats, >= cols) for the column-wise pair.
 * Lets a caller lay several tensors' quantised forms side by side in one matrix -- the gradients of q, k and
 * v for the single dgrad GEMM that contracts over all three and the single wgrad GEMM that produces all
 * three weight gradients (model.py:63-65 in the backward pass) -- without a copy.  q_row, q_col 8-byte
 * aligned.  No counterpart in the reference. */
int tg_quantize_rowcol_ld(const void* x, void* q_row, int64_t q_row_ld, float* s_row, int64_t s_row_ld,
                          void* q_col, int64_t q_col_ld, float* s_col, int64_t s_col_ld, int64_t rows,
                          int64_t cols, void* stream);

/* tg_quantize_rowcol of an MLP activation that is computed on the fly instead of being read:
 * the squared ReLU of model.py:72 (`jax.nn.relu(h) ** 2`) or the GELU the benchmark's training
 * configuration names, and their cotangents for the backward pass.  `x` is the pre-activation (the
 * up-projection's output); the *_BWD variants also read `gate`, the gradient arriving at the
 * activation's output, and quantise gate * act'(x).  The value is computed in float32 and rounded
 * to bf16 once before the quantisation rule of fp8.py:43-46 is applied, so the outputs equal
 * tg_quantize_rowcol of the bf16 tensor an elementwise kernel would have written.
 *   x, gate [rows, cols] bf16 (gate ignored, may be NULL, for the forward variants), cols % 128 == 0
 *   outputs as tg_quantize_rowcol                                                           */
#define TG_ACT_NONE 0
#define TG_ACT_RELU2 1
#define TG_ACT_GELU 2
#define TG_ACT_RELU2_BWD 3
#define TG_ACT_GELU_BWD 4
int tg_act_quantize_rowcol(const void* x, const void* gate, int act, void* q_row, float* s_row,
                           void* q_col, float* s_col, int64_t rows, int64_t cols, void* stream);

/* Tiles of 128 x 128, one scale per tile: the weight granularity the benchmark
 * configurations name (the reference itself uses tg_quantize_colwise's).  Same scale
 * rule, fp8.py:43-46.
 *   x [rows, cols] bf16, cols % 128 == 0;  q [rows, cols] e4m3;
 *   scales [ceil(rows/128), cols/128] float32                                         */
int tg_quantize_block128(const void* x, void* q, float* scales,
                         int64_t rows, int64_t cols, void* stream);

/* No counterpart in the reference.  The quantisers replace the per-element IEEE division
 * x / scale by one reciprocal per tile and a fused correction step; this runs that
 * shortcut against div.rn.f32 over the COMPLETE input domain (every finite bf16 amax,
 * every bf16 |x| <= amax; 2^31 pairs) on the current device.
 *   counts [4] uint64, device memory: [0] pairs checked, [1] bytes that differ with the
 *   bare x*(1/s), [2] with one correction step (the shipped form -- must be 0), [3] with two. */
int tg_selftest_quantise_division(uint64_t* counts, void* stream);

/* No counterpart in the reference.  Every barrier wait inside tg_gemm_fp8_blockscaled is
 * bounded: a wait that runs out raises a CTA-wide abort flag, stores its role code in the
 * caller's status word, every other role leaves its own wait when it sees the flag, and the
 * CTA frees its tensor memory and returns.  This runs exactly that sequence, with the GEMM's
 * own wait routine and teardown, on a barrier that is never arrived at -- so that the give-up
 * path is exercised without a fault and without hanging the device.
 *   status  device uint32: receives the role code of the wait that ran out (5)
 *   report  device uint32[4]: [0] 0 = the short wait gave up, [1] 2 = the long wait left early
 *           on the abort flag, [2] 1 = an ordinary wait still succeeded, [3] 1 = teardown reached
 *   limit_cycles  the short wait's clock64 limit, 1000 .. 50 000 000 (about 25 ms)          */
int tg_selftest_bounded_wait(uint32_t* status, uint32_t* report, int64_t limit_cycles, void* stream);

/* ---- RMSNorm ---------------------------------------------------------------------- */

/* mode for the norm entry points */
#define TG_NORM_FUSED 0 /* kernels.py:44-53: bf16(f32(x) * rsqrt(var+eps) * f32(gamma)), one rounding */
#define TG_NORM_PURE 1  /* kernels.py:30-33: rsqrt rounded to bf16, two bf16 multiplies              */

/* Replaces `rms_norm(x, scale, eps)` (kernels.py:55-99, variance pass :66 included)
 * or `_rms_norm_pure` (kernels.py:30-33), chosen by `mode`, in ONE pass over x.
 *   x [rows, cols] bf16, gamma [cols] bf16, y [rows, cols] bf16, cols % 8 == 0,
 *   cols <= 8192.  rnorm (may be NULL) [rows] float32 receives rsqrt(var+eps).        */
int tg_rmsnorm_fwd(const void* x, const void* gamma, float eps, void* y, float* rnorm,
                   int64_t rows, int64_t cols, int mode, void* stream);

/* The composition the reference runs between a norm and the GEMM that consumes it --
 * rms_norm (model.py:76-77, kernels.py:44-53) -> upcast (fp8.py:66) -> quantise
 * (fp8.py:39-47) -- as one kernel: x is read once, the normalised value is rounded to
 * bf16 exactly as the reference's norm output is, then quantised per 1 x 128 tile.
 *   x [rows, cols] bf16, gamma [cols] bf16, cols % 128 == 0, cols <= 8192
 *   q [rows, cols] e4m3, scales [rows, cols/128] float32
 *   y     (may be NULL) [rows, cols] bf16: the norm output itself
 *   rnorm (may be NULL) [rows] float32                                                */
int tg_rmsnorm_quant_fwd(const void* x, const void* gamma, float eps, void* q, float* scales,
                         void* y, float* rnorm, int64_t rows, int64_t cols, int mode,
                         void* stream);

/* No counterpart in the reference (XLA fuses the add into the norm's first pass by itself).
 * The residual add of model.py:68 / :72 folded into the norm that follows it:
 *   sum_out = bf16(x + res)  (one rounding, as the elementwise add), then
 *   tg_rmsnorm_quant_fwd of sum_out: q / scales / y / rnorm as there.
 *   x, res, sum_out [rows, cols] bf16 (sum_out may alias x or res); cols % 128 == 0, cols <= 2048
 *   (wider rows: TG_ERR_TOO_LARGE -- add first, then tg_rmsnorm_quant_fwd).
 *   q and scales may both be NULL (a norm without a quantised consumer); then y is required. */
int tg_add_rmsnorm_quant_fwd(const void* x, const void* res, const void* gamma, float eps, void* sum_out,
                             void* q, float* scales, void* y, float* rnorm, int64_t rows, int64_t cols,
                             int mode, void* stream);

/* Bytes of scratch tg_rmsnorm_bwd needs for a [rows, cols] problem (float32 partial
 * column sums, one row of `cols` per thread block). */
int64_t tg_rmsnorm_bwd_scratch_bytes(int64_t rows, int64_t cols);

/* Replaces the custom-VJP `_bwd` of the norm (kernels.py:104-118): recomputes var and
 * rnorm from x, returns dx = bf16(rnorm * (g*gamma - normed * mean(g*gamma*normed)))
 * and dgamma = bf16(sum_rows g * normed).
 *   x, g, dx [rows, cols] bf16; gamma, dgamma [cols] bf16; cols % 8 == 0, cols <= 8192
 *   scratch: tg_rmsnorm_bwd_scratch_bytes(rows, cols) bytes, 16-byte aligned, contents
 *   undefined on entry and exit.  Deterministic (no atomics).                         */
int tg_rmsnorm_bwd(const void* x, const void* gamma, const void* g, float eps, void* dx,
                   void* dgamma, void* scratch, int64_t rows, int64_t cols, void* stream);

/* No counterpart in the reference (autodiff adds the two gradients in a separate pass).
 * tg_rmsnorm_bwd with the gradient fan-in of a residual junction folded in:
 *   dx = bf16(addend + d loss / d x through the norm), one rounding; dgamma as tg_rmsnorm_bwd.
 *   addend [rows, cols] bf16: the gradient arriving over the skip path (dx may alias it).
 *   cols <= 2048 (wider rows: TG_ERR_TOO_LARGE -- tg_rmsnorm_bwd, then add). */
int tg_rmsnorm_bwd_add(const void* x, const void* gamma, const void* g, const void* addend, float eps,
                       void* dx, void* dgamma, void* scratch, int64_t rows, int64_t cols, void* stream);

/* No counterpart in the reference.  The same backward as tg_rmsnorm_bwd for hosts that
 * cannot hand over a scratch buffer because they cannot allocate one: a custom-call
 * handler inside a compiled XLA program gets only the buffers XLA planned, and XLA has
 * usually claimed most of the device already (the reference's launchers give it 90 %),
 * so cudaMalloc there can fail or stall.  The partial column sums go to a 4 MiB array
 * built into the library image (held by every GPU that loads the library, until exit).
 *   - Problems whose tg_rmsnorm_bwd_scratch_bytes(rows, cols) exceeds
 *     tg_rmsnorm_bwd_static_max_scratch_bytes() are refused with TG_ERR_TOO_LARGE and a
 *     message in tg_last_cuda_error(); nothing is launched.  (cols = 2048 fits for any
 *     row count; cols = 4096 does not once rows exceed a few hundred.)
 *   - The first call on each device looks up the array's device address (no allocation);
 *     make that first call outside any stream capture.
 *   - All calls on a device share the one array.  The kernels overwrite what they read,
 *     so nothing needs clearing between calls, but two calls whose kernels can overlap on
 *     the GPU (different streams, no dependency between them) race on it: keep them on
 *     one stream or order them with events.
 *   - Calls no cudaMalloc / cudaFree and no allocating library routine.                  */
int64_t tg_rmsnorm_bwd_static_max_scratch_bytes(void);
int tg_rmsnorm_bwd_static(const void* x, const void* gamma, const void* g, float eps, void* dx,
                          void* dgamma, int64_t rows, int64_t cols, void* stream);

/* ---- capped-logit cross-entropy --------------------------------------------------- */

/* train-gpt model.py:97 (`cap * tanh(logits / cap)`, bf16, every op rounding) followed by
 * losses.py:9-12 (float32 log_softmax over the vocabulary, gather of the target, per-token
 * negative log-likelihood; the caller takes the mean).  One pass over the logits.
 *   logits   bf16 [rows, ld], the unembedding GEMM's output, vocab <= ld
 *   targets  int32 [rows]; values outside [0, vocab) clamp, as jnp.take_along_axis does
 *   tanh_out bf16 [rows, ld_tanh] or NULL: bf16(tanh(bf16(logits / cap))), what the backward
 *            needs (cap * tanh_out, rounded to bf16, is the capped logits model.forward returns)
 *   lse, nll float32 [rows]: logsumexp of the capped logits, and lse - capped[target]
 *   ld, ld_tanh multiples of 8 (16-byte row pitch); pointers 16-byte aligned.  vocab itself
 *   may be any positive size (train-gpt's default is 50257, config.py:8): the columns
 *   between vocab and the row pitch are read but take no part and are never written.       */
int tg_softcap_ce_fwd(const void* logits, const int32_t* targets, float cap, void* tanh_out, float* lse,
                      float* nll, int64_t rows, int64_t vocab, int64_t ld, int64_t ld_tanh, void* stream);

/* The gradient of mean(nll) with respect to the uncapped logits (the reference gets it from
 * jax.value_and_grad through losses.py:8-12 and model.py:97, train.py:129):
 *   dlogits = gscale / rows * (softmax(capped) - onehot(target)) * (1 - tanh^2), bf16.
 *   gscale  device float32 scalar (the cotangent of the mean loss) or NULL for 1
 *   dlogits bf16 [rows, ld_d]; may be the very buffer tanh_in points to (in place).       */
int tg_softcap_ce_bwd(const void* tanh_in, const int32_t* targets, const float* lse, const float* gscale,
                      float cap, void* dlogits, int64_t rows, int64_t vocab, int64_t ld_tanh, int64_t ld_d,
                      void* stream);

/* ---- optimiser step --------------------------------------------------------------- */

/* Sum of squares of n bf16 values into out[0] (float32): one term of optax.global_norm
 * (train-gpt train.py:132).  scratch: tg_sumsq_scratch_bytes() bytes, caller-owned.  Block
 * partials are added in index order, so the result does not depend on scheduling.       */
int64_t tg_sumsq_scratch_bytes(void);
int tg_sumsq_bf16(const void* x, int64_t n, float* out, void* scratch, void* stream);

/* One step of optax.chain(clip_by_global_norm, adamw) (train-gpt train.py:120-123,133-134) on n
 * bf16 parameters with bf16 moments, in place:
 *   g' = bf16(g * gscale);  m = bf16(b1 m + (1-b1) g');  v = bf16(b2 v + (1-b2) g'^2);
 *   p = bf16(p - lr * ((m / (1 - b1^t)) / (sqrt(v / (1 - b2^t)) + eps) + weight_decay * p)).
 *   step   device int32: t, the number of this step (1 for the first); a device word so that a
 *          captured CUDA graph can be replayed with a counter the caller increments
 *   gscale device float32 clip factor min(1, clip / global_norm), or NULL for 1           */
int tg_adamw_bf16(void* p, const void* g, void* m, void* v, int64_t n, float lr, float b1, float b2,
                  float eps, float weight_decay, const int32_t* step, const float* gscale, void* stream);

/* ---- block-scaled FP8 GEMM -------------------------------------------------------- */

/* Operand storage, seen from the GEMM  D[m,n] = sum_k A[m,k] * B[n,k]. */
#define TG_MAJOR_K 0  /* the operand is stored [m or n][k], k contiguous  */
#define TG_MAJOR_MN 1 /* the operand is stored [k][m or n], m/n contiguous */

#define TG_OUT_BF16 0
#define TG_OUT_F32 1

typedef struct tg_gemm_args {
  /* D[m,n] = sum_kb SA(m,kb) * SB(n,kb) * sum_{k in block kb} A[m,k] * B[n,k]
   * with 128-element contraction blocks, e4m3 operands, float32 accumulation.        */
  const void* a;    /* e4m3; [M, K] if a_major == TG_MAJOR_K else [K, M]               */
  const void* b;    /* e4m3; [N, K] if b_major == TG_MAJOR_K else [K, N]               */
  int64_t lda, ldb; /* row pitch of a / b in elements (bytes); multiple of 16          */
  int a_major, b_major;
  const float* sa;  /* SA(m,kb) = sa[m*sa_stride_m + kb*sa_stride_kb]                  */
  int64_t sa_stride_m, sa_stride_kb;
  const float* sb;  /* SB(n,kb) = sb[(n/sb_gran_n)*sb_stride_n + kb*sb_stride_kb]      */
  int64_t sb_stride_n, sb_stride_kb;
  int sb_gran_n;    /* 1 (a scale per column n) or 128 (a scale per 128 columns)       */
  void* d;          /* [M, N] bf16 or float32                                          */
  int64_t ldd;      /* row pitch of d in elements; multiple of 8                       */
  int out_dtype;    /* TG_OUT_BF16 / TG_OUT_F32                                        */
  int64_t M, N, K;  /* K = contraction length; a ragged K (K % 128 != 0) is allowed
                       only for MN-major operands whose scales were made by
                       tg_quantize_colwise over the same ragged length                 */
  uint32_t* status; /* device word, must be 0 on entry; a kernel whose bounded wait on
                       a copy or MMA barrier runs out stores a non-zero code here and
                       returns (results are then invalid).  May be NULL.              */
  void* workspace;  /* optional, caller-owned, 16-byte aligned.  With at least
                       tg_gemm_workspace_bytes() bytes here, a GEMM with few output tiles
                       and a long contraction (the weight gradient) is cut along the
                       contraction so that all SMs work; float32 partial sums go here and
                       are added in a fixed order.  NULL or too small: no cut.           */
  int64_t workspace_bytes;
} tg_gemm_args;

/* Bytes of workspace with which tg_gemm_fp8_blockscaled would cut this problem's contraction
 * (0 when it would not).  No counterpart in the reference.                              */
int64_t tg_gemm_workspace_bytes(const tg_gemm_args* a);

/* Replaces `jax.nn.scaled_matmul` as called at fp8.py:70-76 (lhs (M,K), rhs (N,K),
 * scales per 128 of K) followed by the bf16 cast of fp8.py:78 -- and, with other
 * operand orders, the two backward GEMMs of fp8.py:96-97 in FP8:
 *   forward  y  = x W      A = x_q  [M,K] K-major,  B = W_q [K,N] MN-major
 *   dgrad    dx = g W^T    A = g_q  [M,N] K-major,  B = W_q [K,N] K-major (contracts N)
 *   wgrad    dW = x^T g    A = x_q  [T,K] MN-major, B = g_q [T,N] MN-major (contracts T)
 * No operand is transposed in memory: the TMA descriptors and the tcgen05 operand
 * descriptors carry the orientation.                                                 */
int tg_gemm_fp8_blockscaled(const tg_gemm_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TRAIN_GPT_B200_H_ */
