// XLA FFI handlers over the C ABI of libtrain_gpt_b200.so: what train-gpt's JAX code binds with
// jax.ffi.register_ffi_target / jax.ffi.ffi_call in place of jax.nn.scaled_matmul (fp8.py:70-76),
// the XLA quantisation fusions (fp8.py:39-47) and the Pallas norm (kernels.py:87-97).
//
// One handler per kernel entry point of include/train_gpt_b200.h; each is a thin adapter from
// XLA's buffers to one C call, on the stream XLA hands over.  Nothing here allocates: scratch and
// workspace arrive as extra result buffers that XLA plans, the status word as a result buffer
// the handler zeroes itself.
//
// Build (needs the XLA FFI headers that ship with jaxlib; see build.py next to this file):
//   g++ -O2 -std=c++17 -shared -fPIC -I$(python -c 'import jax.ffi; print(jax.ffi.include_dir())')
//       -I<repo>/include -I/usr/local/cuda/include xla_ffi.cc -L<repo>/train_gpt_b200
//       -ltrain_gpt_b200 -lcudart -o libtg_xla.so
#include <cuda_runtime_api.h>

#include <cstdint>
#include <string>

#include "train_gpt_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

using Stream = ffi::PlatformStream<cudaStream_t>;
using BF16 = ffi::Buffer<ffi::BF16>;
using F8 = ffi::Buffer<ffi::F8E4M3FN>;
using F32 = ffi::Buffer<ffi::F32>;
using S32 = ffi::Buffer<ffi::S32>;
using U8 = ffi::Buffer<ffi::U8>;
using U32 = ffi::Buffer<ffi::U32>;
using RBF16 = ffi::ResultBuffer<ffi::BF16>;
using RF8 = ffi::ResultBuffer<ffi::F8E4M3FN>;
using RF32 = ffi::ResultBuffer<ffi::F32>;
using RU8 = ffi::ResultBuffer<ffi::U8>;
using RU32 = ffi::ResultBuffer<ffi::U32>;

ffi::Error Check(int rc, const char* what) {
  if (rc == TG_OK) return ffi::Error::Success();
  const std::string msg = std::string(what) + " returned " + std::to_string(rc) +
                          (rc == TG_ERR_CUDA ? std::string(": ") + tg_last_cuda_error() : std::string());
  return ffi::Error(rc == TG_ERR_CUDA ? ffi::ErrorCode::kInternal : ffi::ErrorCode::kInvalidArgument, msg);
}

// rows x cols of a buffer whose last axis is the feature axis (leading axes are flattened,
// as fp8.py:65 and kernels.py:60-62 do)
template <typename B>
void RowsCols(const B& x, int64_t* rows, int64_t* cols) {
  auto d = x.dimensions();
  *cols = d.size() ? d.back() : 1;
  *rows = *cols ? static_cast<int64_t>(x.element_count()) / *cols : 0;
}

// ---- quantisers (fp8.py:39-47) ----------------------------------------------------------------

ffi::Error QuantizeRowwise(cudaStream_t s, BF16 x, RF8 q, RF32 scales) {
  int64_t rows, cols;
  RowsCols(x, &rows, &cols);
  return Check(tg_quantize_rowwise(x.untyped_data(), q->untyped_data(), scales->typed_data(), rows, cols, s),
               "tg_quantize_rowwise");
}

ffi::Error QuantizeColwise(cudaStream_t s, BF16 x, RF8 q, RF32 scales) {
  auto d = x.dimensions();
  if (d.size() != 2) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "TgQuantizeColwise takes a 2-D operand");
  return Check(tg_quantize_colwise(x.untyped_data(), q->untyped_data(), scales->typed_data(), d[0], d[1], s),
               "tg_quantize_colwise");
}

ffi::Error QuantizeRowcol(cudaStream_t s, BF16 x, RF8 q_row, RF32 s_row, RF8 q_col, RF32 s_col) {
  auto d = x.dimensions();
  if (d.size() != 2) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "TgQuantizeRowcol takes a 2-D operand");
  return Check(tg_quantize_rowcol(x.untyped_data(), q_row->untyped_data(), s_row->typed_data(), q_col->untyped_data(),
                                  s_col->typed_data(), d[0], d[1], s),
               "tg_quantize_rowcol");
}

// Both forms go into columns [col0, col0 + cols) of wider matrices that several calls fill side by side (the
// gradients of q, k and v for the one dgrad GEMM that contracts over all of them and the one wgrad GEMM that
// produces all three weight gradients).  XLA has no strided results: the four wide matrices come in as operands
// and go out as results aliased to them (input_output_aliases={1: 0, 2: 1, 3: 2, 4: 3} on the JAX side), so
// every call writes its slices in place.
ffi::Error QuantizeRowcolInto(cudaStream_t s, BF16 x, F8 wide_q_in, F32 wide_s_in, F8 wide_qc_in, F32 wide_sc_in, RF8 wide_q,
                              RF32 wide_s, RF8 wide_qc, RF32 wide_sc, int64_t col0) {
  auto d = x.dimensions();
  auto wq = wide_q->dimensions();
  auto ws = wide_s->dimensions();
  auto wqc = wide_qc->dimensions();
  auto wsc = wide_sc->dimensions();
  if (d.size() != 2 || wq.size() != 2 || ws.size() != 2 || wqc.size() != 2 || wsc.size() != 2 || wq[0] != d[0] ||
      ws[0] != d[0] || wqc[0] != d[0] || wsc[0] != (d[0] + 127) / 128 || col0 < 0 || col0 % 128 != 0 ||
      col0 + d[1] > wq[1] || (col0 + d[1]) / 128 > ws[1] || col0 + d[1] > wqc[1] || col0 + d[1] > wsc[1])
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "TgQuantizeRowcolInto: the slice does not fit the wide matrices");
  if (wide_q_in.untyped_data() != wide_q->untyped_data() || wide_s_in.untyped_data() != wide_s->untyped_data() ||
      wide_qc_in.untyped_data() != wide_qc->untyped_data() || wide_sc_in.untyped_data() != wide_sc->untyped_data())
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "TgQuantizeRowcolInto: declare input_output_aliases={1: 0, 2: 1, 3: 2, 4: 3}");
  return Check(tg_quantize_rowcol_ld(x.untyped_data(), static_cast<uint8_t*>(wide_q->untyped_data()) + col0, wq[1],
                                     wide_s->typed_data() + col0 / 128, ws[1],
                                     static_cast<uint8_t*>(wide_qc->untyped_data()) + col0, wqc[1],
                                     wide_sc->typed_data() + col0, wsc[1], d[0], d[1], s),
               "tg_quantize_rowcol_ld");
}

// act: TG_ACT_RELU2 / TG_ACT_GELU
ffi::Error ActQuantizeRowcol(cudaStream_t s, BF16 x, RF8 q_row, RF32 s_row, RF8 q_col, RF32 s_col, int32_t act) {
  auto d = x.dimensions();
  if (d.size() != 2) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "TgActQuantizeRowcol takes a 2-D operand");
  return Check(tg_act_quantize_rowcol(x.untyped_data(), nullptr, act, q_row->untyped_data(), s_row->typed_data(),
                                      q_col->untyped_data(), s_col->typed_data(), d[0], d[1], s),
               "tg_act_quantize_rowcol");
}

// act: TG_ACT_RELU2_BWD / TG_ACT_GELU_BWD; gate = the gradient arriving at the activation's output
ffi::Error ActQuantizeRowcolBwd(cudaStream_t s, BF16 x, BF16 gate, RF8 q_row, RF32 s_row, RF8 q_col, RF32 s_col,
                                int32_t act) {
  auto d = x.dimensions();
  if (d.size() != 2) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "TgActQuantizeRowcolBwd takes 2-D operands");
  return Check(tg_act_quantize_rowcol(x.untyped_data(), gate.untyped_data(), act, q_row->untyped_data(),
                                      s_row->typed_data(), q_col->untyped_data(), s_col->typed_data(), d[0], d[1], s),
               "tg_act_quantize_rowcol");
}

ffi::Error QuantizeBlock128(cudaStream_t s, BF16 x, RF8 q, RF32 scales) {
  auto d = x.dimensions();
  if (d.size() != 2) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "TgQuantizeBlock128 takes a 2-D operand");
  return Check(tg_quantize_block128(x.untyped_data(), q->untyped_data(), scales->typed_data(), d[0], d[1], s),
               "tg_quantize_block128");
}

// ---- RMSNorm (kernels.py:30-33, 44-99, 104-118) -------------------------------------------------

ffi::Error RmsnormFwd(cudaStream_t s, BF16 x, BF16 gamma, RBF16 y, RF32 rnorm, float eps, int32_t mode) {
  int64_t rows, cols;
  RowsCols(x, &rows, &cols);
  return Check(tg_rmsnorm_fwd(x.untyped_data(), gamma.untyped_data(), eps, y->untyped_data(), rnorm->typed_data(), rows,
                              cols, mode, s),
               "tg_rmsnorm_fwd");
}

ffi::Error RmsnormQuantFwd(cudaStream_t s, BF16 x, BF16 gamma, RF8 q, RF32 scales, RBF16 y, RF32 rnorm, float eps,
                           int32_t mode) {
  int64_t rows, cols;
  RowsCols(x, &rows, &cols);
  return Check(tg_rmsnorm_quant_fwd(x.untyped_data(), gamma.untyped_data(), eps, q->untyped_data(), scales->typed_data(),
                                    y->untyped_data(), rnorm->typed_data(), rows, cols, mode, s),
               "tg_rmsnorm_quant_fwd");
}

// the residual add folded into the norm that follows it (model.py:68 / :72 then :76-77); rows of at most 2048
ffi::Error AddRmsnormQuantFwd(cudaStream_t s, BF16 x, BF16 res, BF16 gamma, RBF16 sum, RF8 q, RF32 scales, RBF16 y, RF32 rnorm,
                              float eps, int32_t mode) {
  int64_t rows, cols;
  RowsCols(x, &rows, &cols);
  return Check(tg_add_rmsnorm_quant_fwd(x.untyped_data(), res.untyped_data(), gamma.untyped_data(), eps, sum->untyped_data(),
                                        q->untyped_data(), scales->typed_data(), y->untyped_data(), rnorm->typed_data(), rows,
                                        cols, mode, s),
               "tg_add_rmsnorm_quant_fwd");
}

// scratch: a result buffer of tg_rmsnorm_bwd_scratch_bytes(rows, cols) bytes that XLA plans
ffi::Error RmsnormBwd(cudaStream_t s, BF16 x, BF16 gamma, BF16 g, RBF16 dx, RBF16 dgamma, RU8 scratch, float eps) {
  int64_t rows, cols;
  RowsCols(x, &rows, &cols);
  if (static_cast<int64_t>(scratch->element_count()) < tg_rmsnorm_bwd_scratch_bytes(rows, cols))
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "TgRmsnormBwd: scratch result smaller than tg_rmsnorm_bwd_scratch_bytes");
  return Check(tg_rmsnorm_bwd(x.untyped_data(), gamma.untyped_data(), g.untyped_data(), eps, dx->untyped_data(),
                              dgamma->untyped_data(), scratch->untyped_data(), rows, cols, s),
               "tg_rmsnorm_bwd");
}

// the backward with the skip path's gradient added in the same pass; rows of at most 2048
ffi::Error RmsnormBwdAdd(cudaStream_t s, BF16 x, BF16 gamma, BF16 g, BF16 addend, RBF16 dx, RBF16 dgamma, RU8 scratch, float eps) {
  int64_t rows, cols;
  RowsCols(x, &rows, &cols);
  if (static_cast<int64_t>(scratch->element_count()) < tg_rmsnorm_bwd_scratch_bytes(rows, cols))
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "TgRmsnormBwdAdd: scratch result smaller than tg_rmsnorm_bwd_scratch_bytes");
  return Check(tg_rmsnorm_bwd_add(x.untyped_data(), gamma.untyped_data(), g.untyped_data(), addend.untyped_data(), eps,
                                  dx->untyped_data(), dgamma->untyped_data(), scratch->untyped_data(), rows, cols, s),
               "tg_rmsnorm_bwd_add");
}

// the same backward with the scratch inside the library (fixed 4 MiB array; see the header)
ffi::Error RmsnormBwdStatic(cudaStream_t s, BF16 x, BF16 gamma, BF16 g, RBF16 dx, RBF16 dgamma, float eps) {
  int64_t rows, cols;
  RowsCols(x, &rows, &cols);
  return Check(tg_rmsnorm_bwd_static(x.untyped_data(), gamma.untyped_data(), g.untyped_data(), eps, dx->untyped_data(),
                                     dgamma->untyped_data(), rows, cols, s),
               "tg_rmsnorm_bwd_static");
}

// ---- capped-logit cross-entropy (model.py:97, losses.py:8-12) -------------------------------------

// logits (rows, ld) with ld a multiple of 8 >= vocab (pad on the JAX side for a ragged vocabulary)
ffi::Error SoftcapCeFwd(cudaStream_t s, BF16 logits, S32 targets, RBF16 tanh_out, RF32 lse, RF32 nll, float cap,
                        int64_t vocab) {
  int64_t rows, ld;
  RowsCols(logits, &rows, &ld);
  return Check(tg_softcap_ce_fwd(logits.untyped_data(), targets.typed_data(), cap, tanh_out->untyped_data(),
                                 lse->typed_data(), nll->typed_data(), rows, vocab, ld, ld, s),
               "tg_softcap_ce_fwd");
}

// dlogits may alias tanh_in (declare input_output_aliases={0: 0} on the JAX side)
ffi::Error SoftcapCeBwd(cudaStream_t s, BF16 tanh_in, S32 targets, F32 lse, F32 gscale, RBF16 dlogits, float cap,
                        int64_t vocab) {
  int64_t rows, ld;
  RowsCols(tanh_in, &rows, &ld);
  return Check(tg_softcap_ce_bwd(tanh_in.untyped_data(), targets.typed_data(), lse.typed_data(), gscale.typed_data(), cap,
                                 dlogits->untyped_data(), rows, vocab, ld, ld, s),
               "tg_softcap_ce_bwd");
}

// ---- optimiser (train.py:114-123, 132-134) --------------------------------------------------------

ffi::Error SumsqBf16(cudaStream_t s, BF16 x, RF32 out, RU8 scratch) {
  if (static_cast<int64_t>(scratch->element_count()) < tg_sumsq_scratch_bytes())
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "TgSumsqBf16: scratch result smaller than tg_sumsq_scratch_bytes");
  return Check(tg_sumsq_bf16(x.untyped_data(), static_cast<int64_t>(x.element_count()), out->typed_data(),
                             scratch->untyped_data(), s),
               "tg_sumsq_bf16");
}

// p, m, v are updated in place: bind with input_output_aliases={0: 0, 2: 1, 3: 2}
ffi::Error AdamwBf16(cudaStream_t s, BF16 p, BF16 g, BF16 m, BF16 v, S32 step, F32 gscale, RBF16 p_out, RBF16 m_out,
                     RBF16 v_out, float lr, float b1, float b2, float eps, float weight_decay) {
  if (p_out->untyped_data() != p.untyped_data() || m_out->untyped_data() != m.untyped_data() ||
      v_out->untyped_data() != v.untyped_data())
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "TgAdamwBf16 updates in place: alias p, m, v to the results");
  return Check(tg_adamw_bf16(p_out->untyped_data(), g.untyped_data(), m_out->untyped_data(), v_out->untyped_data(),
                             static_cast<int64_t>(p.element_count()), lr, b1, b2, eps, weight_decay, step.typed_data(),
                             gscale.typed_data(), s),
               "tg_adamw_bf16");
}

// ---- block-scaled GEMM (fp8.py:70-78 and the FP8 form of fp8.py:96-97) ------------------------------

// Common tail: zero the status word, attach the workspace XLA planned (may be empty), launch.
ffi::Error LaunchGemm(cudaStream_t s, tg_gemm_args* g, RU32& status, RU8& workspace) {
  if (cudaMemsetAsync(status->typed_data(), 0, sizeof(uint32_t), s) != cudaSuccess)
    return ffi::Error(ffi::ErrorCode::kInternal, "cudaMemsetAsync(status) failed");
  g->status = status->typed_data();
  const int64_t need = tg_gemm_workspace_bytes(g);
  if (need > 0 && static_cast<int64_t>(workspace->element_count()) >= need) {
    g->workspace = workspace->untyped_data();
    g->workspace_bytes = static_cast<int64_t>(workspace->element_count());
  }
  return Check(tg_gemm_fp8_blockscaled(g, s), "tg_gemm_fp8_blockscaled");
}

// y = x W.  a (M, K) row-wise quantised, sa (M, K/128); b (K, N) as stored (no b.T), sb (K/128, N) for
// weight_gran 1 [the reference's granularity] or (K/128, N/128) for weight_gran 128.
ffi::Error GemmFwd(cudaStream_t s, F8 a, F32 sa, F8 b, F32 sb, RBF16 y, RU32 status, RU8 workspace, int32_t weight_gran) {
  const int64_t M = a.dimensions()[0], K = a.dimensions()[1], N = b.dimensions()[1];
  tg_gemm_args g = {};
  g.a = a.untyped_data(); g.lda = K; g.a_major = TG_MAJOR_K;
  g.b = b.untyped_data(); g.ldb = N; g.b_major = TG_MAJOR_MN;
  g.sa = sa.typed_data(); g.sa_stride_m = sa.dimensions()[1]; g.sa_stride_kb = 1;
  g.sb = sb.typed_data(); g.sb_stride_n = 1; g.sb_stride_kb = sb.dimensions()[1]; g.sb_gran_n = weight_gran;
  g.d = y->untyped_data(); g.ldd = N; g.out_dtype = TG_OUT_BF16;
  g.M = M; g.N = N; g.K = K;
  return LaunchGemm(s, &g, status, workspace);
}

// dx = g W^T (contracts N).  g (M, N) row-wise quantised, sg (M, N/128); w (K, N) quantised along N:
// sw (K, N/128) for weight_gran 1, or the forward's (K/128, N/128) tiles for weight_gran 128.
ffi::Error GemmDgrad(cudaStream_t s, F8 gq, F32 sg, F8 w, F32 sw, RBF16 dx, RU32 status, RU8 workspace,
                     int32_t weight_gran) {
  const int64_t M = gq.dimensions()[0], N = gq.dimensions()[1], K = w.dimensions()[0];
  tg_gemm_args g = {};
  g.a = gq.untyped_data(); g.lda = N; g.a_major = TG_MAJOR_K;
  g.b = w.untyped_data(); g.ldb = N; g.b_major = TG_MAJOR_K;
  g.sa = sg.typed_data(); g.sa_stride_m = sg.dimensions()[1]; g.sa_stride_kb = 1;
  g.sb = sw.typed_data(); g.sb_stride_n = sw.dimensions()[1]; g.sb_stride_kb = 1; g.sb_gran_n = weight_gran;
  g.d = dx->untyped_data(); g.ldd = K; g.out_dtype = TG_OUT_BF16;
  g.M = M; g.N = K; g.K = N;
  return LaunchGemm(s, &g, status, workspace);
}

// dW = x^T g (contracts the tokens).  x (T, K) and g (T, N) column-wise quantised (128 tokens x 1):
// sx (ceil(T/128), K), sg (ceil(T/128), N) for grad_gran 1 or (ceil(T/128), N/128) for grad_gran 128.
ffi::Error GemmWgrad(cudaStream_t s, F8 xq, F32 sx, F8 gq, F32 sg, RBF16 dw, RU32 status, RU8 workspace,
                     int32_t grad_gran) {
  const int64_t T = xq.dimensions()[0], K = xq.dimensions()[1], N = gq.dimensions()[1];
  tg_gemm_args g = {};
  g.a = xq.untyped_data(); g.lda = K; g.a_major = TG_MAJOR_MN;
  g.b = gq.untyped_data(); g.ldb = N; g.b_major = TG_MAJOR_MN;
  g.sa = sx.typed_data(); g.sa_stride_m = 1; g.sa_stride_kb = K;
  g.sb = sg.typed_data(); g.sb_stride_n = 1; g.sb_stride_kb = sg.dimensions()[1]; g.sb_gran_n = grad_gran;
  g.d = dw->untyped_data(); g.ldd = N; g.out_dtype = TG_OUT_BF16;
  g.M = K; g.N = N; g.K = T;
  return LaunchGemm(s, &g, status, workspace);
}

}  // namespace

#define TG_QUANT_BINDING ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Ret<F8>().Ret<F32>()

XLA_FFI_DEFINE_HANDLER_SYMBOL(TgQuantizeRowwise, QuantizeRowwise, TG_QUANT_BINDING);
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgQuantizeColwise, QuantizeColwise, TG_QUANT_BINDING);
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgQuantizeBlock128, QuantizeBlock128, TG_QUANT_BINDING);
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgQuantizeRowcol, QuantizeRowcol,
                              ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Ret<F8>().Ret<F32>().Ret<F8>().Ret<F32>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgQuantizeRowcolInto, QuantizeRowcolInto,
                              ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Arg<F8>().Arg<F32>().Arg<F8>().Arg<F32>()
                                  .Ret<F8>().Ret<F32>().Ret<F8>().Ret<F32>().Attr<int64_t>("col0"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgActQuantizeRowcol, ActQuantizeRowcol,
                              ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Ret<F8>().Ret<F32>().Ret<F8>().Ret<F32>()
                                  .Attr<int32_t>("act"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgActQuantizeRowcolBwd, ActQuantizeRowcolBwd,
                              ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Arg<BF16>().Ret<F8>().Ret<F32>().Ret<F8>().Ret<F32>()
                                  .Attr<int32_t>("act"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgRmsnormFwd, RmsnormFwd,
                              ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Arg<BF16>().Ret<BF16>().Ret<F32>()
                                  .Attr<float>("eps").Attr<int32_t>("mode"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgRmsnormQuantFwd, RmsnormQuantFwd,
                              ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Arg<BF16>().Ret<F8>().Ret<F32>().Ret<BF16>().Ret<F32>()
                                  .Attr<float>("eps").Attr<int32_t>("mode"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgAddRmsnormQuantFwd, AddRmsnormQuantFwd,
                              ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Arg<BF16>().Arg<BF16>().Ret<BF16>().Ret<F8>().Ret<F32>()
                                  .Ret<BF16>().Ret<F32>().Attr<float>("eps").Attr<int32_t>("mode"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgRmsnormBwdAdd, RmsnormBwdAdd,
                              ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Arg<BF16>().Arg<BF16>().Arg<BF16>().Ret<BF16>().Ret<BF16>()
                                  .Ret<U8>().Attr<float>("eps"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgRmsnormBwd, RmsnormBwd,
                              ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Arg<BF16>().Arg<BF16>().Ret<BF16>().Ret<BF16>().Ret<U8>()
                                  .Attr<float>("eps"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgRmsnormBwdStatic, RmsnormBwdStatic,
                              ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Arg<BF16>().Arg<BF16>().Ret<BF16>().Ret<BF16>()
                                  .Attr<float>("eps"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgSoftcapCeFwd, SoftcapCeFwd,
                              ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Arg<S32>().Ret<BF16>().Ret<F32>().Ret<F32>()
                                  .Attr<float>("cap").Attr<int64_t>("vocab"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgSoftcapCeBwd, SoftcapCeBwd,
                              ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Arg<S32>().Arg<F32>().Arg<F32>().Ret<BF16>()
                                  .Attr<float>("cap").Attr<int64_t>("vocab"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgSumsqBf16, SumsqBf16, ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Ret<F32>().Ret<U8>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgAdamwBf16, AdamwBf16,
                              ffi::Ffi::Bind().Ctx<Stream>().Arg<BF16>().Arg<BF16>().Arg<BF16>().Arg<BF16>().Arg<S32>().Arg<F32>()
                                  .Ret<BF16>().Ret<BF16>().Ret<BF16>()
                                  .Attr<float>("lr").Attr<float>("b1").Attr<float>("b2").Attr<float>("eps")
                                  .Attr<float>("weight_decay"));

#define TG_GEMM_BINDING(attr) \
  ffi::Ffi::Bind().Ctx<Stream>().Arg<F8>().Arg<F32>().Arg<F8>().Arg<F32>().Ret<BF16>().Ret<U32>().Ret<U8>().Attr<int32_t>(attr)

XLA_FFI_DEFINE_HANDLER_SYMBOL(TgGemmFwd, GemmFwd, TG_GEMM_BINDING("weight_gran"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgGemmDgrad, GemmDgrad, TG_GEMM_BINDING("weight_gran"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TgGemmWgrad, GemmWgrad, TG_GEMM_BINDING("grad_gran"));
