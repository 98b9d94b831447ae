// Capped-logit cross-entropy, forward and backward, one pass over the logits each.
//
// Reference semantics: train-gpt model.py:97 (`cap * tanh(logits / cap)` on the bf16 output of
// the unembedding GEMM, every op rounding to bf16, the Python-float cap weakly typed = bf16)
// followed by losses.py:9-12 (cast to float32, log_softmax over the vocabulary, gather the
// target's log-probability, mean over tokens).  Done op by op that is five elementwise passes
// and two softmax passes over a (tokens x vocab) tensor (3.3 GB in bf16 at 32768 x 50304, twice
// that in float32); here the forward reads the logits once and writes the bf16 tanh values,
// and the backward turns those into the logits' gradient in place.
//
// Layout: one thread block per token row; each thread walks the row in 16-byte pieces (8 bf16)
// and keeps a running (max, sum of exp) pair; the block combines the pairs.
#include <algorithm>

#include "common.cuh"

namespace tg {

constexpr int kLossThreads = 256;

// RN_bf16(v) as a float
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

struct Softcap {
  float c, r;   // the cap rounded to bf16, and RN(1/c)
  __device__ __forceinline__ explicit Softcap(float cap) {
    c = round_bf16(cap);
    r = __frcp_rn(c);
  }
  __device__ __forceinline__ float z_of_tanh(float t) const { return round_bf16(__fmul_rn(c, t)); }
  // bf16(x / c) as a float: the division is q0 = x*r, q = fma(-fma(q0, c, -x), r, q0), which is
  // the correctly rounded quotient when r is the correctly rounded reciprocal (Markstein); the
  // residual is taken as q0*c - x and subtracted so that x = -0 stays -0
  __device__ __forceinline__ float quotient(float x) const {
    const float q0 = __fmul_rn(x, r);
    return round_bf16(__fmaf_rn(-__fmaf_rn(q0, c, -x), r, q0));
  }
};

// bf16(tanh(a)) for a bf16 argument needs no evaluation outside 2^-6 <= |a| < 4: below, tanh(a)
// differs from a by less than a^2/3 <= 2^-13.6 relative, far inside half a bf16 ulp (>= 2^-10), so
// the result is a itself; from 4 on, 1 - tanh(a) <= 6.8e-4 < 2^-9, so it rounds to +-1.  The 1024
// arguments in between (8 binades x 128 mantissas) are evaluated with tanhf.  A thread block keeps
// the result for EVERY magnitude (32768 two-byte entries, index = the bf16 bits without the sign; a
// NaN maps to itself) in shared memory, so that the per-element work is one load and a sign merge, with no
// range tests; blocks are persistent (each walks many rows), so the fill is paid once per block.
constexpr uint32_t kTanhLo = (127u - 6u) << 7;   // bf16 magnitude bits of 2^-6
constexpr uint32_t kTanhHi = (127u + 2u) << 7;   // ... of 4.0
constexpr int kTanhEntries = 32768;
constexpr int kTanhBytes = kTanhEntries * 2;

__device__ __forceinline__ uint32_t tanh_bits_of_magnitude(uint32_t mag) {
  if (mag < kTanhLo || mag > 0x7f80u) return mag;                 // tiny (or NaN): tanh(a) rounds to a
  if (mag >= kTanhHi) return 0x3f80u;                             // 1
  return __float_as_uint(round_bf16(tanhf(__uint_as_float(mag << 16)))) >> 16;
}
__device__ __forceinline__ void tanh_table_fill(uint16_t* table) {
  for (int i = threadIdx.x; i < kTanhEntries; i += blockDim.x) table[i] = uint16_t(tanh_bits_of_magnitude(uint32_t(i)));
}
// a: a bf16 value held in a float (the scalar form: the target's own logit, once per row)
__device__ __forceinline__ float tanh_bf16(float a) {
  const uint32_t bits = __float_as_uint(a);
  return __uint_as_float((bits & 0x80000000u) | (tanh_bits_of_magnitude((bits >> 16) & 0x7fffu) << 16));
}

// (m, s) <- combine with (m2, s2): s counts exp(z - m)
__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
  const float mn = fmaxf(m, m2);
  s = s * __expf(m - mn) + s2 * __expf(m2 - mn);
  m = mn;
}

// The forward is bound by instruction issue, not by DRAM, so the element work is written in packed
// f32x2 operations on the two halves of each loaded word: the exact quotient x / c (one reciprocal multiply and one
// correction step, as in the quantisers), one rounding to a bf16 pair, two table loads, the cap multiply and its
// rounding, and the online softmax.
// 512 threads, three blocks per SM (the table is 64 KB): 1.57 ms at 32768 x 50304 (1.50 with the prefetch below); 256 / 384 / 768
// threads measured 1.98 / 1.66 / 1.65
constexpr int kLossFwdThreads = 512;

__global__ void __launch_bounds__(kLossFwdThreads)
softcap_ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const int32_t* __restrict__ targets, float cap,
                      __nv_bfloat16* __restrict__ tanh_out, float* __restrict__ lse_out, float* __restrict__ nll_out,
                      int rows, int vocab, int64_t ld, int64_t ld_t) {
  __shared__ float s_m[kLossFwdThreads / 32], s_s[kLossFwdThreads / 32];
  extern __shared__ __align__(16) uint16_t s_tanh[];
  tanh_table_fill(s_tanh);
  __syncthreads();
  const Softcap sc(cap);
  const float2 c2 = make_float2(sc.c, sc.c), nr2 = make_float2(-sc.r, -sc.r);
  const float2 l2e = make_float2(1.4426950408889634f, 1.4426950408889634f);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* p = logits + row * ld;
    float m = -3.0e38f, s = 0.f;
    // the next piece is loaded before this one is worked on: the kernel's top stall was the wait for its
    // one 16-byte load per thread
    uint4 w_next = threadIdx.x * 8 < vocab ? ld_nc_v4(p + threadIdx.x * 8) : make_uint4(0u, 0u, 0u, 0u);
    for (int i = threadIdx.x * 8; i < vocab; i += kLossFwdThreads * 8) {
      const uint4 w = w_next;
      if (i + kLossFwdThreads * 8 < vocab) w_next = ld_nc_v4(p + i + kLossFwdThreads * 8);
      const uint32_t xi[4] = {w.x, w.y, w.z, w.w};
      float2 z[4];
      uint4 to;
      uint32_t* tp = &to.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // bf16(x / c) for both halves: q0 = x r, q = fma(-fma(q0, c, -x), r, q0) with the negations folded into
        // the operands (nx = -x, nr = -r), the correctly rounded quotient since r is the correctly rounded reciprocal
        const float2 nx = bf16x2_unpack_neg(xi[j]);
        const float2 q0 = __fmul2_rn(nx, nr2);
        const float2 q = __ffma2_rn(__ffma2_rn(q0, c2, nx), nr2, q0);
        const uint32_t a2 = pack_bf16x2(q.x, q.y);
        // bf16(tanh(.)) of both: table by magnitude, signs put back
        const uint32_t t_lo = s_tanh[a2 & 0x7fffu], t_hi = s_tanh[(a2 >> 16) & 0x7fffu];
        const uint32_t t2 = __byte_perm(t_lo, t_hi, 0x5410) | (a2 & 0x80008000u);
        tp[j] = t2;
        // z = bf16(c tanh)
        const float2 zf = __fmul2_rn(c2, bf16x2_unpack(t2));
        z[j] = bf16x2_unpack(pack_bf16x2(zf.x, zf.y));
      }
      const int valid = vocab - i;        // < 8 only in the last piece of a vocabulary that is not a multiple of 8
      if (valid < 8) {
        // the piece was read whole (the row pitch is a multiple of 8 elements); columns past the
        // vocabulary take no part in the softmax and are not written
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (2 * j >= valid) z[j].x = -INFINITY;
          if (2 * j + 1 >= valid) z[j].y = -INFINITY;
        }
        if (tanh_out != nullptr) {
          const __nv_bfloat16* tv = reinterpret_cast<const __nv_bfloat16*>(&to);
          for (int j = 0; j < valid; ++j) tanh_out[row * ld_t + i + j] = tv[j];
        }
      } else if (tanh_out != nullptr) {
        *reinterpret_cast<uint4*>(tanh_out + row * ld_t + i) = to;
      }
      const float mx = fmaxf(fmaxf(fmaxf(z[0].x, z[0].y), fmaxf(z[1].x, z[1].y)), fmaxf(fmaxf(z[2].x, z[2].y), fmaxf(z[3].x, z[3].y)));
      const float mn = fmaxf(m, mx);
      const float2 nmn = make_float2(-mn, -mn);
      float2 acc = make_float2(s * __expf(m - mn), 0.f);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 d = __fmul2_rn(__fadd2_rn(z[j], nmn), l2e);     // (z - max) log2 e: the difference is exact
        float2 e;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(d.x));
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(d.y));
        acc = __fadd2_rn(acc, e);
      }
      s = acc.x + acc.y;
      m = mn;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lse_merge(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();                       // the previous row's partials have been read
    if (lane == 0) { s_m[warp] = m; s_s[warp] = s; }
    __syncthreads();
    if (threadIdx.x == 0) {
      m = s_m[0]; s = s_s[0];
#pragma unroll
      for (int wi = 1; wi < kLossFwdThreads / 32; ++wi) lse_merge(m, s, s_m[wi], s_s[wi]);
      const float lse = m + logf(s);
      int t = targets[row];
      t = t < 0 ? 0 : (t >= vocab ? vocab - 1 : t);   // out-of-range targets clamp, as jnp.take_along_axis does
      const float zt = sc.z_of_tanh(tanh_bf16(sc.quotient(__bfloat162float(p[t]))));
      lse_out[row] = lse;
      nll_out[row] = lse - zt;
    }
  }
}

// dlogits = gscale / rows * (exp(z - lse) - [col == target]) * (1 - tanh^2), rounded to bf16.
// `d` may be the buffer `tanh_in` lives in: every element is read and then written by one thread.
__global__ void __launch_bounds__(kLossThreads)
softcap_ce_bwd_kernel(const __nv_bfloat16* tanh_in, const int32_t* __restrict__ targets,
                      const float* __restrict__ lse, const float* __restrict__ gscale, float cap, float inv_rows,
                      __nv_bfloat16* d, int vocab, int64_t ld_t, int64_t ld_d) {
  const int64_t row = blockIdx.x;
  const Softcap sc(cap);
  const float l = lse[row];
  const float g = (gscale != nullptr ? *gscale : 1.0f) * inv_rows;
  int t = targets[row];
  t = t < 0 ? 0 : (t >= vocab ? vocab - 1 : t);
  const __nv_bfloat16* p = tanh_in + row * ld_t;
  for (int i = threadIdx.x * 8; i < vocab; i += kLossThreads * 8) {
    const uint4 w = *reinterpret_cast<const uint4*>(p + i);
    const uint32_t ti[4] = {w.x, w.y, w.z, w.w};
    uint4 o;
    uint32_t* op = &o.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float t0 = bf16lo(ti[j]), t1 = bf16hi(ti[j]);
      float p0 = __expf(sc.z_of_tanh(t0) - l), p1 = __expf(sc.z_of_tanh(t1) - l);
      if (i + 2 * j == t) p0 -= 1.0f;
      if (i + 2 * j + 1 == t) p1 -= 1.0f;
      op[j] = pack_bf16x2(p0 * g * __fmaf_rn(-t0, t0, 1.0f), p1 * g * __fmaf_rn(-t1, t1, 1.0f));
    }
    const int valid = vocab - i;
    if (valid < 8) {                     // ragged last piece: nothing is stored past the vocabulary
      const __nv_bfloat16* ov = reinterpret_cast<const __nv_bfloat16*>(&o);
      for (int j = 0; j < valid; ++j) d[row * ld_d + i + j] = ov[j];
    } else {
      *reinterpret_cast<uint4*>(d + row * ld_d + i) = o;
    }
  }
}

}  // namespace tg

using namespace tg;

extern "C" int tg_softcap_ce_fwd(const void* logits, const int32_t* targets, float cap, void* tanh_out, float* lse,
                                 float* nll, int64_t rows, int64_t vocab, int64_t ld, int64_t ld_tanh, void* stream) {
  if (rows < 0 || vocab <= 0 || ld % 8 != 0 || ld < vocab || vocab > INT32_MAX) return TG_ERR_SHAPE;
  if (tanh_out != nullptr && (ld_tanh % 8 != 0 || ld_tanh < vocab)) return TG_ERR_SHAPE;
  if (!(cap > 0.0f)) return TG_ERR_SHAPE;
  if (rows > INT32_MAX) return TG_ERR_TOO_LARGE;
  if (rows == 0) return TG_OK;
  if (!aligned16(logits) || !aligned16(tanh_out)) return TG_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  // persistent blocks, as many as fit (the 64 KB table allows three per SM)
  static int per_sm_of[64] = {0};          // per device: the attribute below is a per-device setting
  int dev = 0;
  TG_CUDA_CHECK(cudaGetDevice(&dev));
  int& per_sm = per_sm_of[dev & 63];
  if (per_sm == 0) {
    TG_CUDA_CHECK(cudaFuncSetAttribute(softcap_ce_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTanhBytes));
    int n = 0;
    TG_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, softcap_ce_fwd_kernel, kLossFwdThreads, kTanhBytes));
    per_sm = n > 0 ? n : 1;
  }
  const int64_t blocks = std::min<int64_t>(rows, int64_t(sm_count()) * per_sm);
  softcap_ce_fwd_kernel<<<int(blocks), kLossFwdThreads, kTanhBytes, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), targets, cap, static_cast<__nv_bfloat16*>(tanh_out), lse, nll,
      int(rows), int(vocab), ld, ld_tanh);
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}

extern "C" int tg_softcap_ce_bwd(const void* tanh_in, const int32_t* targets, const float* lse, const float* gscale,
                                 float cap, void* dlogits, int64_t rows, int64_t vocab, int64_t ld_tanh, int64_t ld_d,
                                 void* stream) {
  if (rows < 0 || vocab <= 0 || ld_tanh % 8 != 0 || ld_d % 8 != 0 || ld_tanh < vocab || ld_d < vocab ||
      vocab > INT32_MAX)
    return TG_ERR_SHAPE;
  if (!(cap > 0.0f)) return TG_ERR_SHAPE;
  if (rows > INT32_MAX) return TG_ERR_TOO_LARGE;
  if (rows == 0) return TG_OK;
  if (!aligned16(tanh_in) || !aligned16(dlogits)) return TG_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  softcap_ce_bwd_kernel<<<int(rows), kLossThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(tanh_in), targets, lse, gscale, cap, 1.0f / float(rows),
      static_cast<__nv_bfloat16*>(dlogits), int(vocab), ld_tanh, ld_d);
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}
