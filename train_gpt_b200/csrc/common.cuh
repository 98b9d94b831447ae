// Shared device/host helpers for the train_gpt_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/train_gpt_b200.h"

namespace tg {

constexpr float kE4M3Max = 448.0f;   // train-gpt fp8.py:26
constexpr float kScaleFloor = 1e-30f;  // train-gpt fp8.py:44
constexpr int kTile = 128;           // train-gpt fp8.py:27

// Records a failing CUDA call for tg_last_cuda_error() and returns TG_ERR_CUDA.
int record_cuda_error(cudaError_t e, const char* where);
// TG_OK if the current device is compute capability 10.x, else TG_ERR_ARCH.
int check_arch();
int sm_count();
// SMs a persistent GEMM grid may occupy: sm_count() minus what tg_set_gemm_reserved_sms left for others.
int gemm_sms();

#define TG_CUDA_CHECK(expr)                                        \
  do {                                                             \
    cudaError_t _e = (expr);                                       \
    if (_e != cudaSuccess) return tg::record_cuda_error(_e, #expr); \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#ifdef __CUDACC__

// max that returns NaN if either input is NaN (jnp.max / jnp.maximum semantics).
__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// two bf16 packed in a 32-bit word -> two floats (exact)
// (the low half moves up by a multiply by 2^16, which the assembler is free to issue as a shift on
// the ALU pipe or as an integer multiply on the FMA pipe; forcing the multiply, with the factor taken
// from constant memory, gained 2.5 % in the row+column quantiser and lost 4-10 % in the row-wise and
// fused-norm ones, whose FMA pipe is the busier)
__device__ __forceinline__ float bf16lo(uint32_t w) {
  uint32_t r;
  asm("mul.lo.u32 %0, %1, 65536;" : "=r"(r) : "r"(w));
  return __uint_as_float(r);
}
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// round two floats to bf16 (RNE) and pack (lo in bits 0..15)
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// scale of a tile from its amax: max(amax / 448, 1e-30) with NaN propagation
__device__ __forceinline__ float scale_from_amax(float amax) {
  return max_nan(__fdiv_rn(amax, kE4M3Max), kScaleFloor);
}

// RNE_e4m3(lo), RNE_e4m3(hi) packed into 16 bits (lo in bits 0..7).  Inputs never exceed
// 448*(1+2^-23) in magnitude here, so saturation never changes a finite result.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

// ---- x / scale, correctly rounded, without a per-element IEEE division -------------------
// The quantised byte is RNE_e4m3(RN_f32(x / s)).  A per-element div.rn.f32 costs ~10
// instructions plus a MUFU.RCP, which makes the streaming quantisers compute-bound.  The
// tile shares one scale, so the reciprocal r = RN(1/s) is taken once and each element gets
//     q0 = x * r;  q = fma(-fma(q0, s, -x), r, q0)
// (one Markstein correction step).  The input domain is tiny -- x is a bf16 value and s is
// max(amax/448, 1e-30) for a bf16 amax >= |x| -- so equality of the resulting BYTE with the
// IEEE-division path is verified exhaustively over the whole domain by
// tg_selftest_quantise_division (2^31 pairs), not argued.  Non-finite scales (NaN or Inf in
// the tile) take the IEEE division so that they propagate exactly as jnp does.
struct QuantDiv {
  float s, r;
  bool finite;
  __device__ __forceinline__ explicit QuantDiv(float scale) {
    s = scale;
    r = __frcp_rn(scale);
    finite = fabsf(scale) <= 3.402823466e38f;
  }
  template <int SCHEME = 2>
  __device__ __forceinline__ float div(float x) const {
    if (SCHEME == 0) return __fdiv_rn(x, s);
    float q = __fmul_rn(x, r);
    // residual taken as q*s - x and subtracted, so that x = -0 stays -0 (fma(+0, s, -0) is +0)
    if (SCHEME >= 2) q = __fmaf_rn(-__fmaf_rn(q, s, -x), r, q);
    if (SCHEME >= 3) q = __fmaf_rn(-__fmaf_rn(q, s, -x), r, q);
    return q;
  }
};

// The same step on two values at once with the packed single-precision instructions of
// sm_100 (mul.f32x2 / fma.rn.f32x2: one issue slot for two lanes of arithmetic).  Negations
// are folded into the operands so that no instruction needs a modifier: with nx = -x and
// nr = -r,
//     q0 = nx * nr          == x * r            (sign of a product is the xor of the signs)
//     e  = fma(q0, s, nx)   == fma(q0, s, -x)
//     q  = fma(e, nr, q0)   == fma(-e, r, q0)
// bit for bit, signed zeros included.
__device__ __forceinline__ float2 bf16x2_unpack(uint32_t w) { return make_float2(bf16lo(w), bf16hi(w)); }
__device__ __forceinline__ float2 bf16x2_unpack_neg(uint32_t w) {
  uint32_t lo;
  asm("mad.lo.u32 %0, %1, 65536, 0x80000000;" : "=r"(lo) : "r"(w));   // (w << 16) ^ sign bit in one instruction
  return make_float2(__uint_as_float(lo), __uint_as_float((w & 0xffff0000u) ^ 0x80000000u));
}
// two bf16 values (one word) -> their quotients by the finite scales s2, nr2 = -RN(1/s2)
__device__ __forceinline__ float2 quotient2_sr(uint32_t w, float2 s2, float2 nr2) {
  const float2 nx = bf16x2_unpack_neg(w);
  const float2 q0 = __fmul2_rn(nx, nr2);
  const float2 e = __ffma2_rn(q0, s2, nx);
  return __ffma2_rn(e, nr2, q0);
}
// two bf16 values (one word) -> two e4m3 bytes (low 16 bits)
__device__ __forceinline__ uint32_t quantize2_sr(uint32_t w, float2 s2, float2 nr2) {
  const float2 q = quotient2_sr(w, s2, nr2);
  return cvt_e4m3x2(q.x, q.y);
}
// four floats -> four e4m3 bytes in memory order.  The two 16-bit conversion results are joined inside one
// asm block: handed out as separate 16-bit values they are each widened (a mask) and then permuted together.
__device__ __forceinline__ uint32_t cvt_e4m3x4(float2 a, float2 b) {
  uint32_t r;
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}"
      : "=r"(r) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return r;
}

// Quantise 8 values with a FINITE scale s and its reciprocal r = RN(1/s) that the caller
// already has.  w holds the values as loaded from memory (element 0 in the low half of w.x);
// the 8 e4m3 bytes come back in memory order.
__device__ __forceinline__ uint2 quantize8_sr(const uint4& w, float s, float r) {
  const float2 s2 = make_float2(s, s), nr2 = make_float2(-r, -r);
  return make_uint2(cvt_e4m3x4(quotient2_sr(w.x, s2, nr2), quotient2_sr(w.y, s2, nr2)),
                    cvt_e4m3x4(quotient2_sr(w.z, s2, nr2), quotient2_sr(w.w, s2, nr2)));
}

// Quantise 8 values with `scale` (any value: a NaN or Inf scale takes the IEEE division).
__device__ __forceinline__ uint2 quantize8(const uint4& w, float scale) {
  if (fabsf(scale) <= 3.402823466e38f) return quantize8_sr(w, scale, __frcp_rn(scale));
  const uint32_t b0 = cvt_e4m3x2(__fdiv_rn(bf16lo(w.x), scale), __fdiv_rn(bf16hi(w.x), scale));
  const uint32_t b1 = cvt_e4m3x2(__fdiv_rn(bf16lo(w.y), scale), __fdiv_rn(bf16hi(w.y), scale));
  const uint32_t b2 = cvt_e4m3x2(__fdiv_rn(bf16lo(w.z), scale), __fdiv_rn(bf16hi(w.z), scale));
  const uint32_t b3 = cvt_e4m3x2(__fdiv_rn(bf16lo(w.w), scale), __fdiv_rn(bf16hi(w.w), scale));
  return make_uint2(b0 | (b1 << 16), b2 | (b3 << 16));
}

// The scale arithmetic (an IEEE division by 448, a max, a correctly rounded reciprocal: ~20
// instructions) is the same for all 16 lanes that share a tile.  When a warp has N tiles'
// amax values in registers (N <= 16, a power of two, every lane of a half-warp holding the N
// values of that half), lane j of each half computes tile j % N only and the results travel
// back by shuffle: N x 20 instructions become 20 + 2 N.  `fin` is false if any scale of the
// warp is not finite (the caller then takes the IEEE-division path).
template <int N>
__device__ __forceinline__ void tile_scales(const float (&amax)[N], float (&s)[N], float (&r)[N], float& s_mine, bool& fin) {
  const int lane = threadIdx.x & 31, j = lane & (N - 1);
  float msel = amax[0];
#pragma unroll
  for (int u = 1; u < N; ++u) msel = (j == u) ? amax[u] : msel;
  s_mine = scale_from_amax(msel);
  const float r_mine = __frcp_rn(s_mine);
  fin = __all_sync(0xffffffffu, fabsf(s_mine) <= 3.402823466e38f);
#pragma unroll
  for (int u = 0; u < N; ++u) {
    s[u] = __shfl_sync(0xffffffffu, s_mine, (lane & 16) | u);
    r[u] = __shfl_sync(0xffffffffu, r_mine, (lane & 16) | u);
  }
}

// |.|-max of bf16 values WITHOUT unpacking them: with the sign bit cleared, bf16 bit patterns
// order like unsigned integers (0 < subnormals < normals < Inf 0x7F80 < NaN 0x7F81..), so a
// per-halfword unsigned max of two packed words is the max of magnitudes, and a NaN wins as
// jnp.max wants.  One LOP3 + one VIMNMX.U16x2 per two values.
constexpr uint32_t kAbsMask2 = 0x7fff7fffu;
__device__ __forceinline__ uint32_t absmax2(uint32_t m, uint32_t w) { return __vmaxu2(m, w & kAbsMask2); }
// Magnitude maximum of eight packed words through the packed bf16 max (NaN-propagating): seven instructions
// on the FMA pipe, which the quantisers leave half idle, instead of eight masks and eight integer maxima on
// the ALU pipe, which bounds them.  |.| is taken on the leaves only.  A NaN comes back as the canonical
// 0x7FFF, still the largest pattern under the unsigned order above.
__device__ __forceinline__ uint32_t absmax2_tree8(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t e, uint32_t f,
                                                  uint32_t g, uint32_t h) {
  uint32_t r;
  asm("{\n\t.reg .b32 t<8>;\n\t"
      "abs.bf16x2 t0, %1;\n\tabs.bf16x2 t1, %2;\n\tabs.bf16x2 t2, %3;\n\tabs.bf16x2 t3, %4;\n\t"
      "abs.bf16x2 t4, %5;\n\tabs.bf16x2 t5, %6;\n\tabs.bf16x2 t6, %7;\n\tabs.bf16x2 t7, %8;\n\t"
      "max.NaN.bf16x2 t0, t0, t1;\n\tmax.NaN.bf16x2 t2, t2, t3;\n\tmax.NaN.bf16x2 t4, t4, t5;\n\tmax.NaN.bf16x2 t6, t6, t7;\n\t"
      "max.NaN.bf16x2 t0, t0, t2;\n\tmax.NaN.bf16x2 t4, t4, t6;\n\tmax.NaN.bf16x2 %0, t0, t4;\n\t}"
      : "=r"(r) : "r"(a), "r"(b), "r"(c), "r"(d), "r"(e), "r"(f), "r"(g), "r"(h));
  return r;
}
__device__ __forceinline__ uint32_t absmax8(const uint4& w, uint32_t m = 0u) {
  return absmax2(absmax2(absmax2(absmax2(m, w.x), w.y), w.z), w.w);
}
// the same through the packed bf16 max (NaN-propagating; |.| folds into the instruction):
// measured ~2 % faster in the fused norm kernel, where the ALU pipe is the busiest
__device__ __forceinline__ uint32_t absmax8_h(const uint4& w) {
  __nv_bfloat162 a = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w.x));
  a = __hmax2_nan(a, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w.y)));
  a = __hmax2_nan(a, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w.z)));
  a = __hmax2_nan(a, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w.w)));
  return *reinterpret_cast<uint32_t*>(&a);
}
// both halfwords -> the float value of the larger
__device__ __forceinline__ float absmax_to_float(uint32_t m) {
  const uint32_t lo = m & 0xffffu, hi = m >> 16;
  return __uint_as_float((lo > hi ? lo : hi) << 16);
}

// Half-warp reduction of N per-lane tile maxima at once (N = 1, 2, 4 or 8 chunks; every lane
// of a half-warp holds, for each chunk, the packed halfword maxima absmax8 returned).  A plain
// butterfly would cost 4 shuffles + 4 max per chunk.  Here the two halfwords of a chunk are
// merged, chunks c and c + N/2 share one word, and each exchange step HALVES what a lane still
// carries (a lane keeps the words / the halfword its own lane bit selects and hands the rest to
// its partner), so N chunks cost about N/2 + 3 shuffles in all.  On return lane l holds, as a
// float, the magnitude maximum of chunk (l & (N-1)) over its half-warp -- the layout
// tile_scales wants.
template <int N>
__device__ __forceinline__ float exchange_tile_amax(const uint32_t (&m)[N]) {
  const int lane = threadIdx.x & 31;
  uint32_t v;
  if constexpr (N == 1) {
    v = __vmaxu2(m[0], m[0] >> 16) & 0xffffu;
  } else {
    uint32_t w[N / 2];
#pragma unroll
    for (int i = 0; i < N / 2; ++i)   // halfwords: (chunk i, chunk i + N/2)
      w[i] = __vmaxu2(__byte_perm(m[i], m[i + N / 2], 0x5410), __byte_perm(m[i], m[i + N / 2], 0x7632));
#pragma unroll
    for (int b = 0; (2 << b) <= N / 2; ++b) {
      const bool up = (lane >> b) & 1;
#pragma unroll
      for (int k = 0; k < (N / 2) >> (b + 1); ++k) {
        const uint32_t keep = up ? w[2 * k + 1] : w[2 * k];
        const uint32_t give = up ? w[2 * k] : w[2 * k + 1];
        w[k] = __vmaxu2(keep, __shfl_xor_sync(0xffffffffu, give, 1 << b));
      }
    }
    const uint32_t other = __shfl_xor_sync(0xffffffffu, w[0], N / 2);
    const bool up = lane & (N / 2);
    const uint32_t mine = up ? (w[0] >> 16) : (w[0] & 0xffffu);
    const uint32_t theirs = up ? (other >> 16) : (other & 0xffffu);
    v = mine > theirs ? mine : theirs;
  }
#pragma unroll
  for (int o = N; o <= 8; o <<= 1) {
    const uint32_t t = __shfl_xor_sync(0xffffffffu, v, o);
    v = v > t ? v : t;
  }
  return __uint_as_float(v << 16);
}

// tile_scales for a lane that already holds its own tile's amax (see exchange_tile_amax):
// lane j of each half computes tile j % N; s[u], r[u] come back by shuffle.
template <int N>
__device__ __forceinline__ void tile_scales_own(float amax_mine, float (&s)[N], float (&r)[N], float& s_mine, bool& fin) {
  const int lane = threadIdx.x & 31;
  s_mine = scale_from_amax(amax_mine);
  const float r_mine = __frcp_rn(s_mine);
  fin = __all_sync(0xffffffffu, fabsf(s_mine) <= 3.402823466e38f);
#pragma unroll
  for (int u = 0; u < N; ++u) {
    s[u] = __shfl_sync(0xffffffffu, s_mine, (lane & 16) | u);
    r[u] = __shfl_sync(0xffffffffu, r_mine, (lane & 16) | u);
  }
}

// |.|-max over the 8 bf16 values of w in float (NaN-propagating); measured faster than the
// packed integer form where the values are unpacked to float anyway (row-wise kernels)
__device__ __forceinline__ float amax8(const uint4& w, float m = 0.f) {
  m = max_nan(m, fabsf(bf16lo(w.x)));
  m = max_nan(m, fabsf(bf16hi(w.x)));
  m = max_nan(m, fabsf(bf16lo(w.y)));
  m = max_nan(m, fabsf(bf16hi(w.y)));
  m = max_nan(m, fabsf(bf16lo(w.z)));
  m = max_nan(m, fabsf(bf16hi(w.z)));
  m = max_nan(m, fabsf(bf16lo(w.w)));
  m = max_nan(m, fabsf(bf16hi(w.w)));
  return m;
}

__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

#endif  // __CUDACC__

}  // namespace tg
