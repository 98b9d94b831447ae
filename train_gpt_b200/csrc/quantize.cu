// e4m3 quantisers with float32 amax/448 scales (train-gpt fp8.py:39-47), three tile
// shapes.  All are HBM-bound streaming kernels: 2 bytes in, 1 byte + 4/128 byte out per
// element, every input byte read once with 128-bit loads and kept in registers between
// the amax pass and the divide pass.
#include "common.cuh"

namespace tg {

// ---------------------------------------------------------------------------------------
// 1 x 128 tiles.  cols % 128 == 0, so tile t is the 256 contiguous bytes at x + 256 t and
// its scale is scales[t].  Sixteen lanes own a tile (16 B = 8 values each); each thread
// keeps kUnroll independent tiles in flight.
// ---------------------------------------------------------------------------------------
constexpr int kRowUnroll = 4;
constexpr int kRowThreads = 256;

__global__ void __launch_bounds__(kRowThreads)
quantize_rowwise_kernel(const uint4* __restrict__ x, uint2* __restrict__ q,
                        float* __restrict__ scales, int64_t n_tiles) {
  const int lane16 = threadIdx.x & 15;
  const int64_t group = (int64_t(blockIdx.x) * kRowThreads + threadIdx.x) >> 4;  // half-warp id
  const int64_t n_groups = (int64_t(gridDim.x) * kRowThreads) >> 4;
  for (int64_t t0 = group * kRowUnroll; t0 < n_tiles; t0 += n_groups * kRowUnroll) {
    uint4 w[kRowUnroll];
#pragma unroll
    for (int u = 0; u < kRowUnroll; ++u) {
      const int64_t t = t0 + u;
      w[u] = (t < n_tiles) ? ld_nc_v4(x + t * 16 + lane16) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kRowUnroll; ++u) {
      float m = amax8(w[u]);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, o));
      const float s = scale_from_amax(m);
      const int64_t t = t0 + u;
      if (t < n_tiles) {
        q[t * 16 + lane16] = quantize8(w[u], s);
        if (lane16 == 0) scales[t] = s;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// 128 x 1 tiles (a scale per column per block of 128 rows).  A thread block owns a
// 128-row x 128-column panel: a half-warp spans the 128 columns (16 lanes x 8 columns), so
// each of the 16 half-warps owns every 16th row (8 rows per thread, kept in registers).
// Column maxima are combined across the warps through shared memory (one thread per column
// finishes the reduction and the reciprocal), then the same registers are divided and stored.
// 64 registers: four blocks per SM, so one block's loads overlap the others' arithmetic.
// ---------------------------------------------------------------------------------------
constexpr int kColPanelCols = 128;
constexpr int kColThreads = 256;
constexpr int kColHalfWarps = kColThreads / 16;           // 16
constexpr int kColRowsPerThread = kTile / kColHalfWarps;  // 8

// Activation folded into the load (ACT != TG_ACT_NONE): the tile that is quantised is
//   relu2      bf16( max(x,0)^2 )                         model.py:72, `jax.nn.relu(h) ** 2`
//   gelu       bf16( x/2 (1 + erf(x/sqrt 2)) )            the activation the benchmark's training configuration names
//   relu2_bwd  bf16( gate * 2 max(x,0) )                  the cotangent of relu2 for upstream gradient `gate`
//   gelu_bwd   bf16( gate * (Phi(x) + x phi(x)) )
// each computed in float32 from the bf16 input(s) and rounded to bf16 ONCE, which is what the
// unfused composition (an elementwise bf16 kernel, then the quantiser) would have handed over.
// The MLP's activation and its gradient are then never written to memory.
// erf(x / sqrt 2) as sign(x) (1 - 2^P(|x|)): P is the degree-9 polynomial (no constant term) fitted to
// log2 erfc(a / sqrt 2) on a in [0, 6.08] with weight erfc, so that the ABSOLUTE error of erfc is 2e-9
// everywhere -- which is what the float32 forms below can see: they add the result to 1.  One
// special-function instruction and ten multiply-adds, against libdevice erff's two branches of that
// size.  Rounded to bf16, x/2 (1 + erf) from this routine and from a correctly rounded erff agree for
// every finite bf16 x in exact float32 arithmetic; the approximate ex2 flips a bf16 ulp on about one
// element in ten thousand.
__device__ __forceinline__ float erf_of_x_over_sqrt2(float x) {
  const float a = fminf(fabsf(x), 6.081118f);       // erfc is 1.2e-9 there: 1 - that is 1
  float p = 5.117859700476401e-07f;
  p = fmaf(p, a, -9.538196536595933e-06f);
  p = fmaf(p, a, 7.480611384380609e-05f);
  p = fmaf(p, a, -0.0002837043721228838f);
  p = fmaf(p, a, 1.3612322618428152e-05f);
  p = fmaf(p, a, 0.006932816002517939f);
  p = fmaf(p, a, -0.05243593826889992f);
  p = fmaf(p, a, -0.4592210352420807f);
  p = fmaf(p, a, -1.1511043310165405f);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(p * a));
  return copysignf(1.0f - e, x);
}

template <int ACT>
__device__ __forceinline__ float act_value(float x, float gate) {
  if (ACT == TG_ACT_RELU2) { const float r = fmaxf(x, 0.f); return r * r; }
  if (ACT == TG_ACT_RELU2_BWD) return gate * (2.f * fmaxf(x, 0.f));
  if (ACT == TG_ACT_GELU) return x * 0.5f * (1.f + erf_of_x_over_sqrt2(x));
  if (ACT == TG_ACT_GELU_BWD) {
    const float cdf = 0.5f * (1.f + erf_of_x_over_sqrt2(x));
    const float pdf = expf(-0.5f * x * x) * 0.39894228040143267794f;
    return gate * (cdf + x * pdf);
  }
  return x;
}
// The same erf for two arguments at once in packed f32x2 instructions (the kernel is bound by instruction
// issue, and the polynomial is most of the activation's instructions); same operations in the same order
// as the scalar routine, so the same bits.  (Forward form 0.201 -> 0.184 ms at 32768 x 4096; backward form, with the density as a
// packed product and two ex2 instead of two expf, 0.268 -> 0.234 ms.)
__device__ __forceinline__ float2 erf_of_x_over_sqrt2_pair(float2 x) {
  const float2 a = make_float2(fminf(fabsf(x.x), 6.081118f), fminf(fabsf(x.y), 6.081118f));
  auto c2 = [](float c) { return make_float2(c, c); };
  float2 p = c2(5.117859700476401e-07f);
  p = __ffma2_rn(p, a, c2(-9.538196536595933e-06f));
  p = __ffma2_rn(p, a, c2(7.480611384380609e-05f));
  p = __ffma2_rn(p, a, c2(-0.0002837043721228838f));
  p = __ffma2_rn(p, a, c2(1.3612322618428152e-05f));
  p = __ffma2_rn(p, a, c2(0.006932816002517939f));
  p = __ffma2_rn(p, a, c2(-0.05243593826889992f));
  p = __ffma2_rn(p, a, c2(-0.4592210352420807f));
  p = __ffma2_rn(p, a, c2(-1.1511043310165405f));
  const float2 t = __fmul2_rn(p, a);
  float2 e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(t.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(t.y));
  const float2 r = __ffma2_rn(e, c2(-1.0f), c2(1.0f));       // 1 - e, exact product
  return make_float2(copysignf(r.x, x.x), copysignf(r.y, x.y));
}

template <int ACT>
__device__ __forceinline__ uint32_t act_pair(uint32_t x2, uint32_t g2) {
  if constexpr (ACT == TG_ACT_GELU) {
    const float2 x = bf16x2_unpack(x2);
    const float2 one_plus = __fadd2_rn(make_float2(1.f, 1.f), erf_of_x_over_sqrt2_pair(x));
    const float2 y = __fmul2_rn(__fmul2_rn(x, make_float2(0.5f, 0.5f)), one_plus);
    return pack_bf16x2(y.x, y.y);
  } else if constexpr (ACT == TG_ACT_GELU_BWD) {
    const float2 x = bf16x2_unpack(x2), gate = bf16x2_unpack(g2);
    const float2 cdf = __fmul2_rn(make_float2(0.5f, 0.5f), __fadd2_rn(make_float2(1.f, 1.f), erf_of_x_over_sqrt2_pair(x)));
    // the density: 2^(-x^2 log2(e) / 2) / sqrt(2 pi); x^2 is exact (a bf16 squared), the product is rounded once
    const float2 t = __fmul2_rn(__fmul2_rn(x, x), make_float2(-0.72134752044448170f, -0.72134752044448170f));
    float2 pdf;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(pdf.x) : "f"(t.x));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(pdf.y) : "f"(t.y));
    pdf = __fmul2_rn(pdf, make_float2(0.39894228040143267794f, 0.39894228040143267794f));
    const float2 y = __fmul2_rn(gate, __ffma2_rn(x, pdf, cdf));
    return pack_bf16x2(y.x, y.y);
  } else {
    return pack_bf16x2(act_value<ACT>(bf16lo(x2), bf16lo(g2)), act_value<ACT>(bf16hi(x2), bf16hi(g2)));
  }
}
template <int ACT>
__device__ __forceinline__ uint4 act_apply(uint4 x, uint4 g) {
  return make_uint4(act_pair<ACT>(x.x, g.x), act_pair<ACT>(x.y, g.y), act_pair<ACT>(x.z, g.z), act_pair<ACT>(x.w, g.w));
}

// FULL: the panel lies wholly inside the tensor (all 128 rows, all 128 columns), the case of every block of
// a launch whose sizes are multiples of 128: no bounds predicate is evaluated and row addresses are
// one 64-bit add apart.  (The kernel is bound by instruction issue; the per-opcode counters showed the
// address arithmetic and the bounds branches of the general form to be a third of its instructions.)
template <bool WITH_ROWS, int ACT, bool FULL>
__device__ __forceinline__ void colwise_panel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                              float* __restrict__ scales, uint8_t* __restrict__ q_row,
                                              float* __restrict__ s_row, int64_t rows, int64_t cols,
                                              const __nv_bfloat16* __restrict__ gate, int64_t q_row_ld, int64_t s_row_ld,
                                              int64_t q_col_ld, int64_t s_col_ld, float (*s_max)[kColPanelCols],
                                              float* s_scale, float* s_rcp) {
  const int cx = threadIdx.x & 15, hw = threadIdx.x >> 4;
  const int64_t col0 = int64_t(blockIdx.x) * kColPanelCols + cx * 8;
  const int64_t row_blk = blockIdx.y;
  const int64_t row0 = row_blk * kTile + hw;  // this thread's rows: row0 + 16 r
  const bool col_ok = FULL || col0 < cols;    // cols % 8 == 0

  uint4 w[kColRowsPerThread];
  {
    const __nv_bfloat16* xp = x + row0 * cols + col0;
    const __nv_bfloat16* gp = gate + row0 * cols + col0;     // only dereferenced by the *_BWD variants
    const int64_t step = int64_t(kColHalfWarps) * cols;
#pragma unroll
    for (int r = 0; r < kColRowsPerThread; ++r, xp += step, gp += step) {
      const bool ok = FULL || (col_ok && row0 + r * kColHalfWarps < rows);
      w[r] = ok ? ld_nc_v4(xp) : make_uint4(0, 0, 0, 0);
      if constexpr (ACT != TG_ACT_NONE) {
        uint4 g = make_uint4(0, 0, 0, 0);
        if constexpr (ACT == TG_ACT_RELU2_BWD || ACT == TG_ACT_GELU_BWD)
          if (ok) g = ld_nc_v4(gp);
        w[r] = act_apply<ACT>(w[r], g);   // rows past the end stay zero: every variant maps (0, 0) to 0
      }
    }
  }
  if constexpr (WITH_ROWS) {   // cols % 128 == 0 here: every lane holds real columns
    // the 8 row tiles of a half-warp: one exchange leaves lane j with the amax of row j % 8
    uint32_t mr[kColRowsPerThread];
#pragma unroll
    for (int r = 0; r < kColRowsPerThread; ++r) mr[r] = absmax8_h(w[r]);
    float sr[kColRowsPerThread], rr[kColRowsPerThread], s_mine;
    bool fin;
    tile_scales_own<kColRowsPerThread>(exchange_tile_amax<kColRowsPerThread>(mr), sr, rr, s_mine, fin);
    {
      const int64_t row = row0 + int64_t(cx & 7) * kColHalfWarps;   // lane j of the half computed row r = j % 8
      if (cx < kColRowsPerThread && (FULL || row < rows)) s_row[row * s_row_ld + blockIdx.x] = s_mine;
    }
    uint8_t* qp = q_row + row0 * q_row_ld + col0;
    const int64_t step = int64_t(kColHalfWarps) * q_row_ld;
    // one branch around the whole loop, not one per row: a NaN or Inf anywhere in the warp's tiles is the rare case
    if (fin) {
#pragma unroll
      for (int r = 0; r < kColRowsPerThread; ++r, qp += step)
        if (FULL || row0 + r * kColHalfWarps < rows) *reinterpret_cast<uint2*>(qp) = quantize8_sr(w[r], sr[r], rr[r]);
    } else {
#pragma unroll
      for (int r = 0; r < kColRowsPerThread; ++r, qp += step)
        if (FULL || row0 + r * kColHalfWarps < rows) *reinterpret_cast<uint2*>(qp) = quantize8(w[r], sr[r]);
    }
  }
  uint32_t m2[4];  // packed |.|-maxima of column pairs (0,1) (2,3) (4,5) (6,7) over this thread's rows
  static_assert(kColRowsPerThread == 8, "the tree below takes 8 rows");
  m2[0] = absmax2_tree8(w[0].x, w[1].x, w[2].x, w[3].x, w[4].x, w[5].x, w[6].x, w[7].x);
  m2[1] = absmax2_tree8(w[0].y, w[1].y, w[2].y, w[3].y, w[4].y, w[5].y, w[6].y, w[7].y);
  m2[2] = absmax2_tree8(w[0].z, w[1].z, w[2].z, w[3].z, w[4].z, w[5].z, w[6].z, w[7].z);
  m2[3] = absmax2_tree8(w[0].w, w[1].w, w[2].w, w[3].w, w[4].w, w[5].w, w[6].w, w[7].w);
  // the two half-warps of a warp hold the same columns: combine them in registers first
#pragma unroll
  for (int j = 0; j < 4; ++j) m2[j] = __vmaxu2(m2[j], __shfl_xor_sync(0xffffffffu, m2[j], 16));
  const int wp = threadIdx.x >> 5;
  if ((threadIdx.x & 16) == 0) {
    float4* dst = reinterpret_cast<float4*>(&s_max[wp][cx * 8]);
    dst[0] = make_float4(__uint_as_float(m2[0] << 16), __uint_as_float(m2[0] & 0xffff0000u),
                         __uint_as_float(m2[1] << 16), __uint_as_float(m2[1] & 0xffff0000u));
    dst[1] = make_float4(__uint_as_float(m2[2] << 16), __uint_as_float(m2[2] & 0xffff0000u),
                         __uint_as_float(m2[3] << 16), __uint_as_float(m2[3] & 0xffff0000u));
  }
  __syncthreads();
  // one thread per column finishes the maximum, derives scale and reciprocal once, and
  // publishes both (conflict-free: consecutive threads, consecutive words)
  if (threadIdx.x < kColPanelCols) {
    float v = s_max[0][threadIdx.x];
#pragma unroll
    for (int h = 1; h < kColThreads / 32; ++h) v = max_nan(v, s_max[h][threadIdx.x]);
    const float sc = scale_from_amax(v);
    s_scale[threadIdx.x] = sc;
    s_rcp[threadIdx.x] = __frcp_rn(sc);
    const int64_t col = int64_t(blockIdx.x) * kColPanelCols + threadIdx.x;
    if (FULL || col < cols) scales[row_blk * s_col_ld + col] = sc;
  }
  __syncthreads();
  if (!col_ok) return;
  float s[8], rc[8];
  {
    const float4 a0 = *reinterpret_cast<const float4*>(&s_scale[cx * 8]), a1 = *reinterpret_cast<const float4*>(&s_scale[cx * 8 + 4]);
    const float4 b0 = *reinterpret_cast<const float4*>(&s_rcp[cx * 8]), b1 = *reinterpret_cast<const float4*>(&s_rcp[cx * 8 + 4]);
    s[0] = a0.x; s[1] = a0.y; s[2] = a0.z; s[3] = a0.w; s[4] = a1.x; s[5] = a1.y; s[6] = a1.z; s[7] = a1.w;
    rc[0] = b0.x; rc[1] = b0.y; rc[2] = b0.z; rc[3] = b0.w; rc[4] = b1.x; rc[5] = b1.y; rc[6] = b1.z; rc[7] = b1.w;
  }
  bool all_finite = true;
#pragma unroll
  for (int j = 0; j < 8; ++j) all_finite = all_finite && (fabsf(s[j]) <= 3.402823466e38f);
  // this thread's four column pairs: scale and negated reciprocal as packed operands (see quantize2_sr)
  float2 s2[4], nr2[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    s2[j] = make_float2(s[2 * j], s[2 * j + 1]);
    nr2[j] = make_float2(-rc[2 * j], -rc[2 * j + 1]);
  }
  uint8_t* qp = q + row0 * q_col_ld + col0;
  const int64_t step = int64_t(kColHalfWarps) * q_col_ld;
  if (all_finite) {
#pragma unroll
    for (int r = 0; r < kColRowsPerThread; ++r, qp += step) {
      if (!FULL && row0 + r * kColHalfWarps >= rows) break;
      const uint4 v = w[r];
      *reinterpret_cast<uint2*>(qp) =
          make_uint2(cvt_e4m3x4(quotient2_sr(v.x, s2[0], nr2[0]), quotient2_sr(v.y, s2[1], nr2[1])),
                     cvt_e4m3x4(quotient2_sr(v.z, s2[2], nr2[2]), quotient2_sr(v.w, s2[3], nr2[3])));
    }
  } else {
#pragma unroll
    for (int r = 0; r < kColRowsPerThread; ++r, qp += step) {
      if (!FULL && row0 + r * kColHalfWarps >= rows) break;
      const uint4 v = w[r];
      const uint32_t b0 = cvt_e4m3x2(__fdiv_rn(bf16lo(v.x), s[0]), __fdiv_rn(bf16hi(v.x), s[1]));
      const uint32_t b1 = cvt_e4m3x2(__fdiv_rn(bf16lo(v.y), s[2]), __fdiv_rn(bf16hi(v.y), s[3]));
      const uint32_t b2 = cvt_e4m3x2(__fdiv_rn(bf16lo(v.z), s[4]), __fdiv_rn(bf16hi(v.z), s[5]));
      const uint32_t b3 = cvt_e4m3x2(__fdiv_rn(bf16lo(v.w), s[6]), __fdiv_rn(bf16hi(v.w), s[7]));
      *reinterpret_cast<uint2*>(qp) = make_uint2(__byte_perm(b0, b1, 0x5410), __byte_perm(b2, b3, 0x5410));
    }
  }
}

// WITH_ROWS: the same pass also emits the 1 x 128 (row-wise) quantisation of the panel -- a
// half-warp spans exactly one row tile -- so a tensor that needs both forms (an upstream
// gradient: row-wise for dgrad, column-wise for wgrad) is read from HBM once, not twice.
template <bool WITH_ROWS, int ACT = TG_ACT_NONE>
// Blocks per SM: the plain variants fit 64 registers without a spill and run four (8-14 % faster than three: the
// top stall is the wait for the panel's loads, and a fourth block is a third more of them in flight); the
// activation variants take 80 registers and three; the GELU cotangent variant, the one with the most live
// values, runs 2 % faster with 128 registers and two blocks than with 80 and three, spilling.
__global__ void __launch_bounds__(kColThreads, ACT == TG_ACT_GELU_BWD ? 2 : (ACT == TG_ACT_NONE ? 4 : 3))
quantize_colwise_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                        float* __restrict__ scales, uint8_t* __restrict__ q_row,
                        float* __restrict__ s_row, int64_t rows, int64_t cols,
                        const __nv_bfloat16* __restrict__ gate = nullptr, int64_t q_row_ld = 0, int64_t s_row_ld = 0,
                        int64_t q_col_ld = 0, int64_t s_col_ld = 0) {
  // row pitches of the outputs (0: dense): a caller may place either form inside a wider matrix, e.g. three
  // gradients side by side for one GEMM that contracts over all of them or produces all their weight gradients
  if (WITH_ROWS && q_row_ld == 0) { q_row_ld = cols; s_row_ld = cols / kTile; }
  if (q_col_ld == 0) { q_col_ld = cols; s_col_ld = cols; }
  __shared__ float s_max[kColThreads / 32][kColPanelCols];
  __shared__ __align__(16) float s_scale[kColPanelCols], s_rcp[kColPanelCols];
  const bool full = (int64_t(blockIdx.y) + 1) * kTile <= rows && (int64_t(blockIdx.x) + 1) * kColPanelCols <= cols;
  if (full)
    colwise_panel<WITH_ROWS, ACT, true>(x, q, scales, q_row, s_row, rows, cols, gate, q_row_ld, s_row_ld, q_col_ld, s_col_ld,
                                        s_max, s_scale, s_rcp);
  else
    colwise_panel<WITH_ROWS, ACT, false>(x, q, scales, q_row, s_row, rows, cols, gate, q_row_ld, s_row_ld, q_col_ld,
                                         s_col_ld, s_max, s_scale, s_rcp);
}

// ---------------------------------------------------------------------------------------
// 128 x 128 tiles, one scale each.  A thread block (256 threads) owns one tile: 16 lanes x
// 8 columns across, 16 row groups x 8 rows down.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
quantize_block128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                         float* __restrict__ scales, int64_t rows, int64_t cols) {
  __shared__ float s_max[8];
  const int cx = threadIdx.x & 15, ry = threadIdx.x >> 4;
  const int64_t col0 = int64_t(blockIdx.x) * kTile + cx * 8;
  const int64_t row0 = int64_t(blockIdx.y) * kTile + ry * 8;
  uint4 w[8];
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const int64_t row = row0 + r;
    w[r] = (row < rows) ? ld_nc_v4(x + row * cols + col0) : make_uint4(0, 0, 0, 0);
  }
  uint32_t mb = 0u;
#pragma unroll
  for (int r = 0; r < 8; ++r) mb = absmax8(w[r], mb);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mb = __vmaxu2(mb, __shfl_xor_sync(0xffffffffu, mb, o));
  float m = absmax_to_float(mb);
  if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = m;
  __syncthreads();
  m = s_max[0];
#pragma unroll
  for (int wv = 1; wv < 8; ++wv) m = max_nan(m, s_max[wv]);
  const float s = scale_from_amax(m);
  if (threadIdx.x == 0) scales[int64_t(blockIdx.y) * (cols / kTile) + blockIdx.x] = s;
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const int64_t row = row0 + r;
    if (row < rows) *reinterpret_cast<uint2*>(q + row * cols + col0) = quantize8(w[r], s);
  }
}

}  // namespace tg

using namespace tg;

extern "C" int tg_quantize_rowwise(const void* x, void* q, float* scales, int64_t rows,
                                   int64_t cols, void* stream) {
  if (rows < 0 || cols < 0 || cols % kTile != 0) return TG_ERR_SHAPE;
  if (rows == 0 || cols == 0) return TG_OK;
  if (!aligned16(x) || !aligned16(q) || (reinterpret_cast<uintptr_t>(scales) & 3u)) return TG_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  const int64_t n_tiles = rows * (cols / kTile);
  const int64_t tiles_per_block = (kRowThreads / 16) * kRowUnroll;
  int64_t blocks = (n_tiles + tiles_per_block - 1) / tiles_per_block;
  const int64_t cap = int64_t(sm_count()) * 8 * 4;  // 8 resident blocks per SM, 4 waves
  if (blocks > cap) blocks = cap;
  quantize_rowwise_kernel<<<dim3(unsigned(blocks)), kRowThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), static_cast<uint2*>(q), scales, n_tiles);
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}

extern "C" int tg_quantize_colwise(const void* x, void* q, float* scales, int64_t rows,
                                   int64_t cols, void* stream) {
  if (rows < 0 || cols < 0 || cols % 8 != 0) return TG_ERR_SHAPE;
  if (rows == 0 || cols == 0) return TG_OK;
  if (!aligned16(x) || !aligned16(q) || !aligned16(scales)) return TG_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  const int64_t gx = (cols + kColPanelCols - 1) / kColPanelCols, gy = (rows + kTile - 1) / kTile;
  if (gy > 65535) return TG_ERR_TOO_LARGE;
  quantize_colwise_kernel<false><<<dim3(unsigned(gx), unsigned(gy)), kColThreads, 0,
                                   static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scales, nullptr, nullptr, rows, cols);
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}

extern "C" int tg_quantize_rowcol_ld(const void* x, void* q_row, int64_t q_row_ld, float* s_row, int64_t s_row_ld,
                                     void* q_col, int64_t q_col_ld, float* s_col, int64_t s_col_ld, int64_t rows,
                                     int64_t cols, void* stream) {
  if (rows < 0 || cols < 0 || cols % kTile != 0) return TG_ERR_SHAPE;
  if (q_row_ld < cols || q_row_ld % 16 != 0 || s_row_ld < cols / kTile) return TG_ERR_SHAPE;
  if (q_col_ld < cols || q_col_ld % 16 != 0 || s_col_ld < cols) return TG_ERR_SHAPE;
  if (rows == 0 || cols == 0) return TG_OK;
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(q_row) & 7u) || (reinterpret_cast<uintptr_t>(q_col) & 7u) ||
      (reinterpret_cast<uintptr_t>(s_col) & 3u) || (reinterpret_cast<uintptr_t>(s_row) & 3u))
    return TG_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  const int64_t gx = cols / kColPanelCols, gy = (rows + kTile - 1) / kTile;
  if (gy > 65535) return TG_ERR_TOO_LARGE;
  quantize_colwise_kernel<true><<<dim3(unsigned(gx), unsigned(gy)), kColThreads, 0,
                                  static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q_col), s_col, static_cast<uint8_t*>(q_row), s_row, rows,
      cols, nullptr, q_row_ld, s_row_ld, q_col_ld, s_col_ld);
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}

extern "C" int tg_quantize_rowcol(const void* x, void* q_row, float* s_row, void* q_col, float* s_col,
                                  int64_t rows, int64_t cols, void* stream) {
  if (cols > 0 && (!aligned16(q_row) || !aligned16(q_col) || !aligned16(s_col))) return TG_ERR_ALIGN;
  const int64_t ld = cols < 16 ? 16 : cols;
  return tg_quantize_rowcol_ld(x, q_row, ld, s_row, cols / kTile, q_col, ld, s_col, cols, rows, cols, stream);
}

extern "C" int tg_act_quantize_rowcol(const void* x, const void* gate, int act, void* q_row, float* s_row, void* q_col,
                                      float* s_col, int64_t rows, int64_t cols, void* stream) {
  if (rows < 0 || cols < 0 || cols % kTile != 0) return TG_ERR_SHAPE;
  const bool bwd = act == TG_ACT_RELU2_BWD || act == TG_ACT_GELU_BWD;
  if (act != TG_ACT_RELU2 && act != TG_ACT_GELU && !bwd) return TG_ERR_SHAPE;
  if (rows == 0 || cols == 0) return TG_OK;
  if (bwd && gate == nullptr) return TG_ERR_SHAPE;
  if (!aligned16(x) || (bwd && !aligned16(gate)) || !aligned16(q_row) || !aligned16(q_col) || !aligned16(s_col) ||
      (reinterpret_cast<uintptr_t>(s_row) & 3u))
    return TG_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  const int64_t gx = cols / kColPanelCols, gy = (rows + kTile - 1) / kTile;
  if (gy > 65535) return TG_ERR_TOO_LARGE;
  const dim3 grid{unsigned(gx), unsigned(gy)};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* gp = static_cast<const __nv_bfloat16*>(gate);
  uint8_t* qc = static_cast<uint8_t*>(q_col);
  uint8_t* qr = static_cast<uint8_t*>(q_row);
  switch (act) {
    case TG_ACT_RELU2: quantize_colwise_kernel<true, TG_ACT_RELU2><<<grid, kColThreads, 0, st>>>(xp, qc, s_col, qr, s_row, rows, cols, gp); break;
    case TG_ACT_GELU: quantize_colwise_kernel<true, TG_ACT_GELU><<<grid, kColThreads, 0, st>>>(xp, qc, s_col, qr, s_row, rows, cols, gp); break;
    case TG_ACT_RELU2_BWD: quantize_colwise_kernel<true, TG_ACT_RELU2_BWD><<<grid, kColThreads, 0, st>>>(xp, qc, s_col, qr, s_row, rows, cols, gp); break;
    default: quantize_colwise_kernel<true, TG_ACT_GELU_BWD><<<grid, kColThreads, 0, st>>>(xp, qc, s_col, qr, s_row, rows, cols, gp); break;
  }
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}

extern "C" int tg_quantize_block128(const void* x, void* q, float* scales, int64_t rows,
                                    int64_t cols, void* stream) {
  if (rows < 0 || cols < 0 || cols % kTile != 0) return TG_ERR_SHAPE;
  if (rows == 0 || cols == 0) return TG_OK;
  if (!aligned16(x) || !aligned16(q) || (reinterpret_cast<uintptr_t>(scales) & 3u)) return TG_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  const int64_t gx = cols / kTile, gy = (rows + kTile - 1) / kTile;
  if (gy > 65535) return TG_ERR_TOO_LARGE;
  quantize_block128_kernel<<<dim3(unsigned(gx), unsigned(gy)), 256, 0,
                             static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scales, rows, cols);
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}
