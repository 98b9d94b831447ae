// RMSNorm forward (optionally fused with the 1x128 e4m3 quantiser) and backward.
//
// Reference semantics: train-gpt kernels.py:44-53 (+ the variance pass at :66) for the
// fused single-rounding norm, kernels.py:30-33 for the "pure" three-rounding norm,
// kernels.py:104-118 for the backward, fp8.py:39-47 + :66 for the quantiser that consumes
// the norm's bf16 output.
//
// Layout: a row is split over WPR warps; each warp owns NCHUNK chunks of 256 columns and
// each lane 8 consecutive columns (one 128-bit load) per chunk, so a half-warp owns
// exactly one 128-column quantisation tile.  The whole row stays in registers between the
// sum-of-squares pass and the normalise/quantise pass: x is read from HBM once.
#include <cstdlib>

#include <atomic>

#include "common.cuh"

namespace tg {

constexpr int kNormWarps = 8;  // warps per thread block


// Sum of squares of the 8 bf16 values in w, as a balanced tree (keeps the rounding error of
// a row's variance at a few 2^-24 regardless of outliers).
__device__ __forceinline__ float sumsq8(const uint4& w) {
  const float2 v0 = bf16x2_unpack(w.x), v1 = bf16x2_unpack(w.y), v2 = bf16x2_unpack(w.z), v3 = bf16x2_unpack(w.w);
  const float2 t = __fadd2_rn(__ffma2_rn(v2, v2, __fmul2_rn(v0, v0)), __ffma2_rn(v3, v3, __fmul2_rn(v1, v1)));
  return t.x + t.y;
}

template <int N>
__device__ __forceinline__ float tree_sum(float (&v)[N]) {
#pragma unroll
  for (int stride = 1; stride < N; stride *= 2)
#pragma unroll
    for (int i = 0; i + stride < N; i += 2 * stride) v[i] += v[i + stride];
  return v[0];
}

template <int WPR>
__device__ __forceinline__ float row_sum(float v, float* s_red, int warp, int lane) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if constexpr (WPR > 1) {
    // s_red: [kNormWarps] floats; the caller separates uses with __syncthreads()
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    const int g0 = (warp / WPR) * WPR;
    v = s_red[g0];
#pragma unroll
    for (int i = 1; i < WPR; ++i) v += s_red[g0 + i];
  }
  return v;
}

// Two blocks per SM when the fused kernel holds a 2048-wide row per warp (three would spill),
// three otherwise.
template <int NCHUNK, int WPR, bool QUANT, bool PURE>
__global__ void __launch_bounds__(kNormWarps * 32, (QUANT && NCHUNK >= 8) ? 2 : 3)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                   float eps, uint8_t* __restrict__ q, float* __restrict__ scales,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ rnorm_out, int64_t rows,
                   int cols) {
  __shared__ float s_red[2][kNormWarps];
  constexpr int RPB = kNormWarps / WPR;  // rows per block per iteration
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col_base = (warp % WPR) * NCHUNK * 256 + lane * 8;

  // gamma lives in shared memory, already widened to float (one conversion per block
  // instead of one per row), not in registers, so that more blocks fit on an SM
  extern __shared__ float4 s_gamma[];
  for (int i = threadIdx.x; i < cols / 8; i += blockDim.x) {
    const uint4 gq = reinterpret_cast<const uint4*>(gamma)[i];
    s_gamma[2 * i] = make_float4(bf16lo(gq.x), bf16hi(gq.x), bf16lo(gq.y), bf16hi(gq.y));
    s_gamma[2 * i + 1] = make_float4(bf16lo(gq.z), bf16hi(gq.z), bf16lo(gq.w), bf16hi(gq.w));
  }
  __syncthreads();

  int it = 0;
  for (int64_t row_base = int64_t(blockIdx.x) * RPB; row_base < rows;
       row_base += int64_t(gridDim.x) * RPB, ++it) {
    const int64_t row = row_base + warp / WPR;
    const bool row_ok = row < rows;
    uint4 w[NCHUNK];
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int col = col_base + c * 256;
      w[c] = (row_ok && col < cols) ? ld_nc_v4(x + row * cols + col) : make_uint4(0, 0, 0, 0);
    }
    float part[NCHUNK];
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) part[c] = sumsq8(w[c]);
    const float ss = row_sum<WPR>(tree_sum(part), s_red[it & 1], warp, lane);
    const float var = __fdiv_rn(ss, float(cols));
    const float rn = __frsqrt_rn(var + eps);
    if (row_ok && rnorm_out != nullptr && lane == 0 && (warp % WPR) == 0) rnorm_out[row] = rn;
    const float rn_b = __bfloat162float(__float2bfloat16_rn(rn));  // kernels.py:32 `.astype(x.dtype)`

    // pass 2a: normalise, round to bf16 (the value the reference's norm returns), per-tile amax
    const float2 rn2 = PURE ? make_float2(rn_b, rn_b) : make_float2(rn, rn);
    uint32_t amax_bits[NCHUNK];
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int col = col_base + c * 256;
      const uint32_t xi[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
      float4 g0 = make_float4(0.f, 0.f, 0.f, 0.f), g1 = g0;
      if (col < cols) {
        g0 = s_gamma[col >> 2];
        g1 = s_gamma[(col >> 2) + 1];
      }
      const float2 gf[4] = {make_float2(g0.x, g0.y), make_float2(g0.z, g0.w), make_float2(g1.x, g1.y), make_float2(g1.z, g1.w)};
      uint4 yo;
      uint32_t* yp = &yo.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 t = __fmul2_rn(bf16x2_unpack(xi[j]), rn2);
        if (PURE) t = bf16x2_unpack(pack_bf16x2(t.x, t.y));   // kernels.py:32 rounds before the gamma multiply
        t = __fmul2_rn(t, gf[j]);
        yp[j] = pack_bf16x2(t.x, t.y);
      }
      if (y != nullptr && row_ok && col < cols) *reinterpret_cast<uint4*>(y + row * cols + col) = yo;
      w[c] = yo;  // the row registers now hold the normalised bf16 values
      if constexpr (QUANT) amax_bits[c] = absmax8(yo);
    }
    if constexpr (QUANT) {
      // pass 2b: one exchange brings lane j of each half the amax of chunk j % NCHUNK; that lane
      // computes the tile's scale and reciprocal, and shuffles hand them to the lanes that need them
      float s[NCHUNK], r[NCHUNK], s_mine;
      bool fin;
      tile_scales_own<NCHUNK>(exchange_tile_amax<NCHUNK>(amax_bits), s, r, s_mine, fin);
      {
        const int j = lane & 15;                       // lane j of a half computed chunk j % NCHUNK
        const int col = col_base - (lane & 15) * 8 + j * 256;   // = first column of that chunk's tile for this half
        if (j < NCHUNK && row_ok && col < cols) scales[row * (cols / kTile) + col / kTile] = s_mine;
      }
      // pass 2c: divide and store
#pragma unroll
      for (int c = 0; c < NCHUNK; ++c) {
        const int col = col_base + c * 256;
        if (row_ok && col < cols)
          *reinterpret_cast<uint2*>(q + row * cols + col) = fin ? quantize8_sr(w[c], s[c], r[c]) : quantize8(w[c], s[c]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Fused norm + quantise for rows that one warp can hold (cols <= 2048), staged through shared
// memory.  The register-resident kernel above needs ~120 registers at 2048 columns, so only
// 16 warps fit on an SM and every warp idles while its next row's loads are in flight.  Here
// each warp owns two row-sized slots of shared memory: cp.async fetches row i+1 into one
// slot while the warp makes its three passes (sum of squares; normalise + amax, writing the
// bf16 result back in place; divide + store) over row i in the other.  A lane only ever
// touches the 16-byte pieces it fetched itself, so cp.async.wait_group is the only
// synchronisation; nothing spins.  Same arithmetic, same results as rmsnorm_fwd_kernel.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

constexpr int kStagedBlocksPerSm = 3;
constexpr int kGroup = 8;   // chunks normalised, scaled and quantised together (their bf16 values stay in registers)

// ADD: the row that is normalised is bf16(x + res) -- the residual add of model.py:68 / :72 folded into
// the norm that follows it -- and is also written to `sum_out` (the new residual stream); `res` rows
// are staged beside the x rows and the sum replaces the x row in shared memory before the first pass.
// q may be NULL (ADD only: the final norm has no quantised consumer), then only y is produced.
template <int NCHUNK, bool PURE, bool FULL, bool ADD = false>
__global__ void __launch_bounds__(kNormWarps * 32, kStagedBlocksPerSm)
rmsnorm_quant_staged_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                            float eps, uint8_t* __restrict__ q, float* __restrict__ scales,
                            __nv_bfloat16* __restrict__ y, float* __restrict__ rnorm_out, int64_t rows,
                            int cols, const __nv_bfloat16* __restrict__ res = nullptr,
                            __nv_bfloat16* __restrict__ sum_out = nullptr) {
  constexpr int kRowBytes = NCHUNK * 512;
  constexpr int kSlotBytes = ADD ? 2 * kRowBytes : kRowBytes;     // x row (then: the sum), res row
  extern __shared__ float4 s_gamma[];   // [cols] floats, then [warps][2][slot] bf16
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col_base = lane * 8;
  const uint32_t slot0 = uint32_t(__cvta_generic_to_shared(s_gamma)) + uint32_t(cols) * 4u +
                         uint32_t(warp) * 2u * kSlotBytes + uint32_t(lane) * 16u;

  // gamma widened to float in two planes (columns 8i..8i+3 of every 8-column piece, then columns
  // 8i+4..8i+7): a warp's 16-byte reads of either plane are contiguous, hence conflict-free
  const int pieces = cols / 8;
  for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
    const uint4 gq = reinterpret_cast<const uint4*>(gamma)[i];
    s_gamma[i] = make_float4(bf16lo(gq.x), bf16hi(gq.x), bf16lo(gq.y), bf16hi(gq.y));
    s_gamma[pieces + i] = make_float4(bf16lo(gq.z), bf16hi(gq.z), bf16lo(gq.w), bf16hi(gq.w));
  }
  __syncthreads();

  const int64_t stride = int64_t(gridDim.x) * kNormWarps;
  int64_t row = int64_t(blockIdx.x) * kNormWarps + warp;
  auto prefetch = [&](int64_t r, int slot) {
    if (r < rows) {
#pragma unroll
      for (int c = 0; c < NCHUNK; ++c) {
        const int col = col_base + c * 256;
        if (FULL || col < cols) {
          cp_async16(slot0 + slot * kSlotBytes + c * 512, x + r * cols + col);
          if (ADD) cp_async16(slot0 + slot * kSlotBytes + kRowBytes + c * 512, res + r * cols + col);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");   // an empty group keeps the wait count uniform
  };
  prefetch(row, 0);
  for (int it = 0; row < rows; row += stride, ++it) {
    const uint32_t base = slot0 + (it & 1) * kSlotBytes;
    prefetch(row + stride, (it & 1) ^ 1);
    asm volatile("cp.async.wait_group 1;" ::: "memory");

    if (ADD) {
      // the residual add, one rounding to bf16 as the elementwise add it replaces
#pragma unroll
      for (int c = 0; c < NCHUNK; ++c) {
        const int col = col_base + c * 256;
        if (FULL || col < cols) {
          const uint4 a = lds128(base + c * 512), b = lds128(base + kRowBytes + c * 512);
          const uint32_t ai[4] = {a.x, a.y, a.z, a.w}, bi[4] = {b.x, b.y, b.z, b.w};
          uint4 o;
          uint32_t* op = &o.x;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 t = __fadd2_rn(bf16x2_unpack(ai[j]), bf16x2_unpack(bi[j]));
            op[j] = pack_bf16x2(t.x, t.y);
          }
          sts128(base + c * 512, o);
          *reinterpret_cast<uint4*>(sum_out + row * cols + col) = o;
        }
      }
    }

    // pass 1: sum of squares
    float part[NCHUNK];
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) part[c] = (FULL || col_base + c * 256 < cols) ? sumsq8(lds128(base + c * 512)) : 0.f;
    float ss = tree_sum(part);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float var = __fdiv_rn(ss, float(cols));
    const float rn = __frsqrt_rn(var + eps);
    if (rnorm_out != nullptr && lane == 0) rnorm_out[row] = rn;
    const float rn_b = __bfloat162float(__float2bfloat16_rn(rn));  // kernels.py:32 `.astype(x.dtype)`

    // pass 2, in groups of G chunks whose normalised values stay in registers: normalise, round
    // to bf16 (the value the reference's norm returns), per-tile amax; one exchange brings lane j
    // of each half the amax of the group's chunk j % G, that lane computes the tile's scale and
    // reciprocal, shuffles hand them to the lanes that need them; divide and store.
    const float2 rn2 = PURE ? make_float2(rn_b, rn_b) : make_float2(rn, rn);
    constexpr int G = NCHUNK < kGroup ? NCHUNK : kGroup;
#pragma unroll
    for (int g = 0; g < NCHUNK / G; ++g) {
      uint4 yo[G];
      uint32_t amax_bits[G];
#pragma unroll
      for (int u = 0; u < G; ++u) {
        const int c = g * G + u;
        const int col = col_base + c * 256;
        amax_bits[u] = 0u;
        yo[u] = make_uint4(0u, 0u, 0u, 0u);
        if (FULL || col < cols) {
          const uint4 xv = lds128(base + c * 512);
          const uint32_t xi[4] = {xv.x, xv.y, xv.z, xv.w};
          const float4 g0 = s_gamma[col >> 3], g1 = s_gamma[pieces + (col >> 3)];
          const float2 gf[4] = {make_float2(g0.x, g0.y), make_float2(g0.z, g0.w), make_float2(g1.x, g1.y), make_float2(g1.z, g1.w)};
          uint32_t* yp = &yo[u].x;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 t = __fmul2_rn(bf16x2_unpack(xi[j]), rn2);
            if (PURE) t = bf16x2_unpack(pack_bf16x2(t.x, t.y));   // kernels.py:32 rounds before the gamma multiply
            t = __fmul2_rn(t, gf[j]);
            yp[j] = pack_bf16x2(t.x, t.y);
          }
          if (y != nullptr) *reinterpret_cast<uint4*>(y + row * cols + col) = yo[u];
          amax_bits[u] = absmax8_h(yo[u]);
        }
      }
      float s[G], r[G], s_mine;
      bool fin;
      tile_scales_own<G>(exchange_tile_amax<G>(amax_bits), s, r, s_mine, fin);
      {
        const int j = lane & 15;
        const int col = (g * G + j) * 256 + (lane & 16) * 8;     // first column of the tile this lane computed
        if (j < G && (FULL || col < cols) && (!ADD || q != nullptr)) scales[row * (cols / kTile) + col / kTile] = s_mine;
      }
      if (ADD && q == nullptr) continue;
      uint8_t* qp = q + row * cols + col_base + g * G * 256;
      if (fin) {   // one branch per group: a NaN or Inf in any of the warp's tiles is the rare case
#pragma unroll
        for (int u = 0; u < G; ++u)
          if (FULL || col_base + (g * G + u) * 256 < cols) *reinterpret_cast<uint2*>(qp + u * 256) = quantize8_sr(yo[u], s[u], r[u]);
      } else {
#pragma unroll
        for (int u = 0; u < G; ++u)
          if (FULL || col_base + (g * G + u) * 256 < cols) *reinterpret_cast<uint2*>(qp + u * 256) = quantize8(yo[u], s[u]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ---------------------------------------------------------------------------------------
// Backward.  Per row: S1 = sum x^2, rnorm = rsqrt(S1/D + eps), normed = x*rnorm,
// gs = g*gamma, dot = mean(gs*normed), dx = rnorm*(gs - normed*dot); per column:
// dgamma = sum_rows g*normed, accumulated per lane in registers over all rows the block
// visits, combined across the block's warps in shared memory, written as one float32 row
// of `partial` per block and reduced over blocks (in block order) by a second kernel.
// ---------------------------------------------------------------------------------------
template <int NCHUNK, int WPR>
__global__ void __launch_bounds__(kNormWarps * 32)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                   const __nv_bfloat16* __restrict__ g, float eps, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ partial, int64_t rows, int cols) {
  extern __shared__ float s_dyn[];  // [cols] column sums of this block
  __shared__ float s_red[4][kNormWarps];
  constexpr int RPB = kNormWarps / WPR;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col_base = (warp % WPR) * NCHUNK * 256 + lane * 8;
  const float inv_d = __fdiv_rn(1.0f, float(cols));

  float acc[NCHUNK][8];
#pragma unroll
  for (int c = 0; c < NCHUNK; ++c)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[c][j] = 0.f;

  int it = 0;
  for (int64_t row_base = int64_t(blockIdx.x) * RPB; row_base < rows;
       row_base += int64_t(gridDim.x) * RPB, ++it) {
    const int64_t row = row_base + warp / WPR;
    const bool row_ok = row < rows;
    uint4 w[NCHUNK], gv[NCHUNK];
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int col = col_base + c * 256;
      const bool ok = row_ok && col < cols;
      w[c] = ok ? ld_nc_v4(x + row * cols + col) : make_uint4(0, 0, 0, 0);
      gv[c] = ok ? ld_nc_v4(g + row * cols + col) : make_uint4(0, 0, 0, 0);
    }
    float part[NCHUNK];
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) part[c] = sumsq8(w[c]);
    const float ss = row_sum<WPR>(tree_sum(part), s_red[(it & 1) * 2], warp, lane);
    const float rn = __frsqrt_rn(__fdiv_rn(ss, float(cols)) + eps);

    // gs*normed summed over the row; dgamma accumulation in the same sweep
    float dpart[NCHUNK];
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      float dsum = 0.f;
      const int col = col_base + c * 256;
      const uint4 gm = (col < cols) ? *reinterpret_cast<const uint4*>(gamma + col) : make_uint4(0, 0, 0, 0);
      const uint32_t xi[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
      const uint32_t gi[4] = {gv[c].x, gv[c].y, gv[c].z, gv[c].w};
      const uint32_t mi[4] = {gm.x, gm.y, gm.z, gm.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float n0 = __fmul_rn(bf16lo(xi[j]), rn), n1 = __fmul_rn(bf16hi(xi[j]), rn);
        const float g0 = bf16lo(gi[j]), g1 = bf16hi(gi[j]);
        acc[c][2 * j] = fmaf(g0, n0, acc[c][2 * j]);
        acc[c][2 * j + 1] = fmaf(g1, n1, acc[c][2 * j + 1]);
        dsum = fmaf(__fmul_rn(g0, bf16lo(mi[j])), n0, dsum);
        dsum = fmaf(__fmul_rn(g1, bf16hi(mi[j])), n1, dsum);
      }
      dpart[c] = dsum;
    }
    const float dsum = row_sum<WPR>(tree_sum(dpart), s_red[(it & 1) * 2 + 1], warp, lane);
    const float dot = __fmul_rn(dsum, inv_d);

#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int col = col_base + c * 256;
      if (!(row_ok && col < cols)) continue;
      const uint4 gm = *reinterpret_cast<const uint4*>(gamma + col);
      const uint32_t xi[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
      const uint32_t gi[4] = {gv[c].x, gv[c].y, gv[c].z, gv[c].w};
      const uint32_t mi[4] = {gm.x, gm.y, gm.z, gm.w};
      uint4 o;
      uint32_t* op = &o.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float n0 = __fmul_rn(bf16lo(xi[j]), rn), n1 = __fmul_rn(bf16hi(xi[j]), rn);
        const float gs0 = __fmul_rn(bf16lo(gi[j]), bf16lo(mi[j]));
        const float gs1 = __fmul_rn(bf16hi(gi[j]), bf16hi(mi[j]));
        // rnorm * (gs - normed*dot), the subtraction fused as kernels.py:114 allows XLA to
        const float d0 = __fmul_rn(rn, fmaf(-n0, dot, gs0));
        const float d1 = __fmul_rn(rn, fmaf(-n1, dot, gs1));
        op[j] = pack_bf16x2(d0, d1);
      }
      *reinterpret_cast<uint4*>(dx + row * cols + col) = o;
    }
  }

  // combine the block's warps in a fixed order, then publish the block's row of partials
  for (int i = threadIdx.x; i < cols; i += blockDim.x) s_dyn[i] = 0.f;
  __syncthreads();
  for (int turn = 0; turn < RPB; ++turn) {
    if (warp / WPR == turn) {
#pragma unroll
      for (int c = 0; c < NCHUNK; ++c) {
        const int col = col_base + c * 256;
        if (col < cols) {
#pragma unroll
          for (int j = 0; j < 8; ++j) s_dyn[col + j] += acc[c][j];
        }
      }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < cols; i += blockDim.x) partial[int64_t(blockIdx.x) * cols + i] = s_dyn[i];
}

// ---------------------------------------------------------------------------------------
// Backward for rows that one warp can hold (cols <= 2048), staged through shared memory.
// The register-resident kernel above keeps x, g and 8 column sums per 16-byte piece live at
// once (246 registers at 2048 columns: one block of eight warps per SM, each idle while its
// next row is in flight; it reached 55 % of the copy bandwidth).  Here each warp owns SLOTS
// pairs of row-sized shared-memory slots and cp.async keeps SLOTS - 1 rows of x and g in flight
// while one is processed:
// x goes to registers once, g is read from shared memory in the column-sum pass and again in
// the dx pass, gamma sits in shared memory widened to float.  Every lane reads only the
// 16-byte pieces it fetched itself, so cp.async.wait_group is the only synchronisation.
// The arithmetic per row is the same sequence as in rmsnorm_bwd_kernel: dx comes out
// bit-identical; dgamma sums the same products in another (still fixed) order.
// ---------------------------------------------------------------------------------------
// ADD: dx = bf16(addend + the norm's input gradient) -- the gradient fan-in at a residual junction (the
// skip path's gradient plus the branch's) folded into the kernel, one rounding instead of two.
template <int NCHUNK, int WARPS, int SLOTS, bool FULL, bool ADD = false>
__global__ void __launch_bounds__(WARPS * 32, 1)
rmsnorm_bwd_staged_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                          const __nv_bfloat16* __restrict__ g, float eps, __nv_bfloat16* __restrict__ dx,
                          float* __restrict__ partial, int64_t rows, int cols,
                          const __nv_bfloat16* __restrict__ addend = nullptr) {
  constexpr int kRowBytes = NCHUNK * 512;
  extern __shared__ float4 s_gamma[];   // [cols] floats in two planes, then [warps][SLOTS][x row | g row] bf16
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col_base = lane * 8;
  const uint32_t stage0 = uint32_t(__cvta_generic_to_shared(s_gamma)) + uint32_t(cols) * 4u;
  const uint32_t slot0 = stage0 + uint32_t(warp) * uint32_t(SLOTS * 2 * kRowBytes) + uint32_t(lane) * 16u;
  const float inv_d = __fdiv_rn(1.0f, float(cols));

  const int pieces = cols / 8;
  for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
    const uint4 gq = reinterpret_cast<const uint4*>(gamma)[i];
    s_gamma[i] = make_float4(bf16lo(gq.x), bf16hi(gq.x), bf16lo(gq.y), bf16hi(gq.y));
    s_gamma[pieces + i] = make_float4(bf16lo(gq.z), bf16hi(gq.z), bf16lo(gq.w), bf16hi(gq.w));
  }
  __syncthreads();

  float acc[NCHUNK][8];
#pragma unroll
  for (int c = 0; c < NCHUNK; ++c)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[c][j] = 0.f;

  const int64_t stride = int64_t(gridDim.x) * WARPS;
  int64_t row = int64_t(blockIdx.x) * WARPS + warp;
  auto prefetch = [&](int64_t r, int slot) {
    if (r < rows) {
      const uint32_t dst = slot0 + uint32_t(slot) * 2u * kRowBytes;
#pragma unroll
      for (int c = 0; c < NCHUNK; ++c) {
        const int col = col_base + c * 256;
        if (FULL || col < cols) {
          cp_async16(dst + c * 512, x + r * cols + col);
          cp_async16(dst + kRowBytes + c * 512, g + r * cols + col);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");   // an empty group keeps the wait count uniform
  };
  // SLOTS - 1 rows are in flight while one is processed
#pragma unroll
  for (int d = 0; d < SLOTS - 1; ++d) prefetch(row + d * stride, d);
  int slot = 0, slot_in = SLOTS - 1;
  for (; row < rows; row += stride) {
    const uint32_t xs = slot0 + uint32_t(slot) * 2u * kRowBytes, gs = xs + kRowBytes;
    prefetch(row + (SLOTS - 1) * stride, slot_in);    // into the slot the previous iteration finished with
    asm volatile("cp.async.wait_group %0;" ::"n"(SLOTS - 1) : "memory");
    slot_in = slot;
    if (++slot == SLOTS) slot = 0;

    uint4 w[NCHUNK];
    float part[NCHUNK];
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      w[c] = (FULL || col_base + c * 256 < cols) ? lds128(xs + c * 512) : make_uint4(0, 0, 0, 0);
      part[c] = sumsq8(w[c]);
    }
    float ss = tree_sum(part);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rn = __frsqrt_rn(__fdiv_rn(ss, float(cols)) + eps);

    // (ADD) the addend's pieces are fetched here, ahead of the pass that uses them, when the row is
    // narrow enough for the registers; wider rows fetch them where they are used
    constexpr bool kAddEarly = ADD && NCHUNK <= 4;
    uint4 ad[kAddEarly ? NCHUNK : 1];
    if constexpr (kAddEarly) {
#pragma unroll
      for (int c = 0; c < NCHUNK; ++c)
        ad[c] = (FULL || col_base + c * 256 < cols) ? ld_nc_v4(addend + row * cols + col_base + c * 256) : make_uint4(0, 0, 0, 0);
    }

    // column sums of g * normed, and gs * normed summed over the row
    float dpart[NCHUNK];
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      float dsum = 0.f;
      const int col = col_base + c * 256;
      if (FULL || col < cols) {
        const uint4 gv = lds128(gs + c * 512);
        const float4 m0 = s_gamma[col >> 3], m1 = s_gamma[pieces + (col >> 3)];
        const float mf[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        const uint32_t xi[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
        const uint32_t gi[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float n0 = __fmul_rn(bf16lo(xi[j]), rn), n1 = __fmul_rn(bf16hi(xi[j]), rn);
          const float g0 = bf16lo(gi[j]), g1 = bf16hi(gi[j]);
          acc[c][2 * j] = fmaf(g0, n0, acc[c][2 * j]);
          acc[c][2 * j + 1] = fmaf(g1, n1, acc[c][2 * j + 1]);
          dsum = fmaf(__fmul_rn(g0, mf[2 * j]), n0, dsum);
          dsum = fmaf(__fmul_rn(g1, mf[2 * j + 1]), n1, dsum);
        }
      }
      dpart[c] = dsum;
    }
    float dsum = tree_sum(dpart);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, o);
    const float dot = __fmul_rn(dsum, inv_d);

    // (no instruction: stops the compiler from keeping the 8 * NCHUNK normalised values of the pass
    // above alive for the pass below, which costs more registers than recomputing them)
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) asm volatile("" : "+r"(w[c].x), "+r"(w[c].y), "+r"(w[c].z), "+r"(w[c].w));
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int col = col_base + c * 256;
      if (!(FULL || col < cols)) continue;
      const uint4 gv = lds128(gs + c * 512);
      const float4 m0 = s_gamma[col >> 3], m1 = s_gamma[pieces + (col >> 3)];
      const float mf[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
      const uint32_t xi[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
      const uint32_t gi[4] = {gv.x, gv.y, gv.z, gv.w};
      uint4 av = make_uint4(0, 0, 0, 0);
      if constexpr (ADD) av = kAddEarly ? ad[kAddEarly ? c : 0] : ld_nc_v4(addend + row * cols + col);
      const uint32_t ai[4] = {av.x, av.y, av.z, av.w};
      uint4 o;
      uint32_t* op = &o.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float n0 = __fmul_rn(bf16lo(xi[j]), rn), n1 = __fmul_rn(bf16hi(xi[j]), rn);
        const float gs0 = __fmul_rn(bf16lo(gi[j]), mf[2 * j]);
        const float gs1 = __fmul_rn(bf16hi(gi[j]), mf[2 * j + 1]);
        // rnorm * (gs - normed*dot), the subtraction fused as kernels.py:114 allows XLA to
        float d0 = __fmul_rn(rn, fmaf(-n0, dot, gs0));
        float d1 = __fmul_rn(rn, fmaf(-n1, dot, gs1));
        if constexpr (ADD) {
          d0 = __fadd_rn(d0, bf16lo(ai[j]));
          d1 = __fadd_rn(d1, bf16hi(ai[j]));
        }
        op[j] = pack_bf16x2(d0, d1);
      }
      *reinterpret_cast<uint4*>(dx + row * cols + col) = o;
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // combine the block's warps in warp order over the (now idle) staging area, then publish the
  // block's row of partial column sums
  __syncthreads();
  float* s_sum = reinterpret_cast<float*>(s_gamma) + cols;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) s_sum[i] = 0.f;
  __syncthreads();
  for (int turn = 0; turn < WARPS; ++turn) {
    if (warp == turn) {
#pragma unroll
      for (int c = 0; c < NCHUNK; ++c) {
        const int col = col_base + c * 256;
        if (FULL || col < cols) {
          float4* dst = reinterpret_cast<float4*>(s_sum + col);
          float4 a = dst[0], b = dst[1];
          a.x += acc[c][0]; a.y += acc[c][1]; a.z += acc[c][2]; a.w += acc[c][3];
          b.x += acc[c][4]; b.y += acc[c][5]; b.z += acc[c][6]; b.w += acc[c][7];
          dst[0] = a; dst[1] = b;
        }
      }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < cols; i += blockDim.x) partial[int64_t(blockIdx.x) * cols + i] = s_sum[i];
}

// Column sums of the per-block partials.  A thread block owns 32 columns; its eight warps take the
// partial rows b = warp, warp + 8, ... (four independent sums each, so a warp has four loads in
// flight), and the eight results are added in warp order: the order of additions is fixed by
// (n_blocks, cols) alone.  With one thread per column walking all rows the kernel was a chain of
// ~n_blocks / 4 dependent L2 round trips on eight thread blocks: 13 us at 1024 columns.
__global__ void __launch_bounds__(256)
rmsnorm_dgamma_reduce_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ dgamma,
                             int n_blocks, int cols) {
  __shared__ float s_part[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (col < cols) {
    int b = warp;
    for (; b + 24 < n_blocks; b += 32) {
      s0 += partial[int64_t(b) * cols + col];
      s1 += partial[int64_t(b + 8) * cols + col];
      s2 += partial[int64_t(b + 16) * cols + col];
      s3 += partial[int64_t(b + 24) * cols + col];
    }
    for (; b < n_blocks; b += 8) s0 += partial[int64_t(b) * cols + col];
  }
  s_part[warp][lane] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (warp == 0 && col < cols) {
    float t = s_part[0][lane];
#pragma unroll
    for (int w = 1; w < 8; ++w) t += s_part[w][lane];
    dgamma[col] = __float2bfloat16_rn(t);
  }
}

struct NormGeom {
  int nchunk, wpr;
};

// Smallest (NCHUNK, WPR) with WPR * NCHUNK * 256 >= cols; NCHUNK <= 8 keeps the row in
// registers, WPR <= 4 keeps at least two rows per block.
static bool norm_geom(int64_t cols, NormGeom* g) {
  if (cols <= 0 || cols > 8192) return false;
  const int chunks = int((cols + 255) / 256);
  int wpr = 1;
  while (chunks > wpr * 8) wpr *= 2;
  int nchunk = 1;
  while (nchunk * wpr < chunks) nchunk *= 2;
  g->nchunk = nchunk;
  g->wpr = wpr;
  return true;
}

static int norm_blocks(int64_t rows, int wpr, int per_sm) {
  const int rpb = kNormWarps / wpr;
  int64_t need = (rows + rpb - 1) / rpb;
  const int64_t cap = int64_t(sm_count()) * per_sm;
  return int(need < cap ? need : cap);
}

template <bool QUANT>
static int launch_fwd(const void* x, const void* gamma, float eps, void* q, float* scales, void* y,
                      float* rnorm, int64_t rows, int64_t cols, int mode, cudaStream_t st) {
  NormGeom g;
  if (!norm_geom(cols, &g)) return cols > 8192 ? TG_ERR_TOO_LARGE : TG_ERR_SHAPE;
  if (QUANT && g.wpr == 1) {
    const size_t smem = size_t(cols) * 4 + size_t(kNormWarps) * 2 * g.nchunk * 512;
    const int blocks = norm_blocks(rows, 1, kStagedBlocksPerSm);
    int dev = 0;
    TG_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return TG_ERR_SHAPE;
#define TG_STAGED_CASE(NC)                                                                       \
  if (g.nchunk == NC) {                                                                          \
    const bool full = cols == NC * 256;   /* no ragged chunk: the column guards compile away */ \
    auto kern = mode == TG_NORM_PURE                                                             \
                    ? (full ? rmsnorm_quant_staged_kernel<NC, true, true> : rmsnorm_quant_staged_kernel<NC, true, false>)   \
                    : (full ? rmsnorm_quant_staged_kernel<NC, false, true> : rmsnorm_quant_staged_kernel<NC, false, false>); \
    static bool attr_set[4][64] = {};                                                            \
    if (!attr_set[(mode == TG_NORM_PURE) * 2 + full][dev]) {                                     \
      TG_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                         int(2048 * 4 + kNormWarps * 2 * NC * 512)));            \
      attr_set[(mode == TG_NORM_PURE) * 2 + full][dev] = true;                                   \
    }                                                                                            \
    kern<<<blocks, kNormWarps * 32, smem, st>>>(                                                 \
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gamma), eps,     \
        static_cast<uint8_t*>(q), scales, static_cast<__nv_bfloat16*>(y), rnorm, rows,           \
        int(cols), nullptr, nullptr);                                                            \
  } else
    TG_STAGED_CASE(1) TG_STAGED_CASE(2) TG_STAGED_CASE(4) TG_STAGED_CASE(8) { return TG_ERR_SHAPE; }
#undef TG_STAGED_CASE
    TG_CUDA_CHECK(cudaGetLastError());
    return TG_OK;
  }
  const int blocks = norm_blocks(rows, g.wpr, 16);
#define TG_FWD_CASE(NC, W)                                                                      \
  if (g.nchunk == NC && g.wpr == W) {                                                           \
    auto kern = mode == TG_NORM_PURE ? rmsnorm_fwd_kernel<NC, W, QUANT, true>                   \
                                     : rmsnorm_fwd_kernel<NC, W, QUANT, false>;                 \
    kern<<<blocks, kNormWarps * 32, size_t(cols) * 4, st>>>(                                    \
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gamma), eps,    \
        static_cast<uint8_t*>(q), scales, static_cast<__nv_bfloat16*>(y), rnorm, rows,          \
        int(cols));                                                                             \
  } else
  TG_FWD_CASE(1, 1) TG_FWD_CASE(2, 1) TG_FWD_CASE(4, 1) TG_FWD_CASE(8, 1) TG_FWD_CASE(8, 2)
  TG_FWD_CASE(8, 4) { return TG_ERR_SHAPE; }
#undef TG_FWD_CASE
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}

constexpr int kBwdBlocksPerSm = 2;

// Rows one warp can hold run staged, one block per SM with 192 KB of row slots: 8 warps x 3 slots
// at 2048 columns, 12 x 4 at 1024, 16 x 4 below; wider rows stay register-resident.
static int bwd_staged_warps(const NormGeom& g) { return g.wpr != 1 ? 0 : g.nchunk >= 8 ? 8 : g.nchunk == 4 ? 12 : 16; }

static int bwd_blocks(int64_t rows, const NormGeom& g) {
  const int w = bwd_staged_warps(g);
  if (w == 0) return norm_blocks(rows, g.wpr, kBwdBlocksPerSm);
  const int64_t need = (rows + w - 1) / w, cap = sm_count();
  return int(need < cap ? need : cap);
}

}  // namespace tg

using namespace tg;

extern "C" int tg_rmsnorm_fwd(const void* x, const void* gamma, float eps, void* y, float* rnorm,
                              int64_t rows, int64_t cols, int mode, void* stream) {
  if (rows < 0 || cols <= 0 || cols % 8 != 0 || (mode != TG_NORM_FUSED && mode != TG_NORM_PURE)) return TG_ERR_SHAPE;
  if (rows == 0) return TG_OK;
  if (!aligned16(x) || !aligned16(gamma) || !aligned16(y)) return TG_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  return launch_fwd<false>(x, gamma, eps, nullptr, nullptr, y, rnorm, rows, cols, mode,
                           static_cast<cudaStream_t>(stream));
}

extern "C" int tg_rmsnorm_quant_fwd(const void* x, const void* gamma, float eps, void* q,
                                    float* scales, void* y, float* rnorm, int64_t rows,
                                    int64_t cols, int mode, void* stream) {
  if (rows < 0 || cols <= 0 || cols % kTile != 0 || (mode != TG_NORM_FUSED && mode != TG_NORM_PURE)) return TG_ERR_SHAPE;
  if (rows == 0) return TG_OK;
  if (!aligned16(x) || !aligned16(gamma) || !aligned16(q) || !aligned16(y)) return TG_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  return launch_fwd<true>(x, gamma, eps, q, scales, y, rnorm, rows, cols, mode,
                          static_cast<cudaStream_t>(stream));
}

extern "C" int tg_add_rmsnorm_quant_fwd(const void* x, const void* res, const void* gamma, float eps, void* sum_out,
                                        void* q, float* scales, void* y, float* rnorm, int64_t rows, int64_t cols,
                                        int mode, void* stream) {
  if (rows < 0 || cols <= 0 || cols % kTile != 0 || (mode != TG_NORM_FUSED && mode != TG_NORM_PURE)) return TG_ERR_SHAPE;
  if (x == nullptr || res == nullptr || sum_out == nullptr || (q == nullptr) != (scales == nullptr)) return TG_ERR_SHAPE;
  if (q == nullptr && y == nullptr) return TG_ERR_SHAPE;
  if (rows == 0) return TG_OK;
  if (!aligned16(x) || !aligned16(res) || !aligned16(gamma) || !aligned16(q) || !aligned16(y) || !aligned16(sum_out)) return TG_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  NormGeom g;
  if (!norm_geom(cols, &g)) return cols > 8192 ? TG_ERR_TOO_LARGE : TG_ERR_SHAPE;
  if (g.wpr != 1) return TG_ERR_TOO_LARGE;      // rows one warp holds (cols <= 2048): the staged kernel
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = size_t(cols) * 4 + size_t(kNormWarps) * 2 * 2 * g.nchunk * 512;
  const int blocks = norm_blocks(rows, 1, kStagedBlocksPerSm);
  int dev = 0;
  TG_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return TG_ERR_SHAPE;
#define TG_ADD_CASE(NC)                                                                          \
  if (g.nchunk == NC) {                                                                          \
    const bool full = cols == NC * 256;                                                          \
    auto kern = mode == TG_NORM_PURE                                                             \
                    ? (full ? rmsnorm_quant_staged_kernel<NC, true, true, true> : rmsnorm_quant_staged_kernel<NC, true, false, true>)   \
                    : (full ? rmsnorm_quant_staged_kernel<NC, false, true, true> : rmsnorm_quant_staged_kernel<NC, false, false, true>); \
    static bool attr_set[4][64] = {};                                                            \
    if (!attr_set[(mode == TG_NORM_PURE) * 2 + full][dev]) {                                     \
      TG_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                         int(2048 * 4 + kNormWarps * 2 * 2 * NC * 512)));        \
      attr_set[(mode == TG_NORM_PURE) * 2 + full][dev] = true;                                   \
    }                                                                                            \
    kern<<<blocks, kNormWarps * 32, smem, st>>>(                                                 \
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gamma), eps,     \
        static_cast<uint8_t*>(q), scales, static_cast<__nv_bfloat16*>(y), rnorm, rows,           \
        int(cols), static_cast<const __nv_bfloat16*>(res), static_cast<__nv_bfloat16*>(sum_out)); \
  } else
  TG_ADD_CASE(1) TG_ADD_CASE(2) TG_ADD_CASE(4) TG_ADD_CASE(8) { return TG_ERR_SHAPE; }
#undef TG_ADD_CASE
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}

extern "C" int64_t tg_rmsnorm_bwd_scratch_bytes(int64_t rows, int64_t cols) {
  NormGeom g;
  if (rows <= 0 || !norm_geom(cols, &g)) return 0;
  return int64_t(bwd_blocks(rows, g)) * cols * int64_t(sizeof(float));
}

static int rmsnorm_bwd_impl(const void* x, const void* gamma, const void* g, const void* addend, float eps, void* dx,
                            void* dgamma, void* scratch, int64_t rows, int64_t cols, void* stream) {
  if (rows < 0 || cols <= 0 || cols % 8 != 0) return TG_ERR_SHAPE;
  NormGeom geo;
  if (!norm_geom(cols, &geo)) return cols > 8192 ? TG_ERR_TOO_LARGE : TG_ERR_SHAPE;
  if (addend != nullptr && bwd_staged_warps(geo) == 0) return TG_ERR_TOO_LARGE;   // the fused add exists for rows one warp holds
  if (!aligned16(x) || !aligned16(gamma) || !aligned16(g) || !aligned16(dx) || !aligned16(scratch) || !aligned16(addend))
    return TG_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    TG_CUDA_CHECK(cudaMemsetAsync(dgamma, 0, size_t(cols) * 2, st));
    return TG_OK;
  }
  const int blocks = bwd_blocks(rows, geo);
  if (bwd_staged_warps(geo) != 0) {
    int dev = 0;
    TG_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return TG_ERR_SHAPE;
    const bool full = cols == int64_t(geo.nchunk) * 256;   // no ragged chunk: the column guards compile away
#define TG_BWD_STAGED_CASE(NC, WARPS, SLOTS)                                                      \
  if (geo.nchunk == NC) {                                                                         \
    const bool add = addend != nullptr;                                                           \
    auto kern = add ? (full ? rmsnorm_bwd_staged_kernel<NC, WARPS, SLOTS, true, true>             \
                            : rmsnorm_bwd_staged_kernel<NC, WARPS, SLOTS, false, true>)           \
                    : (full ? rmsnorm_bwd_staged_kernel<NC, WARPS, SLOTS, true, false>            \
                            : rmsnorm_bwd_staged_kernel<NC, WARPS, SLOTS, false, false>);         \
    constexpr int kStage = WARPS * SLOTS * 2 * NC * 512;                                          \
    static_assert(NC * 256 * 4 + kStage <= 227 * 1024, "row slots exceed shared memory");         \
    static bool attr_set[4][64] = {};                                                             \
    if (!attr_set[add * 2 + full][dev]) {                                                         \
      TG_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                         NC * 256 * 4 + kStage));                                 \
      attr_set[add * 2 + full][dev] = true;                                                       \
    }                                                                                             \
    kern<<<blocks, WARPS * 32, size_t(cols) * 4 + size_t(kStage), st>>>(                          \
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gamma),           \
        static_cast<const __nv_bfloat16*>(g), eps, static_cast<__nv_bfloat16*>(dx),               \
        static_cast<float*>(scratch), rows, int(cols), static_cast<const __nv_bfloat16*>(addend)); \
  } else
    TG_BWD_STAGED_CASE(1, 16, 4) TG_BWD_STAGED_CASE(2, 16, 4) TG_BWD_STAGED_CASE(4, 12, 4) TG_BWD_STAGED_CASE(8, 8, 3) { return TG_ERR_SHAPE; }
#undef TG_BWD_STAGED_CASE
    TG_CUDA_CHECK(cudaGetLastError());
    rmsnorm_dgamma_reduce_kernel<<<int((cols + 31) / 32), 256, 0, st>>>(
        static_cast<const float*>(scratch), static_cast<__nv_bfloat16*>(dgamma), blocks, int(cols));
    TG_CUDA_CHECK(cudaGetLastError());
    return TG_OK;
  }
  const size_t smem = size_t(cols) * sizeof(float);
#define TG_BWD_CASE(NC, W)                                                                      \
  if (geo.nchunk == NC && geo.wpr == W) {                                                       \
    rmsnorm_bwd_kernel<NC, W><<<blocks, kNormWarps * 32, smem, st>>>(                           \
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gamma),         \
        static_cast<const __nv_bfloat16*>(g), eps, static_cast<__nv_bfloat16*>(dx),             \
        static_cast<float*>(scratch), rows, int(cols));                                         \
  } else
  TG_BWD_CASE(1, 1) TG_BWD_CASE(2, 1) TG_BWD_CASE(4, 1) TG_BWD_CASE(8, 1) TG_BWD_CASE(8, 2)
  TG_BWD_CASE(8, 4) { return TG_ERR_SHAPE; }
#undef TG_BWD_CASE
  TG_CUDA_CHECK(cudaGetLastError());
  rmsnorm_dgamma_reduce_kernel<<<int((cols + 31) / 32), 256, 0, st>>>(
      static_cast<const float*>(scratch), static_cast<__nv_bfloat16*>(dgamma), blocks, int(cols));
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}

extern "C" int tg_rmsnorm_bwd(const void* x, const void* gamma, const void* g, float eps, void* dx,
                              void* dgamma, void* scratch, int64_t rows, int64_t cols, void* stream) {
  return rmsnorm_bwd_impl(x, gamma, g, nullptr, eps, dx, dgamma, scratch, rows, cols, stream);
}

extern "C" int tg_rmsnorm_bwd_add(const void* x, const void* gamma, const void* g, const void* addend, float eps,
                                  void* dx, void* dgamma, void* scratch, int64_t rows, int64_t cols, void* stream) {
  if (addend == nullptr) return TG_ERR_SHAPE;
  return rmsnorm_bwd_impl(x, gamma, g, addend, eps, dx, dgamma, scratch, rows, cols, stream);
}

// ---------------------------------------------------------------------------------------
// Norm backward for callers that may not allocate device memory.
//
// tg_rmsnorm_bwd wants a scratch buffer from its caller.  Some hosts of this library have
// nowhere to get one: an XLA custom-call handler receives only the buffers the compiler
// planned for it, and the reference's launchers hand XLA 90 % of the device up front
// (XLA_PYTHON_CLIENT_MEM_FRACTION=0.9, train-gpt bench_fp8_norm.py:64), so a cudaMalloc
// from inside the handler can fail outright or stall the stream it synchronises with.
// For them the partial column sums live in a fixed array inside the library image.  Every
// GPU that loads the library carries these 4 MiB until the process exits.
// ---------------------------------------------------------------------------------------
namespace tg {
constexpr int64_t kStaticBwdScratchBytes = 4ll << 20;
static __device__ __align__(256) unsigned char g_bwd_scratch[kStaticBwdScratchBytes];
}  // namespace tg

extern "C" int64_t tg_rmsnorm_bwd_static_max_scratch_bytes(void) { return tg::kStaticBwdScratchBytes; }

extern "C" int tg_rmsnorm_bwd_static(const void* x, const void* gamma, const void* g, float eps,
                                     void* dx, void* dgamma, int64_t rows, int64_t cols, void* stream) {
  // In host code `g_bwd_scratch` is only a handle for the runtime, not an address a kernel
  // can use; the device address is looked up once per device, with that device current.
  static std::atomic<void*> dev_ptr[64] = {};   // written once per device; host threads may race to be first
  if (rows < 0 || cols <= 0 || cols % 8 != 0) return TG_ERR_SHAPE;
  const int64_t need = tg_rmsnorm_bwd_scratch_bytes(rows, cols);
  if (need > tg::kStaticBwdScratchBytes) {
    // message for tg_last_cuda_error(): the size limit is the caller's to handle
    tg::record_cuda_error(cudaErrorInvalidValue,
                          "tg_rmsnorm_bwd_static: rows x cols needs more than the 4 MiB built-in scratch; "
                          "use tg_rmsnorm_bwd with a caller-owned buffer");
    return TG_ERR_TOO_LARGE;
  }
  int dev = 0;
  TG_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return TG_ERR_SHAPE;
  void* scratch = dev_ptr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    TG_CUDA_CHECK(cudaGetSymbolAddress(&scratch, tg::g_bwd_scratch));
    dev_ptr[dev].store(scratch, std::memory_order_release);  // racing first calls on one device store the same value
  }
  return tg_rmsnorm_bwd(x, gamma, g, eps, dx, dgamma, scratch, rows, cols, stream);
}
