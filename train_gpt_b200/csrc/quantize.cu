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
// Column maxima are combined across the half-warps through shared memory, then the same
// registers are divided and stored.  ~90 registers: two blocks per SM, so one block's loads
// overlap the other's arithmetic.
// ---------------------------------------------------------------------------------------
constexpr int kColPanelCols = 128;
constexpr int kColThreads = 256;
constexpr int kColHalfWarps = kColThreads / 16;           // 16
constexpr int kColRowsPerThread = kTile / kColHalfWarps;  // 8

__global__ void __launch_bounds__(kColThreads, 2)
quantize_colwise_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                        float* __restrict__ scales, int64_t rows, int64_t cols) {
  __shared__ float s_max[kColHalfWarps][kColPanelCols];
  const int cx = threadIdx.x & 15, hw = threadIdx.x >> 4;
  const int64_t col0 = int64_t(blockIdx.x) * kColPanelCols + cx * 8;
  const int64_t row_blk = blockIdx.y;
  const int64_t row0 = row_blk * kTile + hw;  // this thread's rows: row0 + 16 r
  const bool col_ok = col0 < cols;            // cols % 8 == 0

  uint4 w[kColRowsPerThread];
#pragma unroll
  for (int r = 0; r < kColRowsPerThread; ++r) {
    const int64_t row = row0 + r * kColHalfWarps;
    w[r] = (col_ok && row < rows) ? ld_nc_v4(x + row * cols + col0) : make_uint4(0, 0, 0, 0);
  }
  float m[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) m[j] = 0.f;
#pragma unroll
  for (int r = 0; r < kColRowsPerThread; ++r) {
    m[0] = max_nan(m[0], fabsf(bf16lo(w[r].x)));
    m[1] = max_nan(m[1], fabsf(bf16hi(w[r].x)));
    m[2] = max_nan(m[2], fabsf(bf16lo(w[r].y)));
    m[3] = max_nan(m[3], fabsf(bf16hi(w[r].y)));
    m[4] = max_nan(m[4], fabsf(bf16lo(w[r].z)));
    m[5] = max_nan(m[5], fabsf(bf16hi(w[r].z)));
    m[6] = max_nan(m[6], fabsf(bf16lo(w[r].w)));
    m[7] = max_nan(m[7], fabsf(bf16hi(w[r].w)));
  }
  float4* dst = reinterpret_cast<float4*>(&s_max[hw][cx * 8]);
  dst[0] = make_float4(m[0], m[1], m[2], m[3]);
  dst[1] = make_float4(m[4], m[5], m[6], m[7]);
  __syncthreads();
  float s[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float v = s_max[0][cx * 8 + j];
#pragma unroll
    for (int h = 1; h < kColHalfWarps; ++h) v = max_nan(v, s_max[h][cx * 8 + j]);
    s[j] = scale_from_amax(v);
  }
  if (!col_ok) return;
  if (hw == 0) {
    float4* sp = reinterpret_cast<float4*>(scales + row_blk * cols + col0);
    sp[0] = make_float4(s[0], s[1], s[2], s[3]);
    sp[1] = make_float4(s[4], s[5], s[6], s[7]);
  }
  bool all_finite = true;
  float rc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    rc[j] = __frcp_rn(s[j]);
    all_finite = all_finite && (fabsf(s[j]) <= 3.402823466e38f);
  }
#pragma unroll
  for (int r = 0; r < kColRowsPerThread; ++r) {
    const int64_t row = row0 + r * kColHalfWarps;
    if (row >= rows) break;
    const uint4 v = w[r];
    const float xs[8] = {bf16lo(v.x), bf16hi(v.x), bf16lo(v.y), bf16hi(v.y),
                         bf16lo(v.z), bf16hi(v.z), bf16lo(v.w), bf16hi(v.w)};
    float qv[8];
    if (all_finite) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {  // x/s as q0 = x*r, q = fma(-fma(q0,s,-x), r, q0): see QuantDiv
        const float q0 = __fmul_rn(xs[j], rc[j]);
        qv[j] = __fmaf_rn(-__fmaf_rn(q0, s[j], -xs[j]), rc[j], q0);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) qv[j] = __fdiv_rn(xs[j], s[j]);
    }
    const uint32_t b0 = cvt_e4m3x2(qv[0], qv[1]), b1 = cvt_e4m3x2(qv[2], qv[3]);
    const uint32_t b2 = cvt_e4m3x2(qv[4], qv[5]), b3 = cvt_e4m3x2(qv[6], qv[7]);
    *reinterpret_cast<uint2*>(q + row * cols + col0) = make_uint2(b0 | (b1 << 16), b2 | (b3 << 16));
  }
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
  float m = 0.f;
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const int64_t row = row0 + r;
    w[r] = (row < rows) ? ld_nc_v4(x + row * cols + col0) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int r = 0; r < 8; ++r) m = amax8(w[r], m);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, o));
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
  quantize_colwise_kernel<<<dim3(unsigned(gx), unsigned(gy)), kColThreads, 0,
                            static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scales, rows, cols);
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
