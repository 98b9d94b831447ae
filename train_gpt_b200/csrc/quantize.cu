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
// 128-row x 256-column panel: 32 lanes x 8 columns across, 8 warps x 16 rows down.  Each
// thread holds its 16 x 8 values in registers, column maxima are combined across the 8
// warps through shared memory, then the same registers are divided and stored.
// ---------------------------------------------------------------------------------------
constexpr int kColPanelCols = 256;
constexpr int kColWarps = 8;
constexpr int kColRowsPerWarp = kTile / kColWarps;  // 16

__global__ void __launch_bounds__(kColWarps * 32)
quantize_colwise_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                        float* __restrict__ scales, int64_t rows, int64_t cols) {
  __shared__ float s_max[kColWarps][kColPanelCols];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t col0 = int64_t(blockIdx.x) * kColPanelCols + lane * 8;
  const int64_t row_blk = blockIdx.y;
  const int64_t row0 = row_blk * kTile + warp * kColRowsPerWarp;
  const bool col_ok = col0 < cols;  // cols % 8 == 0

  uint4 w[kColRowsPerWarp];
#pragma unroll
  for (int r = 0; r < kColRowsPerWarp; ++r) {
    const int64_t row = row0 + r;
    w[r] = (col_ok && row < rows) ? ld_nc_v4(x + row * cols + col0) : make_uint4(0, 0, 0, 0);
  }
  float m[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) m[j] = 0.f;
#pragma unroll
  for (int r = 0; r < kColRowsPerWarp; ++r) {
    m[0] = max_nan(m[0], fabsf(bf16lo(w[r].x)));
    m[1] = max_nan(m[1], fabsf(bf16hi(w[r].x)));
    m[2] = max_nan(m[2], fabsf(bf16lo(w[r].y)));
    m[3] = max_nan(m[3], fabsf(bf16hi(w[r].y)));
    m[4] = max_nan(m[4], fabsf(bf16lo(w[r].z)));
    m[5] = max_nan(m[5], fabsf(bf16hi(w[r].z)));
    m[6] = max_nan(m[6], fabsf(bf16lo(w[r].w)));
    m[7] = max_nan(m[7], fabsf(bf16hi(w[r].w)));
  }
  float4* dst = reinterpret_cast<float4*>(&s_max[warp][lane * 8]);
  dst[0] = make_float4(m[0], m[1], m[2], m[3]);
  dst[1] = make_float4(m[4], m[5], m[6], m[7]);
  __syncthreads();
  float s[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float v = s_max[0][lane * 8 + j];
#pragma unroll
    for (int wv = 1; wv < kColWarps; ++wv) v = max_nan(v, s_max[wv][lane * 8 + j]);
    s[j] = scale_from_amax(v);
  }
  if (!col_ok) return;
  if (warp == 0) {
    float4* sp = reinterpret_cast<float4*>(scales + row_blk * cols + col0);
    sp[0] = make_float4(s[0], s[1], s[2], s[3]);
    sp[1] = make_float4(s[4], s[5], s[6], s[7]);
  }
#pragma unroll
  for (int r = 0; r < kColRowsPerWarp; ++r) {
    const int64_t row = row0 + r;
    if (row >= rows) break;
    const uint4 v = w[r];
    uint32_t b0 = cvt_e4m3x2(__fdiv_rn(bf16lo(v.x), s[0]), __fdiv_rn(bf16hi(v.x), s[1]));
    uint32_t b1 = cvt_e4m3x2(__fdiv_rn(bf16lo(v.y), s[2]), __fdiv_rn(bf16hi(v.y), s[3]));
    uint32_t b2 = cvt_e4m3x2(__fdiv_rn(bf16lo(v.z), s[4]), __fdiv_rn(bf16hi(v.z), s[5]));
    uint32_t b3 = cvt_e4m3x2(__fdiv_rn(bf16lo(v.w), s[6]), __fdiv_rn(bf16hi(v.w), s[7]));
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
  quantize_colwise_kernel<<<dim3(unsigned(gx), unsigned(gy)), kColWarps * 32, 0,
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
