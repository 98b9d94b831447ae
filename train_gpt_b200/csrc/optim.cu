// Global gradient norm, clip and AdamW for bf16 parameters: the optimiser half of the
// reference's train step (train-gpt train.py:114-123,132-134: optax.chain(clip_by_global_norm,
// adamw) with bf16 parameters, hence bf16 moments).  Bandwidth-bound: the update reads p, g, m,
// v and writes p, m, v once (14 bytes per parameter); the clip factor is applied to the
// gradient on the fly instead of in a pass of its own.
#include "common.cuh"

namespace tg {

constexpr int kOptThreads = 256;
constexpr int kSumsqBlocks = 1024;   // partial sums of tg_sumsq_bf16 (caller scratch: this many floats)

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__global__ void __launch_bounds__(kOptThreads)
sumsq_partial_kernel(const __nv_bfloat16* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float s_w[kOptThreads / 32];
  float acc = 0.f;
  const long long vecs = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < vecs; i += (long long)gridDim.x * blockDim.x) {
    const uint4 w = ld_nc_v4(x + 8 * i);
    const float2 a = bf16x2_unpack(w.x), b = bf16x2_unpack(w.y), c = bf16x2_unpack(w.z), d = bf16x2_unpack(w.w);
    const float2 t = __fadd2_rn(__ffma2_rn(c, c, __fmul2_rn(a, a)), __ffma2_rn(d, d, __fmul2_rn(b, b)));
    acc += t.x + t.y;
  }
  if (blockIdx.x == 0)   // ragged tail (n % 8 elements)
    for (long long i = vecs * 8 + threadIdx.x; i < n; i += blockDim.x) {
      const float f = __bfloat162float(x[i]);
      acc = fmaf(f, f, acc);
    }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = s_w[0];
#pragma unroll
    for (int i = 1; i < kOptThreads / 32; ++i) t += s_w[i];
    partial[blockIdx.x] = t;
  }
}

// out[0] = sum of the partials, in index order (deterministic), by one warp
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int count, float* __restrict__ out) {
  float acc = 0.f;
  for (int i = threadIdx.x; i < count; i += 32) acc += partial[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (threadIdx.x == 0) out[0] = acc;
}

struct AdamwArgs {
  float lr, b1, b2, eps, wd;
};

// One AdamW step on n bf16 parameters.  Rounding points follow optax with bf16 moments: the
// clipped gradient, the stored moments and the stored parameter are bf16 values; everything
// between two stores is float32.
__global__ void __launch_bounds__(kOptThreads)
adamw_kernel(__nv_bfloat16* __restrict__ p, const __nv_bfloat16* __restrict__ g, __nv_bfloat16* __restrict__ m,
             __nv_bfloat16* __restrict__ v, long long n, AdamwArgs a, const int* __restrict__ step,
             const float* __restrict__ gscale) {
  const float t = float(*step);
  const float inv_bc1 = 1.0f / (1.0f - powf(a.b1, t));
  const float inv_bc2 = 1.0f / (1.0f - powf(a.b2, t));
  const float gs = gscale != nullptr ? *gscale : 1.0f;
  const long long vecs = n / 8;
  auto one = [&](float pf, float gf, float& mf, float& vf) {
    const float gc = bf16_round(gf * gs);                               // optax.clip_by_global_norm
    mf = bf16_round(a.b1 * mf + (1.0f - a.b1) * gc);                     // scale_by_adam: mu
    vf = bf16_round(a.b2 * vf + (1.0f - a.b2) * gc * gc);                //                nu
    const float u = (mf * inv_bc1) / (sqrtf(vf * inv_bc2) + a.eps) + a.wd * pf;   // + add_decayed_weights
    return bf16_round(pf - a.lr * u);                                   // apply_updates
  };
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < vecs; i += (long long)gridDim.x * blockDim.x) {
    uint4 pw = *reinterpret_cast<const uint4*>(p + 8 * i);
    const uint4 gw = ld_nc_v4(g + 8 * i);
    uint4 mw = *reinterpret_cast<const uint4*>(m + 8 * i);
    uint4 vw = *reinterpret_cast<const uint4*>(v + 8 * i);
    uint32_t* pp = &pw.x; const uint32_t* gp = &gw.x; uint32_t* mp = &mw.x; uint32_t* vp = &vw.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float m0 = bf16lo(mp[j]), m1 = bf16hi(mp[j]), v0 = bf16lo(vp[j]), v1 = bf16hi(vp[j]);
      const float p0 = one(bf16lo(pp[j]), bf16lo(gp[j]), m0, v0);
      const float p1 = one(bf16hi(pp[j]), bf16hi(gp[j]), m1, v1);
      pp[j] = pack_bf16x2(p0, p1);
      mp[j] = pack_bf16x2(m0, m1);
      vp[j] = pack_bf16x2(v0, v1);
    }
    *reinterpret_cast<uint4*>(p + 8 * i) = pw;
    *reinterpret_cast<uint4*>(m + 8 * i) = mw;
    *reinterpret_cast<uint4*>(v + 8 * i) = vw;
  }
  if (blockIdx.x == 0)
    for (long long i = vecs * 8 + threadIdx.x; i < n; i += blockDim.x) {
      float mf = __bfloat162float(m[i]), vf = __bfloat162float(v[i]);
      const float pn = one(__bfloat162float(p[i]), __bfloat162float(g[i]), mf, vf);
      p[i] = __float2bfloat16_rn(pn);
      m[i] = __float2bfloat16_rn(mf);
      v[i] = __float2bfloat16_rn(vf);
    }
}

}  // namespace tg

using namespace tg;

extern "C" int64_t tg_sumsq_scratch_bytes(void) { return int64_t(kSumsqBlocks) * int64_t(sizeof(float)); }

extern "C" int tg_sumsq_bf16(const void* x, int64_t n, float* out, void* scratch, void* stream) {
  if (n < 0 || out == nullptr || scratch == nullptr) return TG_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(scratch)) return TG_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int64_t want = (n / 8 + kOptThreads - 1) / kOptThreads;
  const int blocks = int(want < 1 ? 1 : (want > kSumsqBlocks ? kSumsqBlocks : want));
  sumsq_partial_kernel<<<blocks, kOptThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), n, static_cast<float*>(scratch));
  TG_CUDA_CHECK(cudaGetLastError());
  sumsq_final_kernel<<<1, 32, 0, st>>>(static_cast<const float*>(scratch), blocks, out);
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}

extern "C" int tg_adamw_bf16(void* p, const void* g, void* m, void* v, int64_t n, float lr, float b1, float b2,
                             float eps, float weight_decay, const int32_t* step, const float* gscale, void* stream) {
  if (n < 0 || step == nullptr) return TG_ERR_SHAPE;
  if (!(b1 >= 0.f && b1 < 1.f && b2 >= 0.f && b2 < 1.f)) return TG_ERR_SHAPE;
  if (n == 0) return TG_OK;
  if (!aligned16(p) || !aligned16(g) || !aligned16(m) || !aligned16(v)) return TG_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  int64_t want = (n / 8 + kOptThreads - 1) / kOptThreads;
  const int64_t cap = int64_t(sm_count()) * 8;
  const int blocks = int(want < 1 ? 1 : (want > cap ? cap : want));
  const AdamwArgs a = {lr, b1, b2, eps, weight_decay};
  adamw_kernel<<<blocks, kOptThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(p), static_cast<const __nv_bfloat16*>(g), static_cast<__nv_bfloat16*>(m),
      static_cast<__nv_bfloat16*>(v), n, a, step, gscale);
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}
