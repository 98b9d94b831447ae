// Exhaustive device self-test of the quantisers' division shortcut (see QuantDiv in
// common.cuh): for EVERY finite bf16 amax >= 0 and EVERY bf16 x with |x| <= amax, the byte
// produced by the shortcut must equal RNE_e4m3(div.rn.f32(x, s)) with s = max(amax/448, 1e-30).
// 2^31 pairs; a few milliseconds on a B200.
#include "common.cuh"

namespace tg {

__global__ void __launch_bounds__(256)
selftest_division_kernel(unsigned long long* __restrict__ counts) {
  // blockIdx.x = amax bit pattern (0 .. 0x7F7F), threads sweep all 65536 x patterns
  const uint32_t amax_bits = blockIdx.x;
  const float amax = __uint_as_float(amax_bits << 16);
  const float s = scale_from_amax(amax);
  const QuantDiv d(s);
  unsigned int bad1 = 0, bad2 = 0, bad3 = 0, n = 0;
  for (uint32_t xb = threadIdx.x; xb < 65536u; xb += blockDim.x) {
    const float x = __uint_as_float(xb << 16);
    if (!(fabsf(x) <= amax)) continue;  // also drops NaN
    const uint32_t ref = cvt_e4m3x2(__fdiv_rn(x, s), 0.f) & 0xffu;
    bad1 += (cvt_e4m3x2(d.div<1>(x), 0.f) & 0xffu) != ref;
    bad2 += (cvt_e4m3x2(d.div<2>(x), 0.f) & 0xffu) != ref;
    // the packed two-at-a-time form the kernels use: both halves must give the same byte
    bad2 += quantize2_sr(xb | (xb << 16), make_float2(s, s), make_float2(-d.r, -d.r)) != (ref | (ref << 8));
    bad3 += (cvt_e4m3x2(d.div<3>(x), 0.f) & 0xffu) != ref;
    ++n;
  }
  if (bad1) atomicAdd(&counts[1], (unsigned long long)bad1);
  if (bad2) atomicAdd(&counts[2], (unsigned long long)bad2);
  if (bad3) atomicAdd(&counts[3], (unsigned long long)bad3);
  atomicAdd(&counts[0], (unsigned long long)n);
}

}  // namespace tg

extern "C" int tg_selftest_quantise_division(uint64_t* counts, void* stream) {
  if (counts == nullptr) return TG_ERR_SHAPE;
  if (int rc = tg::check_arch()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  TG_CUDA_CHECK(cudaMemsetAsync(counts, 0, 4 * sizeof(uint64_t), st));
  tg::selftest_division_kernel<<<0x7F80, 256, 0, st>>>(reinterpret_cast<unsigned long long*>(counts));
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}
