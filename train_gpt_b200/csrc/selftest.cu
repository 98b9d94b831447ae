// Exhaustive device self-test of the quantisers' division shortcut (see QuantDiv in
// common.cuh): for EVERY finite bf16 amax >= 0 and EVERY bf16 x with |x| <= amax, the byte
// produced by the shortcut must equal RNE_e4m3(div.rn.f32(x, s)) with s = max(amax/448, 1e-30).
// 2^31 pairs; a few milliseconds on a B200.
#include "common.cuh"
#include "mbarrier.cuh"

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

// ---- the give-up path of the GEMM's bounded waits -------------------------------------------
// Four warps stand in for the GEMM's roles, with the same helpers and the same teardown:
//   warp 0  owns a TMEM allocation (as the MMA issuer does) and waits, with the SHORT limit, on a
//           barrier that nobody ever arrives at: the wait must run out, raise the CTA's abort flag
//           and store its role code in *status;
//   warp 1  waits on another such barrier with a limit 64 times longer: it must come back early
//           because it sees the abort flag, not because its own limit ran out;
//   warp 2  waits on a barrier that warp 3 does arrive at: an ordinary wait still succeeds.
// All four then meet at the common teardown and TMEM is freed.  Nothing here traps or spins without
// a bound: the longest possible wait is 64 x limit_cycles, and the host caps limit_cycles.
__global__ void __launch_bounds__(128)
selftest_bounded_wait_kernel(unsigned* status, unsigned* report, long long limit_cycles) {
  __shared__ __align__(8) uint64_t bars[3];
  __shared__ uint32_t tmem_ptr;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 3; ++i) mbar_init(smem_u32(&bars[i]), 1);
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_ptr), 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_ptr);
  const long long t0 = clock64();
  if (warp == 0) {
    const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars[0]), 0u, abort_flag, status, 5u, limit_cycles));
    if (lane == 0) report[0] = ok ? 1u : 0u;                       // expected 0: gave up
  } else if (warp == 1) {
    const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars[1]), 0u, abort_flag, status, 3u, 64 * limit_cycles));
    const long long waited = clock64() - t0;
    if (lane == 0) report[1] = (ok ? 1u : 0u) | (waited < 8 * limit_cycles ? 2u : 0u);   // expected 2: false, and early
  } else if (warp == 2) {
    const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars[2]), 0u, abort_flag, status, 2u, 64 * limit_cycles));
    if (lane == 0) report[2] = ok ? 1u : 0u;                       // expected 1
  } else {
    if (lane == 0) mbar_arrive(smem_u32(&bars[2]));
  }
  // the GEMM's teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 32);
    if (lane == 0) report[3] = 1u;                                 // teardown reached, TMEM freed
  }
}

}  // namespace tg

extern "C" int tg_selftest_bounded_wait(uint32_t* status, uint32_t* report, int64_t limit_cycles, void* stream) {
  if (status == nullptr || report == nullptr) return TG_ERR_SHAPE;
  if (limit_cycles < 1000 || limit_cycles > 50000000) return TG_ERR_SHAPE;   // at most ~25 ms per wait, 64 x that in all
  if (int rc = tg::check_arch()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  TG_CUDA_CHECK(cudaMemsetAsync(status, 0, sizeof(uint32_t), st));
  TG_CUDA_CHECK(cudaMemsetAsync(report, 0xff, 4 * sizeof(uint32_t), st));
  tg::selftest_bounded_wait_kernel<<<1, 128, 0, st>>>(status, report, limit_cycles);
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}

extern "C" int tg_selftest_quantise_division(uint64_t* counts, void* stream) {
  if (counts == nullptr) return TG_ERR_SHAPE;
  if (int rc = tg::check_arch()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  TG_CUDA_CHECK(cudaMemsetAsync(counts, 0, 4 * sizeof(uint64_t), st));
  tg::selftest_division_kernel<<<0x7F80, 256, 0, st>>>(reinterpret_cast<unsigned long long*>(counts));
  TG_CUDA_CHECK(cudaGetLastError());
  return TG_OK;
}
