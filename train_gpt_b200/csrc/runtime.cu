// Host-side glue shared by the launchers: error text, device checks.
#include <stdio.h>
#include <string.h>

#include <atomic>

#include "common.cuh"

namespace tg {

static thread_local char g_err[512] = "";

int record_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_err, sizeof(g_err), "%s: %s (%s)", where, cudaGetErrorName(e), cudaGetErrorString(e));
  return TG_ERR_CUDA;
}

struct DevInfo {
  int major = -1;
  int sms = 0;
};

static int query(DevInfo* out) {
  // one cached entry per device ordinal; benign race (same values written)
  static DevInfo cache[64];
  int dev = 0;
  TG_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return TG_ERR_SHAPE;
  if (cache[dev].major < 0) {
    int major = 0, sms = 0;
    TG_CUDA_CHECK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    TG_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    cache[dev].sms = sms;
    cache[dev].major = major;
  }
  *out = cache[dev];
  return TG_OK;
}

int check_arch() {
  DevInfo d;
  if (int rc = query(&d)) return rc;
  return d.major == 10 ? TG_OK : TG_ERR_ARCH;
}

int sm_count() {
  DevInfo d;
  if (query(&d) != TG_OK || d.sms <= 0) return 148;
  return d.sms;
}

static std::atomic<int> g_reserved_sms{0};

int gemm_sms() {
  const int n = sm_count() - g_reserved_sms.load(std::memory_order_relaxed);
  return n < 1 ? 1 : n;
}

}  // namespace tg

extern "C" int tg_version(void) { return 101; }

extern "C" int tg_set_gemm_reserved_sms(int n) {
  if (n < 0) n = 0;
  if (n > 64) n = 64;
  return tg::g_reserved_sms.exchange(n, std::memory_order_relaxed);
}

extern "C" const char* tg_last_cuda_error(void) { return tg::g_err; }
