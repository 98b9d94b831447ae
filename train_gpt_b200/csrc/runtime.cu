// Host-side glue shared by the launchers: error text, device checks.
#include <stdio.h>
#include <string.h>

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

}  // namespace tg

extern "C" int tg_version(void) { return 100; }

extern "C" const char* tg_last_cuda_error(void) { return tg::g_err; }
