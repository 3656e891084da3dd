// Error plumbing and device probing behind the C ABI.
#include <cstring>
#include <mutex>

#include "common.h"

namespace hb {

static thread_local char g_err[1024] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int device_info(int device, DeviceInfo* out) {
  static std::mutex mu;
  static DeviceInfo cache[64];
  static bool have[64] = {false};
  std::lock_guard<std::mutex> lock(mu);
  if (device < 0 || device >= 64) return fail(HB_ERR_INVALID_ARG, "device %d out of range", device);
  if (!have[device]) {
    cudaDeviceProp p;
    HB_CUDA_CHECK(cudaGetDeviceProperties(&p, device));
    cache[device].sm_count = p.multiProcessorCount;
    cache[device].cc_major = p.major;
    cache[device].cc_minor = p.minor;
    cache[device].smem_optin = p.sharedMemPerBlockOptin;
    cache[device].l2_bytes = (size_t)p.l2CacheSize;
    have[device] = true;
  }
  *out = cache[device];
  return HB_OK;
}

}  // namespace hb

extern "C" {

const char* hb_last_error(void) { return hb::g_err; }

const char* hb_version(void) { return "libhb 0.1 (sm_100a)"; }

int hb_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

}  // extern "C"
