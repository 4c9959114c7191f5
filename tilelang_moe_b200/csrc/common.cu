// Error reporting and device-attribute cache of the moe_b200 library.
#include "common.cuh"

#include <mutex>

namespace moe {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  snprintf(last_error_buffer(), 512, "CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
  return (int)e > 0 ? (int)e : 1;
}

int current_device_info(DeviceInfo* out) {
  static std::mutex mu;
  static DeviceInfo cache[64];
  static bool have[64] = {false};
  int dev = 0;
  MOE_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(MOE_ERR_DEVICE, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!have[dev]) {
    DeviceInfo d;
    MOE_CUDA_CHECK(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
    MOE_CUDA_CHECK(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    MOE_CUDA_CHECK(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
    MOE_CUDA_CHECK(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    cache[dev] = d;
    have[dev] = true;
  }
  *out = cache[dev];
  if (out->cc_major != 10)
    return fail(MOE_ERR_DEVICE, "moe_b200 needs an sm_100 device, found sm_%d%d", out->cc_major, out->cc_minor);
  return MOE_OK;
}

}  // namespace moe

extern "C" const char* moe_last_error(void) { return moe::last_error_buffer(); }

extern "C" int moe_abi_version(void) { return 1; }

extern "C" int moe_device_info(int device, int* sm_count, int* cc_major, int* cc_minor) {
  if (!sm_count || !cc_major || !cc_minor) return moe::fail(MOE_ERR_ARG, "null output pointer");
  MOE_CUDA_CHECK(cudaDeviceGetAttribute(sm_count, cudaDevAttrMultiProcessorCount, device));
  MOE_CUDA_CHECK(cudaDeviceGetAttribute(cc_major, cudaDevAttrComputeCapabilityMajor, device));
  MOE_CUDA_CHECK(cudaDeviceGetAttribute(cc_minor, cudaDevAttrComputeCapabilityMinor, device));
  return MOE_OK;
}
