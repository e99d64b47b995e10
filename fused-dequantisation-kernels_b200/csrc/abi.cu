// Status plumbing and device queries of libfdk_b200.
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "fdk_common.cuh"

namespace fdk {

namespace {
thread_local char g_detail[512] = "";
}

void set_error_detail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_detail, sizeof(g_detail), fmt, ap);
  va_end(ap);
}

int cuda_status(cudaError_t e, const char* what) {
  set_error_detail("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
  return FDK_ERR_CUDA;
}

int device_info(DeviceInfo* out) {
  constexpr int kMaxDevices = 64;
  static DeviceInfo cache[kMaxDevices];
  static bool have[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  FDK_CUDA(cudaGetDevice(&dev));
  FDK_CHECK_ARG(dev >= 0 && dev < kMaxDevices, FDK_ERR_BAD_ARG, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!have[dev]) {
    DeviceInfo d{};
    FDK_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
    FDK_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    FDK_CUDA(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
    FDK_CUDA(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    cache[dev] = d;
    have[dev] = true;
  }
  *out = cache[dev];
  return FDK_OK;
}

}  // namespace fdk

extern "C" int fdk_version(void) { return 100; /* 0.1.0 */ }

extern "C" const char* fdk_status_string(int status) {
  switch (status) {
    case FDK_OK: return "ok";
    case FDK_ERR_BAD_ARG: return "bad argument";
    case FDK_ERR_SHAPE: return "unsupported shape";
    case FDK_ERR_ALIGN: return "misaligned pointer";
    case FDK_ERR_ARCH: return "device is not sm_100";
    case FDK_ERR_CUDA: return "CUDA runtime error";
    case FDK_ERR_WORKSPACE: return "workspace missing or too small";
    default: return "unknown status";
  }
}

extern "C" const char* fdk_last_error_detail(void) { return fdk::g_detail; }
