// Library-wide pieces of the C ABI: error text, device cache, the reciprocal test helper.
#include "common.cuh"
#include "resinfer_b200.h"

#include <mutex>

namespace ri {

static thread_local char g_error[1024] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
}

int device_info(DeviceInfo* out) {
  constexpr int kMaxDev = 64;
  static DeviceInfo cache[kMaxDev];
  static bool have[kMaxDev] = {};
  static std::mutex mu;
  int dev = 0;
  RI_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDev) {
    set_error("device ordinal %d out of range", dev);
    return RI_ERR_DEVICE;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!have[dev]) {
    DeviceInfo d{};
    d.ordinal = dev;
    RI_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
    RI_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    RI_CUDA(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
    RI_CUDA(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    cache[dev] = d;
    have[dev] = true;
  }
  *out = cache[dev];
  if (out->cc_major != 10) {
    set_error("No compiled kernel for this device: sm_%d%d found, sm_100a (B200) required",
              out->cc_major, out->cc_minor);
    return RI_ERR_DEVICE;
  }
  return RI_OK;
}

namespace {
__global__ void rcp_kernel(const float* in, float* out, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = rcp_approx_ftz(in[i]);
}
}  // namespace
}  // namespace ri

extern "C" int ri_abi_version(void) { return RI_ABI_VERSION; }
extern "C" const char* ri_last_error(void) { return ri::g_error; }

extern "C" int ri_device_info(int* sm_count, int* cc_major, int* cc_minor) {
  ri::DeviceInfo d;
  int s = ri::device_info(&d);
  if (s) return s;
  if (sm_count) *sm_count = d.sm_count;
  if (cc_major) *cc_major = d.cc_major;
  if (cc_minor) *cc_minor = d.cc_minor;
  return 0;
}

extern "C" int ri_rcp_approx(const float* in, float* out, int n, void* stream) {
  if (n <= 0) return 0;
  ri::rcp_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(in, out, n);
  return ri::cuda_status(cudaGetLastError(), "ri_rcp_approx");
}
