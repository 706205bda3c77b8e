// ri_fp4_gemm_static_scratch: the block-scaled FP4 GEMM for callers that cannot hand over a workspace.
//
// Who needs this.  ri_fp4_gemm splits the K dimension over CTAs for small batches and merges FP32
// partial tiles through a scratch buffer that the caller allocates.  Some callers have no way to do
// that: a serving engine that gave every free byte of device memory to its page pool at start-up
// (a later cudaMalloc can fail, or stall the whole device while it synchronises), a host runtime
// whose allocator is not reachable from the language binding that calls this library, or a code
// path that is forbidden from calling the CUDA allocator at all.  For them the scratch lives in a
// fixed array inside this library's device image, so the call needs only the operand and output
// pointers.
//
// What it costs.  The array is a single per-device buffer of RI_STATIC_SCRATCH_BYTES bytes that
// every call on that device shares:
//   * problem sizes whose plan needs more scratch than that are rejected with RI_ERR_ARG and a
//     message naming both sizes; nothing is launched in that case;
//   * two calls that overlap in time on one device (different streams, or different host threads
//     on the same stream without ordering) write the same partial tiles and tickets and corrupt
//     each other's results.  Calls must be ordered one after the other, e.g. on one stream;
//   * the array keeps whatever the previous call left.  The partial tiles are always written before
//     they are read, and the ticket counters, which must start at zero, are cleared on the caller's
//     stream at the start of every call.
//
// Set-up.  The first call on each device resolves the array's device address (the array's name is
// not an address the host can use) and caches it; that first call must be made with the device
// current that owns `stream`, and should come before any stream capture begins.  Later calls do
// no set-up.  No call allocates or frees memory.
#include <cuda_runtime.h>

#include <mutex>

#include "common.cuh"
#include "../../include/resinfer_b200.h"

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[RI_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// Device address of the array on the current device; looked up once per device.
int scratch_for_current_device(void** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return ri::cuda_status(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) {
    ri::set_error("device ordinal %d outside the supported range [0, %d)", dev, kMaxDevices);
    return RI_ERR_ARG;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return ri::cuda_status(e, "cudaGetSymbolAddress(static scratch)");
    if (p == nullptr || (reinterpret_cast<uintptr_t>(p) & 255) != 0) {
      ri::set_error("static scratch resolved to an unusable address %p", p);
      return RI_ERR_DEVICE;
    }
    g_scratch_ptr[dev] = p;
  }
  *ptr = g_scratch_ptr[dev];
  return ri::RI_OK;
}

}  // namespace

extern "C" int ri_fp4_gemm_static_scratch(const uint8_t* act, int64_t act_row_bytes, const uint8_t* act_sf,
                                          int64_t act_sf_bytes, const uint8_t* w, int64_t w_row_bytes,
                                          const uint8_t* w_sf, int64_t w_sf_bytes, const float* alpha,
                                          int n_alpha, void* out, int out_dtype, int64_t out_row_stride,
                                          int m, int n, int k, int fmt, int layout, int splits,
                                          int32_t* status, int enable_pdl, void* stream) {
  RI_CHECK_ARG(m >= 0 && n > 0 && k > 0, "positive dimensions required");
  const int64_t need = ri_fp4_gemm_workspace_bytes(m, n, k, fmt, layout, splits);
  if (need < 0) {
    ri::set_error("no tile plan for M=%d N=%d K=%d", m, n, k);
    return RI_ERR_ARG;
  }
  RI_CHECK_ARG(need <= int64_t(RI_STATIC_SCRATCH_BYTES),
               "M=%d N=%d K=%d needs %lld bytes of scratch but the built-in array holds %lld; "
               "use ri_fp4_gemm with a caller-allocated workspace",
               m, n, k, (long long)need, (long long)RI_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  int s = scratch_for_current_device(&scratch);
  if (s) return s;
  if (m > 0 && splits != 1) {
    // tickets must read zero when the kernel starts; the previous call may have been cut short.  (Cleared
    // whenever the launch may choose a K-split plan, whatever the size query above planned.)
    const int64_t counters = ri_fp4_gemm_counter_bytes(m, n);
    cudaError_t e = cudaMemsetAsync(scratch, 0, size_t(counters), static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return ri::cuda_status(e, "clearing the static scratch tickets");
  }
  return ri_fp4_gemm(act, act_row_bytes, act_sf, act_sf_bytes, w, w_row_bytes, w_sf, w_sf_bytes, alpha, n_alpha,
                     out, out_dtype, out_row_stride, m, n, k, fmt, layout, splits, scratch,
                     int64_t(RI_STATIC_SCRATCH_BYTES), status, enable_pdl, stream);
}
