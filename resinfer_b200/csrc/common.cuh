// Shared device/host helpers of libresinfer_b200 (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

// ------------------------------------------------------------------------------------------
// error reporting of the C ABI: 0 = ok, < 0 = rejected arguments, > 0 = cudaError_t
// ------------------------------------------------------------------------------------------
namespace ri {

enum : int {
  RI_OK = 0,
  RI_ERR_ARG = -1,        // bad shape / dtype / alignment / size
  RI_ERR_UNSUPPORTED = -2,
  RI_ERR_DEVICE = -3,     // not an sm_100 device
  RI_ERR_TIMEOUT = -4,    // a bounded device-side wait gave up (status word set by the kernel)
};

void set_error(const char* fmt, ...);   // defined in api.cu; message is thread local

inline int fail_arg(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
inline int fail_arg(const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  set_error("%s", buf);
  return RI_ERR_ARG;
}

inline int cuda_status(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return RI_OK;
  set_error("%s: %s", what, cudaGetErrorString(e));
  return (int)e;
}

#define RI_CHECK_ARG(cond, ...) \
  do {                          \
    if (!(cond)) return ::ri::fail_arg(__VA_ARGS__); \
  } while (0)

#define RI_CUDA(expr)                                        \
  do {                                                       \
    int _s = ::ri::cuda_status((expr), #expr);               \
    if (_s != 0) return _s;                                  \
  } while (0)

struct DeviceInfo {
  int ordinal;                 // device the calling thread has current
  int sm_count;
  int cc_major, cc_minor;
  int max_smem_optin;
};
// Cached per device ordinal (the reference caches the first device's value only).
int device_info(DeviceInfo* out);
// how long a kernel waits for another rank before it gives up (ri_peer_allreduce_set_wait_ms)
long long peer_wait_ns();

// ------------------------------------------------------------------------------------------
// device arithmetic that must match the reference build (-O3 --use_fast_math): flush-to-zero
// multiplies, one fused multiply-add for the residue, rcp.approx.ftz reciprocals
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float rcp_approx_ftz(float a) {
  float b;
  asm volatile("rcp.approx.ftz.f32 %0, %1;" : "=f"(b) : "f"(a));
  return b;
}
__device__ __forceinline__ float mul_ftz(float a, float b) {
  float c;
  asm("mul.rn.ftz.f32 %0, %1, %2;" : "=f"(c) : "f"(a), "f"(b));
  return c;
}
// x - hat * inv with a single rounding
__device__ __forceinline__ float residue_fma(float x, float hat, float inv) {
  float c;
  asm("fma.rn.ftz.f32 %0, %1, %2, %3;" : "=f"(c) : "f"(-hat), "f"(inv), "f"(x));
  return c;
}

// two floats -> one byte of E2M1 codes: `lo` in the low nibble, `hi` in the high nibble
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
  uint32_t r;
  asm("{\n\t.reg .b8 b;\n\tcvt.rn.satfinite.e2m1x2.f32 b, %2, %1;\n\tcvt.u32.u8 %0, b;\n\t}"
      : "=r"(r) : "f"(lo), "f"(hi));
  return r;
}
// 8 floats -> 8 packed codes, element i in nibble i
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float (&v)[8]) {
  uint32_t r;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(r)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  return r;
}
// one byte of codes -> two floats (exact)
__device__ __forceinline__ float2 e2m1x2_to_float2(uint32_t byte) {
  uint32_t h2;
  asm("{\n\t.reg .b8 b;\n\tcvt.u8.u32 b, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b;\n\t}" : "=r"(h2) : "r"(byte));
  __half2 h = *reinterpret_cast<__half2*>(&h2);
  return __half22float2(h);
}
__device__ __forceinline__ __half2 e2m1x2_to_half2(uint32_t byte) {
  uint32_t h2;
  asm("{\n\t.reg .b8 b;\n\tcvt.u8.u32 b, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b;\n\t}" : "=r"(h2) : "r"(byte));
  return *reinterpret_cast<__half2*>(&h2);
}
// 8 packed codes -> 8 floats
__device__ __forceinline__ void e2m1x8_to_float(uint32_t packed, float (&out)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = e2m1x2_to_float2((packed >> (8 * i)) & 0xFFu);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

// E4M3 block scale: byte and its value (round-to-nearest-even, saturating)
__device__ __forceinline__ float encode_e4m3(float v, uint8_t* byte) {
  __nv_fp8_e4m3 t = __nv_fp8_e4m3(v);
  *byte = *reinterpret_cast<uint8_t*>(&t);
  return float(t);
}
__device__ __forceinline__ float decode_e4m3(uint8_t b) {
  __nv_fp8_e4m3 t;
  *reinterpret_cast<uint8_t*>(&t) = b;
  return float(t);
}

// NVFP4 block scale from the block's absolute maximum: SF = e4m3(gs * (amax * rcp(6))),
// multiplier = gs * rcp(SF) (0 for an all-zero block)
__device__ __forceinline__ float nvfp4_scale(float amax, float gs, uint8_t* sf_byte) {
  float sf = mul_ftz(gs, mul_ftz(amax, rcp_approx_ftz(6.0f)));
  float sfv = encode_e4m3(sf, sf_byte);
  return sfv != 0.0f ? mul_ftz(gs, rcp_approx_ftz(sfv)) : 0.0f;
}

// byte offset of the scale of (row m, k-group kg) in the 128x4-swizzled scale buffer
template <int VEC>
__host__ __device__ __forceinline__ int64_t sf_offset(int m, int kg, int k_total) {
  int k_tiles = (k_total + 4 * VEC - 1) / (4 * VEC);
  return int64_t(m / 128) * (int64_t(k_tiles) * 512) + int64_t(kg / 4) * 512 + (m % 32) * 16 +
         ((m % 128) / 32) * 4 + (kg % 4);
}
__host__ __device__ __forceinline__ int64_t sf_offset_rt(int m, int kg, int k_total, int vec) {
  int k_tiles = (k_total + 4 * vec - 1) / (4 * vec);
  return int64_t(m / 128) * (int64_t(k_tiles) * 512) + int64_t(kg / 4) * 512 + (m % 32) * 16 +
         ((m % 128) / 32) * 4 + (kg % 4);
}

// 16 consecutive 16-bit inputs (32 bytes) -> float; 256-bit load when the address allows
template <typename T>
__device__ __forceinline__ void load16(const T* p, float (&v)[16]) {
  uint32_t u[8];
  if ((reinterpret_cast<uintptr_t>(p) & 31) == 0) {
    asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7])
                 : "l"(p));
  } else {
    uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
    uint4 b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
    u[0] = a.x; u[1] = a.y; u[2] = a.z; u[3] = a.w;
    u[4] = b.x; u[5] = b.y; u[6] = b.z; u[7] = b.w;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if constexpr (sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) {
      v[2 * i] = __uint_as_float(u[i] << 16);
      v[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
    } else {
      float2 f = __half22float2(*reinterpret_cast<__half2*>(&u[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
}


// ------------------------------------------------------------------------------------------
// NVFP4 block quantisation shared by the quantiser kernels and the ResAttn query prologue
// ------------------------------------------------------------------------------------------
struct BlockQ {
  uint2 base;       // 16 base codes
  uint2 res;        // 16 residue codes (MEXT)
  uint8_t sf, sf_res;
};

// Base quantisation of one 16-block; leaves the FP32 residues x - deq(q(x)) in r[].
__device__ __forceinline__ uint2 quant_base16(const float (&x)[16], float gs, uint8_t* sf, float (&r)[16]) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));
  float mult = nvfp4_scale(amax, gs, sf);
  float s[8];
  uint2 out;
#pragma unroll
  for (int i = 0; i < 8; ++i) s[i] = mul_ftz(x[i], mult);
  out.x = cvt_e2m1x8(s);
#pragma unroll
  for (int i = 0; i < 8; ++i) s[i] = mul_ftz(x[8 + i], mult);
  out.y = cvt_e2m1x8(s);
  float inv = mult != 0.0f ? rcp_approx_ftz(mult) : 0.0f;
  float hat[8];
  e2m1x8_to_float(out.x, hat);
#pragma unroll
  for (int i = 0; i < 8; ++i) r[i] = residue_fma(x[i], hat[i], inv);
  e2m1x8_to_float(out.y, hat);
#pragma unroll
  for (int i = 0; i < 8; ++i) r[8 + i] = residue_fma(x[8 + i], hat[i], inv);
  return out;
}

__device__ __forceinline__ uint2 quant_plain16(const float (&r)[16], float mult) {
  float s[8];
  uint2 out;
#pragma unroll
  for (int i = 0; i < 8; ++i) s[i] = mul_ftz(r[i], mult);
  out.x = cvt_e2m1x8(s);
#pragma unroll
  for (int i = 0; i < 8; ++i) s[i] = mul_ftz(r[8 + i], mult);
  out.y = cvt_e2m1x8(s);
  return out;
}

__device__ __forceinline__ BlockQ quant_mext16(const float (&x)[16], float gs, float gs_res) {
  BlockQ q;
  float r[16];
  q.base = quant_base16(x, gs, &q.sf, r);
  float ramax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) ramax = fmaxf(ramax, fabsf(r[i]));
  float rmult = nvfp4_scale(ramax, gs_res, &q.sf_res);
  q.res = quant_plain16(r, rmult);
  return q;
}


// ------------------------------------------------------------------------------------------
// mbarrier / bulk-copy helpers.  Every wait is bounded: it gives up after kWaitLimitCycles (or as
// soon as another role of the CTA has given up) and reports that to the caller.
// ------------------------------------------------------------------------------------------
constexpr long long kWaitLimitCycles = 4000000000ll;   // about 2 s at 2 GHz
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// try_wait with a suspend-time hint: the thread may sleep in hardware for up to `hint_ns` and is woken
// when the phase completes, so a waiting warp does not burn issue slots that working warps need
__device__ __forceinline__ bool mbar_try_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity), "r"(hint_ns) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when another role aborted or the cycle limit expired (then sets
// the abort flag itself).  The fast path is one try_wait; after that the thread sleeps in hardware
// between polls; the SM cycle counter and the abort flag are looked at every 64 failed polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int site = 1) {
  if (mbar_try(bar, parity)) return true;
  long long t0 = 0;
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_hint(bar, parity, 20000u)) return true;
    if ((spin & 63u) == 0) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitLimitCycles) {
        *abort_flag = site;                     // which wait gave up (reported in the status word)
        return false;
      }
    }
  }
}

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}


}  // namespace ri
