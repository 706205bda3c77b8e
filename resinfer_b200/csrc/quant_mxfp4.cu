// MXFP4 activation quantisers: MEXT (base + full residue in row_pair / tile8 layout) and the
// selective (KEXT) variant.  32-element blocks, E8M0 "ceil" scale, no global scale.
//
// Arithmetic follows ShawRong/ResInfer csrc/mxfp4/cuda/mxfp4_residue_quant.cu:19-29, 55-81,
// 147-258 (explicit round-to-nearest multiplies and subtract, rcp.approx of 6); every thread
// owns one 32-element block (two 256-bit loads, two 128-bit code stores).  The kernel also
// zero-fills what the reference zero-fills: padding scales, padded tile8 rows and the K tail of
// the selective layout.
#include "common.cuh"
#include "resinfer_b200.h"

namespace ri {
namespace {

__device__ __forceinline__ uint8_t e8m0_ceil(float v) {
  return (uint8_t)__nv_cvt_float_to_e8m0(v, __NV_SATFINITE, cudaRoundPosInf);
}
// scale code of a block and the multiplier 2^(127-e) (0 for an all-zero block)
__device__ __forceinline__ uint8_t mx_scale(float amax, float& mult) {
  uint8_t e = e8m0_ceil(__fmul_rn(amax, rcp_approx_ftz(6.0f)));
  mult = e == 0 ? 0.f : __uint_as_float(uint32_t(254 - e) << 23);
  return e;
}
__device__ __forceinline__ uint32_t quant8(const float* v, float mult) {
  float s[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) s[i] = __fmul_rn(v[i], mult);
  return cvt_e2m1x8(s);
}

template <typename T>
__device__ __forceinline__ void load32(const T* p, int64_t col_stride, float (&v)[32]) {
  if (col_stride == 1 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    float a[16], b[16];
    load16(p, a);
    load16(p + 16, b);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      v[i] = a[i];
      v[16 + i] = b[i];
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = float(p[i * col_stride]);
  }
}

// PER8 == 8: MEXT (full residue rows).  PER8 in {1,2,4}: selective residue appended along K.
// PER8 == 0: plain quantisation, no residue.
template <typename T, int PER8>
__global__ void __launch_bounds__(128) mxfp4_quant_kernel(
    const T* __restrict__ x, int64_t row_stride, int64_t col_stride, const uint8_t* __restrict__ masks,
    uint8_t* __restrict__ out, uint8_t* __restrict__ out_sf, int rows, int k, int k_total,
    int out_rows, int padded_rows, int swizzle, int tile8) {
  constexpr bool MEXT = PER8 == 8;
  const int lane = threadIdx.x & 31;
  const int groups_in = k / 32;                                   // base blocks per row
  const int sf_groups = k_total / 32;
  const int sf_groups_out = swizzle ? (sf_groups + 3) / 4 * 4 : sf_groups;
  const int sel = (MEXT || PER8 == 0) ? 0 : k / 8 * PER8;
  const int sel_groups = (sel + 31) / 32;
  // logical rows this grid walks: tokens for MEXT (two physical rows each), rows otherwise
  const int sf_rows = swizzle ? padded_rows : out_rows;
  const int walk_rows = MEXT ? sf_rows / 2 : sf_rows;
  const int groups_walk = sf_groups_out > groups_in ? sf_groups_out : groups_in;
  const int warps_per_row = (groups_walk + 31) / 32;
  const int total_warps = walk_rows * warps_per_row;
  // let the dependent kernel (the GEMM) be scheduled now: it prefetches weights while this grid runs and
  // waits for this grid (griddepcontrol.wait) before it reads the codes
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < total_warps;
       w += (gridDim.x * blockDim.x) >> 5) {
    const int row = w / warps_per_row;
    const int g = (w % warps_per_row) * 32 + lane;                // base block index in the row
    const bool valid = row < rows;
    int base_row = row, res_row = row;
    if (MEXT) {
      if (tile8) {
        base_row = (row / 8) * 16 + (row % 8);
        res_row = base_row + 8;
      } else {
        base_row = 2 * row;
        res_row = 2 * row + 1;
      }
    }
    auto sf_at = [&](int r, int grp) -> uint8_t& {
      return out_sf[swizzle ? sf_offset<32>(r, grp, k_total) : int64_t(r) * sf_groups + grp];
    };
    const bool has = valid && g < groups_in;
    if (!valid) {
      // padding rows: zero scales (and zero codes for padded tile8 rows)
      if (g < sf_groups_out && base_row < sf_rows) {
        sf_at(base_row, g) = 0;
        if (MEXT) sf_at(res_row, g) = 0;
      }
      if (MEXT && tile8 && row < out_rows / 2 && g < groups_in) {
        uint4 z = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(out + int64_t(base_row) * (k_total / 2) + g * 16) = z;
        *reinterpret_cast<uint4*>(out + int64_t(res_row) * (k_total / 2) + g * 16) = z;
      }
      continue;
    }
    float v[32], d[32];
    if (has) {
      load32(x + int64_t(row) * row_stride + int64_t(g) * 32 * col_stride, col_stride, v);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    float mult;
    const uint8_t e = mx_scale(amax, mult);
    const float deq_scale = __uint_as_float(uint32_t(e) << 23);   // 2^(e-127); e == 0 -> codes are 0
    uint4 codes;
    codes.x = quant8(v, mult);
    codes.y = quant8(v + 8, mult);
    codes.z = quant8(v + 16, mult);
    codes.w = quant8(v + 24, mult);
    {
      const uint32_t c[4] = {codes.x, codes.y, codes.z, codes.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float hat[8];
        e2m1x8_to_float(c[j], hat);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          d[8 * j + i] = __fsub_rn(v[8 * j + i], __fmul_rn(hat[i], deq_scale));   // residue
      }
    }
    if (has) {
      *reinterpret_cast<uint4*>(out + int64_t(base_row) * (k_total / 2) + g * 16) = codes;
      sf_at(base_row, g) = e;
    }
    if constexpr (MEXT) {
      float rmax = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) rmax = fmaxf(rmax, fabsf(d[i]));
      float rmult;
      const uint8_t er = mx_scale(rmax, rmult);
      if (has) {
        uint4 rc;
        rc.x = quant8(d, rmult);
        rc.y = quant8(d + 8, rmult);
        rc.z = quant8(d + 16, rmult);
        rc.w = quant8(d + 24, rmult);
        *reinterpret_cast<uint4*>(out + int64_t(res_row) * (k_total / 2) + g * 16) = rc;
        sf_at(res_row, g) = er;
      } else if (g < sf_groups_out) {
        sf_at(base_row, g) = 0;
        sf_at(res_row, g) = 0;
      }
    } else if constexpr (PER8 == 0) {
      if (!has && g < sf_groups_out) sf_at(row, g) = 0;
    } else {
      constexpr int NRES = 4 * PER8;              // residues per thread (32 channels = 4 mask bytes)
      constexpr int SF_THREADS = 32 / NRES;       // threads sharing one residue scale
      float selv[NRES];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        uint32_t m = has ? masks[g * 4 + b] : 0u;
#pragma unroll
        for (int j = 0; j < PER8; ++j) {
          int bit = __ffs(m) - 1;
          float val = 0.f;
#pragma unroll
          for (int c = 0; c < 8; ++c)
            if (c == bit) val = d[8 * b + c];
          selv[b * PER8 + j] = val;
          m &= m - 1;
        }
      }
      float rmax = 0.f;
#pragma unroll
      for (int j = 0; j < NRES; ++j) rmax = fmaxf(rmax, fabsf(selv[j]));
#pragma unroll
      for (int off = 1; off < SF_THREADS; off <<= 1)
        rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, off));
      float rmult;
      const uint8_t er = mx_scale(rmax, rmult);
      const int res_start = g * NRES;
      uint8_t* rowp = out + int64_t(row) * (k_total / 2);
      if (has) {
        if ((lane % SF_THREADS) == 0) sf_at(row, groups_in + res_start / 32) = er;
        if constexpr (NRES >= 8) {
#pragma unroll
          for (int j = 0; j < NRES / 8; ++j)
            *reinterpret_cast<uint32_t*>(rowp + k / 2 + res_start / 2 + 4 * j) = quant8(selv + 8 * j, rmult);
        }
      }
      if constexpr (NRES == 4) {                  // two threads fill one 32-bit word
        float s0 = __fmul_rn(selv[0], rmult), s1 = __fmul_rn(selv[1], rmult);
        float s2 = __fmul_rn(selv[2], rmult), s3 = __fmul_rn(selv[3], rmult);
        uint32_t word = (cvt_e2m1x2(s0, s1) | (cvt_e2m1x2(s2, s3) << 8)) << (16 * (lane & 1));
        word |= __shfl_xor_sync(0xffffffffu, word, 1);
        if (has && (lane & 1) == 0) *reinterpret_cast<uint32_t*>(rowp + k / 2 + res_start / 2) = word;
      }
      // scales of padding groups and the zero tail of the row
      if (!has && g < sf_groups_out && g >= groups_in + sel_groups) sf_at(row, g) = 0;
      {
        // bytes [k/2 + ceil(sel/8)*4, k_total/2) are zero; spread them over the row's threads
        const int tail_begin = k / 2 + (sel + 7) / 8 * 4;
        const int tail_bytes = k_total / 2 - tail_begin;
        for (int j = g; j < tail_bytes; j += warps_per_row * 32) rowp[tail_begin + j] = 0;
      }
    }
  }
}

template <typename T, int PER8>
int launch_mx(cudaStream_t st, int pdl, const T* x, int64_t rs, int64_t cs, const uint8_t* masks,
              uint8_t* out, uint8_t* sf, int rows, int k, int k_total, int out_rows, int padded_rows,
              int swizzle, int tile8) {
  DeviceInfo di;
  int s = device_info(&di);
  if (s) return s;
  const int sf_groups = k_total / 32;
  const int sf_groups_out = swizzle ? (sf_groups + 3) / 4 * 4 : sf_groups;
  const int groups_walk = sf_groups_out > k / 32 ? sf_groups_out : k / 32;
  const int sf_rows = swizzle ? padded_rows : out_rows;
  const int walk_rows = PER8 == 8 ? sf_rows / 2 : sf_rows;
  int64_t warps = int64_t(walk_rows) * ((groups_walk + 31) / 32);
  int64_t blocks = (warps + 3) / 4;
  int64_t cap = int64_t(di.sm_count) * 64;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(128);
  cfg.stream = st;
  cudaLaunchAttribute attr{};
  if (pdl) {
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  return cuda_status(cudaLaunchKernelEx(&cfg, mxfp4_quant_kernel<T, PER8>, x, rs, cs, masks, out, sf, rows,
                                        k, k_total, out_rows, padded_rows, swizzle, tile8),
                     "mxfp4 quantiser launch");
}

template <typename T>
int dispatch_mx(int per8, bool has_masks, cudaStream_t st, int pdl, const T* x, int64_t rs, int64_t cs,
                const uint8_t* masks, uint8_t* out, uint8_t* sf, int rows, int k, int k_total,
                int out_rows, int padded_rows, int swizzle, int tile8) {
  if (!has_masks && per8 == 0 && out_rows == rows && !tile8)
    return launch_mx<T, 0>(st, pdl, x, rs, cs, masks, out, sf, rows, k, k_total, out_rows, padded_rows, swizzle, tile8);
  if (!has_masks) return launch_mx<T, 8>(st, pdl, x, rs, cs, masks, out, sf, rows, k, k_total, out_rows, padded_rows, swizzle, tile8);
  switch (per8) {
    case 1: return launch_mx<T, 1>(st, pdl, x, rs, cs, masks, out, sf, rows, k, k_total, out_rows, padded_rows, swizzle, tile8);
    case 2: return launch_mx<T, 2>(st, pdl, x, rs, cs, masks, out, sf, rows, k, k_total, out_rows, padded_rows, swizzle, tile8);
    default: return launch_mx<T, 4>(st, pdl, x, rs, cs, masks, out, sf, rows, k, k_total, out_rows, padded_rows, swizzle, tile8);
  }
}

}  // namespace
}  // namespace ri

using namespace ri;

extern "C" int ri_mxfp4_quant(const void* x, int dtype, int m, int k, int64_t row_stride,
                              int64_t col_stride, const uint8_t* masks, int per8, uint8_t* codes,
                              int out_rows, int out_row_bytes, uint8_t* sf, int64_t sf_bytes,
                              int swizzle, int tile8, int pdl_mode, void* stream) {
  RI_CHECK_ARG(pdl_mode >= 0 && pdl_mode <= 2, "pdl_mode must be 0/off, 1/tail or 2/early");
  RI_CHECK_ARG(dtype == RI_DTYPE_BF16 || dtype == RI_DTYPE_FP16, "fp16/bf16 required");
  RI_CHECK_ARG(k > 0 && k % 32 == 0, "invalid MXFP4 extent");
  RI_CHECK_ARG(!masks || per8 == 1 || per8 == 2 || per8 == 4, "per8 must be 1/2/4");
  RI_CHECK_ARG(!tile8 || (!masks && swizzle), "tile8 requires full residue and 128x4 scales");
  const int sel = masks ? k / 8 * per8 : 0;
  const bool plain = !masks && per8 == 0 && out_rows == m && !tile8 && m > 0;
  RI_CHECK_ARG(plain || (tile8 ? (out_rows >= 2 * m && out_rows % 16 == 0) : out_rows == m * (masks ? 1 : 2)),
               "invalid output rows");
  const int k_total = out_row_bytes * 2;
  RI_CHECK_ARG(k_total % 32 == 0 && (masks ? k_total >= k + sel : k_total == k), "invalid output K");
  const int64_t need = swizzle ? int64_t((out_rows + 127) / 128) * ((k_total + 127) / 128) * 512
                               : int64_t(out_rows) * (k_total / 32);
  RI_CHECK_ARG(sf_bytes == need, "invalid SF extent");
  RI_CHECK_ARG((reinterpret_cast<uintptr_t>(codes) & 15) == 0 && out_row_bytes % 16 == 0,
               "packed output rows must be 16-byte aligned");
  if (m == 0) return RI_OK;
  const int padded_rows = swizzle ? (out_rows + 127) / 128 * 128 : out_rows;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == RI_DTYPE_BF16)
    return dispatch_mx(per8, masks != nullptr, st, pdl_mode != 0, static_cast<const __nv_bfloat16*>(x),
                       row_stride, col_stride, masks, codes, sf, m, k, k_total, out_rows, padded_rows, swizzle, tile8);
  return dispatch_mx(per8, masks != nullptr, st, pdl_mode != 0, static_cast<const __half*>(x), row_stride,
                     col_stride, masks, codes, sf, m, k, k_total, out_rows, padded_rows, swizzle, tile8);
}
