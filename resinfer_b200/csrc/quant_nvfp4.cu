// NVFP4 activation quantisers: MEXT (base + full residue, five layouts), KEXT (base + masked
// residue) and the grouped query quantiser of ResAttn.
//
// HBM-bound streaming kernels: every thread owns one 16-element scale block, reads it with one
// 256-bit load and writes two 64-bit code words and its scale bytes.  The arithmetic follows the
// reference operation by operation (ShawRong/ResInfer csrc/common/fp4/nvfp4_utils.cuh:402-429,
// 467-556, 895-1019) so that codes and scales are bit-identical; the thread/block decomposition
// is this library's own.
#include "common.cuh"
#include "resinfer_b200.h"

namespace ri {
namespace {

// token row -> physical rows of the layout (0 concat, 1 row_pair, 2 tile8, 4 attn_tile8);
// reference: nvfp4_utils.cuh:1109-1160
__device__ __forceinline__ void mext_rows(int i, int rows, int layout, int& base, int& res, int& sfb,
                                          int& sfr) {
  if (layout == 2 || layout == 4) {
    base = (i / 8) * 16 + (i % 8);
    res = base + 8;
    if (layout == 4) {
      sfb = (i / 8) * 128 + (i % 8);
      sfr = sfb + 8;
    } else {
      sfb = base;
      sfr = res;
    }
  } else if (layout == 1) {
    base = sfb = 2 * i;
    res = sfr = 2 * i + 1;
  } else {
    base = sfb = i;
    res = sfr = i + rows;
  }
}

// ---------------------------------------------------------------------------------------------
// MEXT: x[M,K] -> base and residue codes + scales.  A thread owns BPT consecutive 16-element blocks of
// one row: BPT = 1 for decode-sized inputs (as many threads as there are blocks, spread over several
// CTAs), BPT = 2 for large inputs (two 256-bit loads in flight per thread, 128-bit code stores, 16-bit
// scale stores).  The grid is (block columns of a row, rows): no index divisions in the kernel.
// ---------------------------------------------------------------------------------------------
template <typename T, int BPT>
__global__ void __launch_bounds__(256) nvfp4_mext_kernel(const T* __restrict__ x, int64_t row_stride,
                                                         int in_rows, int out_rows, int k,
                                                         const float* __restrict__ gs_inv, int n_gs,
                                                         uint8_t* __restrict__ codes,
                                                         uint8_t* __restrict__ sf, int layout) {
  const int blocks_per_row = k / 16;
  const int blk = (blockIdx.x * blockDim.x + threadIdx.x) * BPT;      // first block of this thread
  // let the dependent kernel (the GEMM) be scheduled now: it prefetches weights while this grid runs and
  // waits for this grid (griddepcontrol.wait) before it reads the codes
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");   // inputs may come from a kernel still running
  const bool active = blk < blocks_per_row;
  // BPT = 1: four neighbouring lanes hold the four scale bytes of one 32-bit word of the 128x4 layout
  // (k-groups 4j .. 4j+3 of a row); when every row has whole groups of four they are gathered with
  // shuffles and stored as one word.  Lanes past the end of the row then stay for the shuffles.
  const bool gather_sf = BPT == 1 && blocks_per_row % 4 == 0 && (reinterpret_cast<uintptr_t>(sf) & 3) == 0;
  if (!active && !gather_sf) return;
  const float gs = gs_inv ? __ldg(gs_inv) : 1.0f;
  const float gs_res = (gs_inv && n_gs > 1) ? __ldg(gs_inv + 1) : gs;
  for (int row = blockIdx.y; row < out_rows; row += gridDim.y) {
    float v[BPT][16];
#pragma unroll
    for (int j = 0; j < BPT; ++j) {
      if (row < in_rows && active) {
        load16(x + int64_t(row) * row_stride + (blk + j) * 16, v[j]);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[j][i] = 0.f;
      }
    }
    BlockQ q[BPT];
#pragma unroll
    for (int j = 0; j < BPT; ++j) q[j] = quant_mext16(v[j], gs, gs_res);
    // destinations of the base and residue halves: code rows (bytes) and scale (row, first k-group)
    uint8_t* base_codes;
    uint8_t* res_codes = nullptr;
    int sb, sr = 0, kg_res = blk, k_sf = k;
    if (layout == 5) {          // base codes only (plain NVFP4 activation quantisation)
      base_codes = codes + int64_t(row) * (k / 2);
      sb = row;
    } else if (layout == 3) {   // concat_k: [M, 2K] elements, scales over Ktot = 2K
      base_codes = codes + int64_t(row) * k;
      res_codes = base_codes + k / 2;
      sb = sr = row;
      kg_res = blocks_per_row + blk;
      k_sf = 2 * k;
    } else {
      int br, rr;
      mext_rows(row, out_rows, layout, br, rr, sb, sr);
      base_codes = codes + int64_t(br) * (k / 2);
      res_codes = codes + int64_t(rr) * (k / 2);
    }
    if constexpr (BPT == 1) {
      if (gather_sf) {
        uint32_t wb = q[0].sf, wr = q[0].sf_res;
        wb |= __shfl_down_sync(0xffffffffu, wb, 1) << 8;
        wr |= __shfl_down_sync(0xffffffffu, wr, 1) << 8;
        wb |= __shfl_down_sync(0xffffffffu, wb, 2) << 16;
        wr |= __shfl_down_sync(0xffffffffu, wr, 2) << 16;
        if (active) {
          *reinterpret_cast<uint2*>(base_codes + blk * 8) = q[0].base;
          if (res_codes) *reinterpret_cast<uint2*>(res_codes + blk * 8) = q[0].res;
          if ((blk & 3) == 0) {
            *reinterpret_cast<uint32_t*>(sf + sf_offset<16>(sb, blk, k_sf)) = wb;
            if (res_codes) *reinterpret_cast<uint32_t*>(sf + sf_offset<16>(sr, kg_res, k_sf)) = wr;
          }
        }
      } else {
        *reinterpret_cast<uint2*>(base_codes + blk * 8) = q[0].base;
        sf[sf_offset<16>(sb, blk, k_sf)] = q[0].sf;
        if (res_codes) {
          *reinterpret_cast<uint2*>(res_codes + blk * 8) = q[0].res;
          sf[sf_offset<16>(sr, kg_res, k_sf)] = q[0].sf_res;
        }
      }
    } else {                    // two adjacent blocks: one 128-bit code store, one 16-bit scale store (blk is even)
      *reinterpret_cast<uint4*>(base_codes + blk * 8) = make_uint4(q[0].base.x, q[0].base.y, q[1].base.x, q[1].base.y);
      *reinterpret_cast<uint16_t*>(sf + sf_offset<16>(sb, blk, k_sf)) = uint16_t(q[0].sf | (uint32_t(q[1].sf) << 8));
      if (res_codes) {
        *reinterpret_cast<uint4*>(res_codes + blk * 8) = make_uint4(q[0].res.x, q[0].res.y, q[1].res.x, q[1].res.y);
        *reinterpret_cast<uint16_t*>(sf + sf_offset<16>(sr, kg_res, k_sf)) = uint16_t(q[0].sf_res | (uint32_t(q[1].sf_res) << 8));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// KEXT: base codes of all K channels + residues of the channels selected by mask[K/8] (exactly
// PER8 bits per byte).  One warp covers 512 consecutive channels of one row; residue j (selected
// channels in increasing order) lands at logical column K + j, one scale per 16 residues.
// ---------------------------------------------------------------------------------------------
template <typename T, int PER8>
__global__ void __launch_bounds__(256) nvfp4_kext_kernel(const T* __restrict__ x, int64_t row_stride,
                                                         int rows, int rows_padded, int k, int n_ext,
                                                         const float* __restrict__ gs_inv,
                                                         const uint8_t* __restrict__ mask,
                                                         uint8_t* __restrict__ codes,
                                                         uint8_t* __restrict__ sf) {
  constexpr int NRES = 2 * PER8;             // residues per thread (16 channels = 2 mask bytes)
  constexpr int SF_THREADS = 16 / NRES;      // threads sharing one residue scale
  constexpr int PACK_THREADS = 8 / NRES > 0 ? 8 / NRES : 1;   // threads filling one 32-bit word
  const int lane = threadIdx.x & 31;
  const int blocks_per_row = k / 16;
  const int warps_per_row = (blocks_per_row + 31) / 32;
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int total_warps = rows_padded * warps_per_row;
  // let the dependent kernel (the GEMM) be scheduled now: it prefetches weights while this grid runs and
  // waits for this grid (griddepcontrol.wait) before it reads the codes
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const float gs = gs_inv ? __ldg(gs_inv) : 1.0f;
  for (int w = warp_global; w < total_warps; w += (gridDim.x * blockDim.x) >> 5) {
    const int row = w / warps_per_row;
    const int blk = (w % warps_per_row) * 32 + lane;
    const bool in_k = blk < blocks_per_row;
    const int res_start = blk * NRES;                       // index of this thread's first residue
    if (row >= rows) {                                      // padded row: scales are zero
      if (in_k) {
        sf[sf_offset<16>(row, blk, n_ext)] = 0;
        if ((lane % SF_THREADS) == 0) sf[sf_offset<16>(row, (k + res_start) / 16, n_ext)] = 0;
      }
      continue;
    }
    float v[16], r[16];
    uint32_t m2 = 0;
    if (in_k) {
      load16(x + int64_t(row) * row_stride + blk * 16, v);
      m2 = uint32_t(mask[blk * 2]) | (uint32_t(mask[blk * 2 + 1]) << 8);
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = 0.f;
    }
    uint8_t sfb;
    uint2 base = quant_base16(v, gs, &sfb, r);
    // pick the selected residues in channel order
    float sel[NRES];
#pragma unroll
    for (int j = 0; j < NRES; ++j) {
      int bit = __ffs(m2) - 1;
      float val = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c)
        if (c == bit) val = r[c];
      sel[j] = val;
      m2 &= m2 - 1;
    }
    float ramax = 0.f;
#pragma unroll
    for (int j = 0; j < NRES; ++j) ramax = fmaxf(ramax, fabsf(sel[j]));
#pragma unroll
    for (int off = 1; off < SF_THREADS; off <<= 1)
      ramax = fmaxf(ramax, __shfl_xor_sync(0xffffffffu, ramax, off));
    uint8_t sfr;
    float rmult = nvfp4_scale(ramax, gs, &sfr);
    // encode this thread's residues (NRES nibbles) and merge to 32-bit words inside the warp
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < NRES; j += 2)
      word |= cvt_e2m1x2(mul_ftz(sel[j], rmult), mul_ftz(sel[j + 1], rmult)) << (4 * j);
    if (PACK_THREADS > 1) {
      word <<= (4 * NRES) * (lane % PACK_THREADS);
#pragma unroll
      for (int off = 1; off < PACK_THREADS; off <<= 1) word |= __shfl_xor_sync(0xffffffffu, word, off);
    }
    if (in_k) {
      uint8_t* rowp = codes + int64_t(row) * (n_ext / 2);
      *reinterpret_cast<uint2*>(rowp + blk * 8) = base;
      sf[sf_offset<16>(row, blk, n_ext)] = sfb;
      if ((lane % PACK_THREADS) == 0)
        *reinterpret_cast<uint32_t*>(rowp + (k + res_start) / 2) = word;
      if ((lane % SF_THREADS) == 0) sf[sf_offset<16>(row, (k + res_start) / 16, n_ext)] = sfr;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// grouped query quantiser: q[B,Hkv,G,D] -> q_pack[B,Hkv,P,D/2] (rows g and P/2+g), scales in a
// private 128-row swizzled tile per (b, hkv); global scale 1.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) nvfp4_grouped_q_kernel(const __nv_bfloat16* __restrict__ q,
                                                              uint8_t* __restrict__ q_pack,
                                                              uint8_t* __restrict__ q_sf, int groups,
                                                              int g, int p, int d) {
  const int blocks_per_row = d / 16;
  const int per_group = g * blocks_per_row;
  const int64_t total = int64_t(groups) * per_group;
  // let the dependent kernel (the GEMM) be scheduled now: it prefetches weights while this grid runs and
  // waits for this grid (griddepcontrol.wait) before it reads the codes
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += int64_t(gridDim.x) * blockDim.x) {
    const int grp = int(t / per_group);
    const int rem = int(t % per_group);
    const int row = rem / blocks_per_row, blk = rem % blocks_per_row;
    float v[16];
    load16(q + (int64_t(grp) * g + row) * d + blk * 16, v);
    BlockQ bq = quant_mext16(v, 1.0f, 1.0f);
    uint8_t* pack = q_pack + int64_t(grp) * p * (d / 2);
    uint8_t* sfp = q_sf + int64_t(grp) * 128 * blocks_per_row;
    *reinterpret_cast<uint2*>(pack + int64_t(row) * (d / 2) + blk * 8) = bq.base;
    *reinterpret_cast<uint2*>(pack + int64_t(p / 2 + row) * (d / 2) + blk * 8) = bq.res;
    sfp[sf_offset<16>(row, blk, d)] = bq.sf;
    sfp[sf_offset<16>(p / 2 + row, blk, d)] = bq.sf_res;
  }
}

template <typename K, typename... Args>
int launch(K kernel, int64_t work_items, int threads, int pdl, cudaStream_t stream, Args... args) {
  DeviceInfo di;
  int s = device_info(&di);
  if (s) return s;
  int64_t blocks = (work_items + threads - 1) / threads;
  int64_t cap = int64_t(di.sm_count) * (2048 / threads) * 4;   // grid-stride beyond a few waves
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(threads);
  cfg.stream = stream;
  cudaLaunchAttribute attr{};
  if (pdl) {
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  return cuda_status(cudaLaunchKernelEx(&cfg, kernel, args...), "quantiser launch");
}

}  // namespace
}  // namespace ri

using namespace ri;

extern "C" int ri_nvfp4_quant_mext(const void* x, int dtype, int m, int k, int64_t row_stride,
                                   const float* gs_inv, int n_gs, uint8_t* codes, int64_t codes_bytes,
                                   uint8_t* sf, int64_t sf_bytes, int layout, int enable_pdl,
                                   void* stream) {
  RI_CHECK_ARG(dtype == RI_DTYPE_BF16 || dtype == RI_DTYPE_FP16, "Unsupported input data type for quantize_to_fp4.");
  RI_CHECK_ARG(m >= 0 && k > 0 && k % 16 == 0, "The N dimension must be multiple of 16.");
  RI_CHECK_ARG(layout >= 0 && layout <= 5, "unknown MEXT layout mode %d", layout);
  RI_CHECK_ARG(n_gs >= 1 && n_gs <= 2, "input_sf must have 1 (single-alpha) or 2 (dual-alpha: [base, residue]) elements.");
  RI_CHECK_ARG(row_stride >= k && (row_stride * 2) % 16 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0,
               "input rows must be 16-byte aligned");
  const bool tile8 = layout == RI_MEXT_TILE8 || layout == RI_MEXT_ATTN_TILE8;
  const int64_t out_m = tile8 ? (int64_t(m) + 7) / 8 * 8 : m;
  RI_CHECK_ARG(codes_bytes >= (layout == RI_MEXT_BASE_ONLY ? out_m * k / 2 : out_m * k),
               "M-extension output tensor is too small for the derived output_m (caller buffer "
               "undersized for the padded row count).");
  int64_t m_tiles, k_tiles;
  if (layout == RI_MEXT_CONCAT_K) {
    m_tiles = (out_m + 127) / 128;
    k_tiles = (2 * int64_t(k) + 63) / 64;
  } else if (layout == RI_MEXT_ATTN_TILE8) {
    m_tiles = out_m / 8;
    k_tiles = (int64_t(k) + 63) / 64;
  } else if (layout == RI_MEXT_BASE_ONLY) {
    m_tiles = (out_m + 127) / 128;
    k_tiles = (int64_t(k) + 63) / 64;
  } else {
    m_tiles = (2 * out_m + 127) / 128;
    k_tiles = (int64_t(k) + 63) / 64;
  }
  RI_CHECK_ARG(sf_bytes >= m_tiles * k_tiles * 512,
               "M-extension output scale tensor is too small for layout mode %d: need %lld bytes, got %lld",
               layout, (long long)(m_tiles * k_tiles * 512), (long long)sf_bytes);
  RI_CHECK_ARG((reinterpret_cast<uintptr_t>(codes) & 7) == 0, "codes buffer must be 8-byte aligned");
  if (m == 0) return RI_OK;
  // Geometry: a thread per 16-element block for small inputs; two blocks per thread once the input fills
  // the machine anyway (needs an even block count per row, 16-byte aligned code rows and even scale groups).
  DeviceInfo di;
  int s = device_info(&di);
  if (s) return s;
  const int blocks_per_row = k / 16;
  const bool wide = blocks_per_row % 2 == 0 && out_m * blocks_per_row >= int64_t(di.sm_count) * 2048 &&
                    (reinterpret_cast<uintptr_t>(codes) & 15) == 0 && (k / 2) % 16 == 0 &&
                    (reinterpret_cast<uintptr_t>(sf) & 1) == 0;
  const int units = wide ? blocks_per_row / 2 : blocks_per_row;          // threads per row
  const int col_blocks = (units + 255) / 256;
  const int threads = ((units + col_blocks - 1) / col_blocks + 31) / 32 * 32;
  int64_t rows_y = out_m;
  const int64_t cap = int64_t(di.sm_count) * (2048 / threads) * 4 / col_blocks;   // a few waves, then rows are looped
  if (rows_y > cap) rows_y = cap < 1 ? 1 : cap;
  if (rows_y > 65535) rows_y = 65535;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)col_blocks, (unsigned)rows_y);
  cfg.blockDim = dim3(threads);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr{};
  if (enable_pdl) {
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  auto go = [&](auto kernel, auto* xp) {
    return cuda_status(cudaLaunchKernelEx(&cfg, kernel, xp, row_stride, m, int(out_m), k, gs_inv, n_gs, codes, sf, layout),
                       "quantiser launch");
  };
  if (dtype == RI_DTYPE_BF16) {
    const auto* xp = static_cast<const __nv_bfloat16*>(x);
    return wide ? go(nvfp4_mext_kernel<__nv_bfloat16, 2>, xp) : go(nvfp4_mext_kernel<__nv_bfloat16, 1>, xp);
  }
  const auto* xp = static_cast<const __half*>(x);
  return wide ? go(nvfp4_mext_kernel<__half, 2>, xp) : go(nvfp4_mext_kernel<__half, 1>, xp);
}

template <typename T>
static int launch_kext(int per8, int64_t work, cudaStream_t st, const T* x, int64_t row_stride, int m,
                       int rows_padded, int k, int n_ext, const float* gs_inv, const uint8_t* mask,
                       uint8_t* codes, uint8_t* sf) {
  switch (per8) {
    case 1: return launch(nvfp4_kext_kernel<T, 1>, work, 256, 1, st, x, row_stride, m, rows_padded, k, n_ext, gs_inv, mask, codes, sf);
    case 2: return launch(nvfp4_kext_kernel<T, 2>, work, 256, 1, st, x, row_stride, m, rows_padded, k, n_ext, gs_inv, mask, codes, sf);
    default: return launch(nvfp4_kext_kernel<T, 4>, work, 256, 1, st, x, row_stride, m, rows_padded, k, n_ext, gs_inv, mask, codes, sf);
  }
}

extern "C" int ri_nvfp4_quant_kext(const void* x, int dtype, int m, int k, int64_t row_stride,
                                   const float* gs_inv, const uint8_t* mask, int per8, int n_ext,
                                   uint8_t* codes, int64_t codes_bytes, uint8_t* sf, int64_t sf_bytes,
                                   int use_swapped_residue, void* stream) {
  RI_CHECK_ARG(dtype == RI_DTYPE_BF16 || dtype == RI_DTYPE_FP16, "Unsupported input data type for quantize_to_fp4.");
  RI_CHECK_ARG(m >= 0 && k > 0 && k % 16 == 0, "The N dimension must be multiple of 16.");
  RI_CHECK_ARG(per8 != 8, "residue_per_8 == 8 (ratio 1.0) K-extension is no longer supported; use "
                          "scaled_fp4_quant_mext_r1 (M-extension).");
  RI_CHECK_ARG(per8 == 1 || per8 == 2 || per8 == 4, "Unsupported residue_per_8 value %d. Supported values: 1 (12.5%%), 2 (25%%), 4 (50%%).", per8);
  if (use_swapped_residue) {
    set_error("swapped-residue K-extension is not implemented");
    return RI_ERR_UNSUPPORTED;
  }
  const int s = k / 8 * per8;
  RI_CHECK_ARG(n_ext == k + s, "n_ext must equal K + K/8*residue_per_8 (%d), got %d", k + s, n_ext);
  RI_CHECK_ARG(s % 16 == 0, "the number of residue channels (%d) must be a multiple of 16", s);
  RI_CHECK_ARG(row_stride >= k && (row_stride * 2) % 16 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0,
               "input rows must be 16-byte aligned");
  RI_CHECK_ARG(codes_bytes >= int64_t(m) * n_ext / 2, "output tensor is too small");
  const int64_t need_sf = ((int64_t(m) + 127) / 128) * ((int64_t(n_ext) + 63) / 64) * 512;
  RI_CHECK_ARG(sf_bytes >= need_sf, "output scale tensor is too small: need %lld bytes, got %lld",
               (long long)need_sf, (long long)sf_bytes);
  RI_CHECK_ARG((reinterpret_cast<uintptr_t>(codes) & 7) == 0 && (n_ext / 2) % 4 == 0, "codes rows must be 4-byte aligned");
  if (m == 0) return RI_OK;
  const int rows_padded = (m + 127) / 128 * 128;
  const int64_t work = int64_t(rows_padded) * ((k / 16 + 31) / 32) * 32;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == RI_DTYPE_BF16)
    return launch_kext(per8, work, st, static_cast<const __nv_bfloat16*>(x), row_stride, m, rows_padded, k, n_ext, gs_inv, mask, codes, sf);
  return launch_kext(per8, work, st, static_cast<const __half*>(x), row_stride, m, rows_padded, k, n_ext, gs_inv, mask, codes, sf);
}

extern "C" int ri_nvfp4_quant_grouped_q(const void* q_bf16, int batch, int num_kv_heads, int group,
                                        int head_dim, uint8_t* q_pack, int64_t q_pack_bytes,
                                        uint8_t* q_sf, int64_t q_sf_bytes, void* stream) {
  RI_CHECK_ARG(group == 4 || group == 6 || group == 8, "grouped residue Q supports GQA4/6/8");
  RI_CHECK_ARG(head_dim == 128 || head_dim == 256, "grouped residue Q requires head_dim=128 or 256");
  RI_CHECK_ARG(batch >= 0 && num_kv_heads > 0, "bad batch / head count");
  const int p = group == 4 ? 8 : 16;
  RI_CHECK_ARG(q_pack_bytes >= int64_t(batch) * num_kv_heads * p * (head_dim / 2),
               "q_pack shape must match the physical Q tile");
  RI_CHECK_ARG(q_sf_bytes >= int64_t(batch) * num_kv_heads * 128 * (head_dim / 16),
               "grouped Q scale buffer is too small");
  RI_CHECK_ARG((reinterpret_cast<uintptr_t>(q_bf16) & 15) == 0 && (reinterpret_cast<uintptr_t>(q_pack) & 7) == 0,
               "q / q_pack must be 16 / 8-byte aligned");
  if (batch == 0) return RI_OK;
  const int64_t work = int64_t(batch) * num_kv_heads * group * (head_dim / 16);
  return launch(nvfp4_grouped_q_kernel, work, 128, 1, static_cast<cudaStream_t>(stream),
                static_cast<const __nv_bfloat16*>(q_bf16), q_pack, q_sf, batch * num_kv_heads, group, p, head_dim);
}
