// ResAttn: residue-compensated paged NVFP4-KV decode attention (one query token per sequence).
//
// The query is quantised in the CTA prologue to NVFP4 plus an NVFP4 residue with the arithmetic of
// the grouped-Q quantiser (bit-identical codes); the scores of both are added, so the K cache is read
// once and nothing but the 4-bit KV codes and their E4M3 block scales crosses HBM.  The decode kernel
// (resattn_pv_kernel, resattn_pv.cuh) computes the scores on the block-scaled FP4 tensor cores (tcgen05)
// with an online softmax (lazy rescale: only when a row maximum moves by more than 2^8, row sums in
// unrounded FP32) and P.V on tcgen05 as well, with V expanded to an operand tile in shared memory.
// KV splits write (o, l, m) partials; the CTA that finishes last merges them in split order (deterministic,
// no second launch, nobody waits).
//
// Stands in for the reference's CuTeDSL decode kernel and its reducers (ShawRong/ResInfer
// csrc/resattn/kernel_paged_decode.py:722-2433, 2729-2861).
#include "common.cuh"
#include "resinfer_b200.h"
#include "tc05.cuh"

namespace ri {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLazyThreshold = 8.0f;     // rescale only when the row maximum grows by > 2^8

struct AttnParams {
  const __nv_bfloat16* q;                  // [B, Hq, D]
  const uint8_t* k_data; const uint8_t* k_sf;
  const uint8_t* v_data; const uint8_t* v_sf;
  const int32_t* block_tables; int64_t bt_stride;
  const int32_t* seq_lens;
  int64_t num_pages;
  int64_t code_page_stride, sf_page_stride; // bytes from one page's [Hkv, page_size] rows of codes (scales) to the next page's
  int batch, hq, hkv, group, page_size;
  int page_shift;                          // log2(page_size) when it is a power of two, else -1
  int tma_pages;                           // pages hold whole 128-token tiles: codes and V scales come by TMA
  int tiles_per_split;                     // 128-token tiles a KV split covers (the same for every sequence)
  float score_scale_log2;                  // sm_scale * k_global_scale * log2(e)
  float out_scale;
  void* out;                               // [B, Hq, D] bf16 (or fp32 when out_f32), or NVFP4 codes [B, Hq*D/2]
  int out_f32;
  int out_nvfp4;                           // packed NVFP4 output: codes in `out`, block scales in out_sf
  const float* out_gs;                     // device FP32: global scale of the NVFP4 output (1 / global scale of the consumer)
  uint8_t* out_sf;                         // 128x4-swizzled E4M3 block scales over [B, Hq*D]
  float* o_part; float* l_part; float* m_part;   // [splits, B, Hq, (D)]
  int* split_counter;                      // [B, Hkv] tickets of the fused split merge (zero between calls)
  uint8_t* q_pack; uint8_t* q_sf;          // optional copies of the quantised query
  int splits, q_residue;
  int sm_count;                            // host side only: SMs of the device
  int cluster_merge;                       // the splits of a (sequence, KV head) are one cluster and merge through its shared memory
  int32_t* status;
};

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void store_nvfp4_out16(const float (&v)[16], float gs, uint8_t* codes_row, uint8_t* sf,
                                                  int row, int block, int hidden);

namespace tcattn {
using namespace tc;
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
constexpr int kTile = 128;                                  // tokens per tile
constexpr int kColS = 0, kColSfa = 32, kColSfb = 64;        // tensor-memory columns: scores, K scales, Q scales

template <int D>
struct TCfg {
  static constexpr int kRowBytes = D / 2;
  static constexpr int kSfPerRow = D / 16;
  static constexpr int kMma = D / 64;
  static constexpr int kKBytes = kTile * kRowBytes;
  static constexpr int kSfBytes = kTile * kSfPerRow;
  static constexpr int kStageBytes = 2 * kKBytes + 2 * kSfBytes;
  static constexpr int kOffV = kKBytes, kOffKsf = 2 * kKBytes, kOffVsf = 2 * kKBytes + kSfBytes;
  static constexpr uint32_t kLayout = D == 128 ? 4u : 2u;      // 64-byte / 128-byte swizzle (row = D/2 bytes)
  static constexpr uint32_t kSbo = 8 * kRowBytes;
};

// byte offset of (row, byte) in a K-major operand tile with rows of D/2 bytes and the matching swizzle
template <int D>
__device__ __forceinline__ uint32_t swz_off(int row, int byte) {
  const int chunk = byte >> 4;
  if constexpr (D == 128) return row * 64 + (((chunk ^ ((row >> 1) & 3)) << 4) | (byte & 15));
  else return row * 128 + (((chunk ^ (row & 7)) << 4) | (byte & 15));
}

#include "resattn_pv.cuh"
}  // namespace tcattn


// One 16-element block of the attention output -> NVFP4 codes + E4M3 block scale, the arithmetic of the
// reference's packed output path (ShawRong/ResInfer csrc/resattn/output.py:10-34):
// scale = e4m3(amax * gs * (1/6)), multiplier = gs * rcp(scale) (0 for an all-zero block).
__device__ __forceinline__ void store_nvfp4_out16(const float (&v)[16], float gs, uint8_t* codes_row, uint8_t* sf,
                                                  int row, int block, int hidden) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  uint8_t sf_byte;
  const float sfv = encode_e4m3(amax * gs * (1.0f / 6.0f), &sf_byte);
  const float mult = sfv != 0.f ? gs * rcp_approx_ftz(sfv) : 0.f;
  *reinterpret_cast<uint2*>(codes_row + block * 8) = quant_plain16(v, mult);
  sf[sf_offset<16>(row, block, hidden)] = sf_byte;
}

}  // namespace
}  // namespace ri

using namespace ri;

namespace {
int g_pv_e4m3 = 0;        // number format of V and P in the second product: 0 = FP16, 1 = E4M3
}
extern "C" void ri_resattn_set_pv_format(int e4m3) { g_pv_e4m3 = e4m3 ? 1 : 0; }
extern "C" int ri_resattn_get_pv_format(void) { return g_pv_e4m3; }

extern "C" int64_t ri_resattn_counter_bytes(int batch, int num_q_heads) {
  // one ticket per (sequence, KV head); sized by the query heads, which bound the KV heads
  return (int64_t(batch) * num_q_heads * 4 + 255) / 256 * 256;
}

extern "C" int64_t ri_resattn_workspace_bytes(int batch, int num_q_heads, int head_dim, int splits) {
  if (splits <= 1) return 0;
  const int64_t rows = int64_t(splits) * batch * num_q_heads;
  return ri_resattn_counter_bytes(batch, num_q_heads) + rows * head_dim * 4 + 2 * rows * 4;
}

extern "C" int ri_resattn_decode_strided(const void* q_bf16, const uint8_t* k_data, const uint8_t* k_sf,
                                 const uint8_t* v_data, const uint8_t* v_sf, int64_t num_pages,
                                 int64_t code_page_stride, int64_t sf_page_stride,
                                 const int32_t* block_tables, int64_t bt_stride, const int32_t* seq_lens,
                                 int batch, int num_q_heads, int num_kv_heads, int head_dim, int page_size,
                                 int max_kv_len, float score_scale, float out_scale, void* out, int out_dtype, uint8_t* q_pack,
                                 int64_t q_pack_bytes, uint8_t* q_sf, int64_t q_sf_bytes,
                                 const float* out_global_scale, uint8_t* out_block_scale,
                                 int64_t out_block_scale_bytes, int splits, int reducer,
                                 void* workspace, int64_t workspace_bytes, int q_residue, int32_t* status,
                                 void* stream) {
  RI_CHECK_ARG(head_dim == 128 || head_dim == 256, "ResAttn supports head_dim=128 or 256");
  RI_CHECK_ARG(reducer == RI_ATTN_REDUCER_TICKET || reducer == RI_ATTN_REDUCER_CLUSTER, "unknown split reducer %d", reducer);
  RI_CHECK_ARG(reducer != RI_ATTN_REDUCER_CLUSTER ||
                   (((splits >= 2 && splits <= 8) || splits == 16) && out_dtype != RI_DTYPE_NVFP4),
               "the cluster reducer takes 2 to 8 or 16 splits and BF16 / FP32 output, got %d splits, output type %d",
               splits, out_dtype);
  RI_CHECK_ARG(out_dtype == RI_DTYPE_BF16 || out_dtype == RI_DTYPE_F32 || out_dtype == RI_DTYPE_NVFP4,
               "output must be bf16 (or packed NVFP4)");
  if (out_dtype == RI_DTYPE_NVFP4) {
    const int64_t hidden = int64_t(num_q_heads) * head_dim;
    const int64_t need = ((int64_t(batch) + 127) / 128) * ((hidden + 63) / 64) * 512;
    RI_CHECK_ARG(out_global_scale != nullptr && out_block_scale != nullptr && out_block_scale_bytes >= need,
                 "NVFP4 output needs a global scale and a 128x4 block-scale buffer of %lld bytes, got %lld",
                 (long long)need, (long long)out_block_scale_bytes);
    RI_CHECK_ARG((reinterpret_cast<uintptr_t>(out) & 7) == 0, "NVFP4 output must be 8-byte aligned");
  }
  RI_CHECK_ARG(num_kv_heads > 0 && num_q_heads % num_kv_heads == 0, "H_q=%d must be divisible by H_kv=%d",
               num_q_heads, num_kv_heads);
  const int group = num_q_heads / num_kv_heads;
  RI_CHECK_ARG(group == 4 || group == 6 || group == 8,
               "decode residue Q8/Q16 supports logical GQA ratios (4, 6, 8), got %d", group);
  RI_CHECK_ARG(page_size >= 16 && page_size % 16 == 0, "page size must be a multiple of 16, got %d", page_size);
  RI_CHECK_ARG(batch >= 0 && num_pages > 0 && bt_stride >= 1, "bad batch / page pool / block table");
  {
    const int64_t page_rows = int64_t(num_kv_heads) * page_size;
    if (code_page_stride == 0) code_page_stride = page_rows * (head_dim / 2);
    if (sf_page_stride == 0) sf_page_stride = page_rows * (head_dim / 16);
    RI_CHECK_ARG(code_page_stride >= page_rows * (head_dim / 2) && sf_page_stride >= page_rows * (head_dim / 16) &&
                     code_page_stride % 16 == 0 && sf_page_stride % 16 == 0,
                 "page strides (%lld, %lld bytes) must be multiples of 16 and hold a page's %lld rows",
                 (long long)code_page_stride, (long long)sf_page_stride, (long long)page_rows);
  }
  RI_CHECK_ARG(splits >= 1 && splits <= 256, "splits must be in [1, 256]");
  RI_CHECK_ARG(max_kv_len >= 0, "max_kv_len must be non-negative");
  RI_CHECK_ARG((reinterpret_cast<uintptr_t>(k_data) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_data) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(k_sf) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_sf) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(q_bf16) & 15) == 0,
               "q and the KV pool must be 16-byte aligned");
  if (q_pack) {
    const int P = group == 4 ? 8 : 16;
    RI_CHECK_ARG(q_sf != nullptr && q_pack_bytes >= int64_t(batch) * num_kv_heads * P * (head_dim / 2) &&
                     q_sf_bytes >= int64_t(batch) * num_kv_heads * 128 * (head_dim / 16),
                 "q_pack / q_sf scratch too small");
  }
  if (batch == 0) return RI_OK;
  DeviceInfo di;
  int s = device_info(&di);
  if (s) return s;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q_bf16);
  p.k_data = k_data; p.k_sf = k_sf; p.v_data = v_data; p.v_sf = v_sf;
  p.block_tables = block_tables; p.bt_stride = bt_stride; p.seq_lens = seq_lens; p.num_pages = num_pages;
  p.code_page_stride = code_page_stride; p.sf_page_stride = sf_page_stride;
  p.batch = batch; p.hq = num_q_heads; p.hkv = num_kv_heads; p.group = group; p.page_size = page_size;
  p.page_shift = -1;
  for (int sft = 4; sft < 31; ++sft)
    if ((1 << sft) == page_size) p.page_shift = sft;
  // tiled TMA coordinates are 32-bit (row within the page, page): always in range for a page pool
  p.tma_pages = (page_size % 128 == 0 && num_pages < (int64_t(1) << 31)) ? 1 : 0;
  p.score_scale_log2 = score_scale * kLog2e;
  p.out_scale = out_scale;
  p.out = out;
  p.out_f32 = out_dtype == RI_DTYPE_F32;
  p.out_nvfp4 = out_dtype == RI_DTYPE_NVFP4;
  p.out_gs = out_global_scale;
  p.out_sf = out_block_scale;
  p.q_pack = q_pack; p.q_sf = q_sf;
  p.splits = splits; p.q_residue = q_residue; p.status = status;
  {
    const int64_t cap = bt_stride * page_size;
    const int64_t bound = max_kv_len > 0 && max_kv_len < cap ? max_kv_len : cap;
    const int64_t tiles = (bound + 127) / 128;
    p.tiles_per_split = int((tiles + splits - 1) / splits);
    if (p.tiles_per_split < 1) p.tiles_per_split = 1;
  }
  p.cluster_merge = reducer == RI_ATTN_REDUCER_CLUSTER;
  p.sm_count = di.sm_count;
  if (splits > 1 && !p.cluster_merge) {
    const int64_t need = ri_resattn_workspace_bytes(batch, num_q_heads, head_dim, splits);
    RI_CHECK_ARG(workspace != nullptr && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
                 "split-KV with %d splits needs a 16-byte aligned workspace of %lld bytes, got %lld", splits,
                 (long long)need, (long long)workspace_bytes);
    const int64_t rows = int64_t(splits) * batch * num_q_heads;
    p.split_counter = static_cast<int*>(workspace);
    p.o_part = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + ri_resattn_counter_bytes(batch, num_q_heads));
    p.l_part = p.o_part + rows * head_dim;
    p.m_part = p.l_part + rows;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (g_pv_e4m3)
    s = head_dim == 128 ? tcattn::launch_decode_pv<128, true>(p, st) : tcattn::launch_decode_pv<256, true>(p, st);
  else
    s = head_dim == 128 ? tcattn::launch_decode_pv<128, false>(p, st) : tcattn::launch_decode_pv<256, false>(p, st);
  return s;
}

extern "C" int ri_resattn_prepare(int head_dim) {
  RI_CHECK_ARG(head_dim == 128 || head_dim == 256, "ResAttn supports head_dim=128 or 256");
  int s = head_dim == 128 ? tcattn::prepare_decode_pv<128, false>() : tcattn::prepare_decode_pv<256, false>();
  if (s) return s;
  return head_dim == 128 ? tcattn::prepare_decode_pv<128, true>() : tcattn::prepare_decode_pv<256, true>();
}

extern "C" int ri_resattn_decode(const void* q_bf16, const uint8_t* k_data, const uint8_t* k_sf,
                                 const uint8_t* v_data, const uint8_t* v_sf, int64_t num_pages,
                                 const int32_t* block_tables, int64_t bt_stride, const int32_t* seq_lens,
                                 int batch, int num_q_heads, int num_kv_heads, int head_dim, int page_size,
                                 int max_kv_len, float score_scale, float out_scale, void* out, int out_dtype, uint8_t* q_pack,
                                 int64_t q_pack_bytes, uint8_t* q_sf, int64_t q_sf_bytes,
                                 const float* out_global_scale, uint8_t* out_block_scale,
                                 int64_t out_block_scale_bytes, int splits,
                                 void* workspace, int64_t workspace_bytes, int q_residue, int32_t* status,
                                 void* stream) {
  return ri_resattn_decode_strided(q_bf16, k_data, k_sf, v_data, v_sf, num_pages, 0, 0, block_tables, bt_stride, seq_lens,
                                   batch, num_q_heads, num_kv_heads, head_dim, page_size, max_kv_len, score_scale,
                                   out_scale, out, out_dtype, q_pack, q_pack_bytes, q_sf, q_sf_bytes, out_global_scale,
                                   out_block_scale, out_block_scale_bytes, splits, RI_ATTN_REDUCER_TICKET, workspace,
                                   workspace_bytes, q_residue, status, stream);
}
