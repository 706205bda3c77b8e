// ResAttn: residue-compensated paged NVFP4-KV decode attention (one query token per sequence).
//
// The query is quantised in the CTA prologue to NVFP4 plus an NVFP4 residue with the arithmetic of
// the grouped-Q quantiser (bit-identical codes); the scores of both are added, so the K cache is read
// once and nothing but the 4-bit KV codes and their E4M3 block scales crosses HBM.  Both kernels compute
// the scores on the block-scaled FP4 tensor cores (tcgen05) with an online softmax (lazy rescale: only
// when a row maximum moves by more than 2^8, row sums in unrounded FP32).  resattn_pv_kernel
// (resattn_pv.cuh, the one that runs) also does P.V on tcgen05, with V expanded to an FP16 operand tile in
// shared memory; resattn_tc_kernel below does P.V on mma.sync with V expanded in registers and is kept for
// comparisons (RI_ATTN_PV=0).  KV splits write (o, l, m) partials that a second kernel merges in split
// order (deterministic).
//
// Stands in for the reference's CuTeDSL decode kernel and its reducers (ShawRong/ResInfer
// csrc/resattn/kernel_paged_decode.py:722-2433, 2729-2861).
#include <cstdlib>

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
  int batch, hq, hkv, group, page_size;
  int page_shift;                          // log2(page_size) when it is a power of two, else -1
  int tiles_per_split;                     // 128-token tiles a KV split covers (the same for every sequence)
  float score_scale_log2;                  // sm_scale * k_global_scale * log2(e)
  float out_scale;
  void* out;                               // [B, Hq, D] bf16 (or fp32 when out_f32), or NVFP4 codes [B, Hq*D/2]
  int out_f32;
  int out_nvfp4;                           // packed NVFP4 output: codes in `out`, block scales in out_sf
  const float* out_gs;                     // device FP32: global scale of the NVFP4 output (1 / global scale of the consumer)
  uint8_t* out_sf;                         // 128x4-swizzled E4M3 block scales over [B, Hq*D]
  float* o_part; float* l_part; float* m_part;   // [splits, B, Hq, (D)]
  uint8_t* q_pack; uint8_t* q_sf;          // optional copies of the quantised query
  int splits, q_residue, stages;
  int32_t* status;
  long long* trace;                        // development builds only (RI_ATTN_PROFILE)
};

__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ __half e4m3_to_half(uint32_t byte) {
  __half_raw r = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)byte, __NV_E4M3);
  return __half(r);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// =================================================================================================
// Tensor-memory version: Q.K^T on the block-scaled FP4 tensor cores (tcgen05), P.V on mma.sync.
//
// One CTA per (KV split, KV head, sequence), 24 warps, tiles of 128 tokens:
//   warps 0-3  front end.  All four move the tile's K block scales from shared to tensor memory
//              (one warp per 32-lane quarter); warp 0 then issues
//              S^T[128 tokens x 16] = K[128 x D] . Qpack[16 x D]^T as D/64 tcgen05.mma
//              kind::mxf4nvf4.block_scale instructions -- the K codes and E4M3 scales are consumed
//              as stored, nothing is dequantised for the scores.  Qpack rows 0-7 are the NVFP4
//              query heads of the group, rows 8-15 their NVFP4 residues.
//   warps 4-7  copy producers: 16-byte cp.async copies of the K codes (written in the operand
//              swizzle), V codes and both scale arrays, 32 rows of the tile per warp.
//   warps 8-23 consumers.  A consumer reads its quarter of S^T from tensor memory, folds base +
//              residue columns, runs the online softmax for 16 tokens (head_dim 128) or the 32 tokens
//              of the quarter (head_dim 256) and accumulates P.V for 64 of the output columns, with V
//              expanded to FP16 on the fly (exact) and multiplied on mma.sync m16n8k16.  Warps that
//              share tokens repeat the (cheap) softmax so that sixteen warps hide each other's
//              latencies; the accumulators of a warp are only 8 n-tiles.
// S is double buffered in tensor memory, so the MMA of tile i+1 runs under the softmax of tile i.
// Every mbarrier wait is bounded (status word + normal teardown on expiry).
// =================================================================================================
__device__ __forceinline__ void store_nvfp4_out16(const float (&v)[16], float gs, uint8_t* codes_row, uint8_t* sf,
                                                  int row, int block, int hidden);

namespace tcattn {
using namespace tc;
// per-tile event times of CTA (0,0,0) in development builds: row `ev`, first 32 tiles
__device__ __forceinline__ void attn_event(const AttnParams& p, int ev, int tile) {
#ifdef RI_ATTN_PROFILE
  if (p.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && tile < 32) p.trace[ev * 32 + tile] = clock64();
#endif
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
constexpr int kTile = 128;
constexpr int kFront = 4, kCons = 16;
constexpr int kProd = 4;                                    // copy producer warps, 32 rows of a tile each
constexpr int kFirstCons = kFront + kProd;
constexpr int kThreadsTc = (kFront + kProd + kCons) * 32;   // 768
constexpr int kTmemColsTc = 128;
constexpr int kColS = 0, kColSfa = 32, kColSfb = 64;
constexpr int kMaxStagesTc = 12;
constexpr int kHeaderBytes = 20 * 1024;       // Qpack operand (2 KB), its scales (1 KB), score staging (16 KB)
constexpr int kColsPerWarp = 64;              // output columns a consumer accumulates

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
  static constexpr int kChunksPerWarp = D == 128 ? 1 : 2;      // 16-token chunks a consumer warp handles per tile
};

// byte offset of (row, byte) in a K-major operand tile with rows of D/2 bytes and the matching swizzle
template <int D>
__device__ __forceinline__ uint32_t swz_off(int row, int byte) {
  const int chunk = byte >> 4;
  if constexpr (D == 128) return row * 64 + (((chunk ^ ((row >> 1) & 3)) << 4) | (byte & 15));
  else return row * 128 + (((chunk ^ (row & 7)) << 4) | (byte & 15));
}

template <int D>
__global__ void __launch_bounds__(kThreadsTc, 1)
resattn_tc_kernel(const AttnParams p) {
  using C = TCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kMaxStagesTc];
  __shared__ __align__(8) uint64_t bar_empty[kMaxStagesTc];
  __shared__ __align__(8) uint64_t bar_sfull[2];
  __shared__ __align__(8) uint64_t bar_sempty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // stays a shared-space pointer
  uint8_t* q_op = smem;                                        // [16][D/2] swizzled FP4 codes
  uint8_t* qsf_s = smem + 2048;                                // [16][D/16] E4M3 scales
  float* sbuf = reinterpret_cast<float*>(smem + 3072);         // [16 warps][32 tokens][8 heads]
  uint8_t* stage0 = smem + kHeaderBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int G = p.group;
  const int S = p.stages;

  // ---------------------------------------------------------------- this CTA's tile range
  // A split covers a fixed number of tiles, so long sequences use many splits and short ones few;
  // a CTA whose range lies past the end of its sequence records an empty partial and leaves at once.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int L = min(max(__ldg(p.seq_lens + b), 0), int(p.bt_stride) * p.page_size);
  const int n_tiles = (L + kTile - 1) / kTile;
  const int t_begin = min(split * p.tiles_per_split, n_tiles);
  const int t_end = min(t_begin + p.tiles_per_split, n_tiles);
  const int my_tiles = t_end - t_begin;
  if (my_tiles == 0 && p.splits > 1 && !(p.q_pack && split == 0)) {     // (split 0 also emits the quantised query)
    if (threadIdx.x < G) {
      const int64_t slot = (int64_t(split) * p.batch + b) * p.hq + hkv * G + threadIdx.x;
      p.l_part[slot] = 0.f;
      p.m_part[slot] = -INFINITY;                  // the merge skips partials with m = -inf
    }
    return;
  }
  const int32_t* bt = p.block_tables + int64_t(b) * p.bt_stride;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&bar_full[s]), kProd * 32);    // one arrival per producer lane
      mbar_init(smem_u32(&bar_empty[s]), kCons);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_sfull[s]), 1);
      mbar_init(smem_u32(&bar_sempty[s]), kCons);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"(kTmemColsTc) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  for (int i = threadIdx.x; i < 3072 / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  // ---------------------------------------------------------------- query prologue
  // thread (g, blk) quantises one 16-block of head g to NVFP4 + NVFP4 residue (global scale 1, the
  // arithmetic of the grouped-Q quantiser) and stores the codes as the MMA B operand
  if (threadIdx.x < G * C::kSfPerRow) {
    const int g = threadIdx.x / C::kSfPerRow, blk = threadIdx.x % C::kSfPerRow;
    float v[16];
    load16(p.q + (int64_t(b) * p.hq + hkv * G + g) * D + blk * 16, v);
    BlockQ bq = quant_mext16(v, 1.0f, 1.0f);
    *reinterpret_cast<uint2*>(q_op + swz_off<D>(g, blk * 8)) = bq.base;
    qsf_s[g * C::kSfPerRow + blk] = bq.sf;
    if (p.q_residue) {
      *reinterpret_cast<uint2*>(q_op + swz_off<D>(8 + g, blk * 8)) = bq.res;
      qsf_s[(8 + g) * C::kSfPerRow + blk] = bq.sf_res;
    }
    if (p.q_pack && split == 0) {
      const int P = G == 4 ? 8 : 16;
      uint8_t* pack = p.q_pack + (int64_t(b) * p.hkv + hkv) * P * (D / 2);
      uint8_t* sfp = p.q_sf + (int64_t(b) * p.hkv + hkv) * 128 * C::kSfPerRow;
      *reinterpret_cast<uint2*>(pack + int64_t(g) * (D / 2) + blk * 8) = bq.base;
      *reinterpret_cast<uint2*>(pack + int64_t(P / 2 + g) * (D / 2) + blk * 8) = bq.res;
      sfp[sf_offset<16>(g, blk, D)] = bq.sf;
      sfp[sf_offset<16>(P / 2 + g, blk, D)] = bq.sf_res;
    }
  }
  // the operand was written with ordinary stores: make it visible to the tensor core's async reads
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  // everybody but the copy producers meets here; the producers are already filling the pipeline
  if (warp < kFront || warp >= kFirstCons)
    asm volatile("bar.sync 2, %0;" ::"n"(kThreadsTc - kProd * 32) : "memory");

  float oacc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) oacc[j][0] = oacc[j][1] = oacc[j][2] = oacc[j][3] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  const int tq = lane & 3, nq = lane >> 2;
  // consumer coordinates: tensor-memory quarter q, token half h (head_dim 128 only), column group e
  const int cw = warp - kFirstCons;
  const int cq = warp & 3, ck = cw >> 2;
  const int ch_half = D == 128 ? (ck & 1) : 0;
  const int ce = D == 128 ? (ck >> 1) : ck;

  if (warp < kFront) {
    // ============================================================ front end
    const int q = warp;
    const uint32_t lane_base = tmem_base + (uint32_t(q * 32) << 16);
    // Qpack block scales -> tensor memory (rows 0-15 live in lanes 0-15 of column 0 of each group of 4)
#pragma unroll
    for (int j = 0; j < C::kMma; ++j) {
      uint4 w = make_uint4(0, 0, 0, 0);
      if (lane < 16) w.x = *reinterpret_cast<const uint32_t*>(qsf_s + lane * C::kSfPerRow + 4 * j);
      tmem_st4(lane_base + kColSfb + 4 * j, w);
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    const uint32_t idesc = (1u << 7) | (1u << 10) | (uint32_t(16 >> 3) << 17) | (uint32_t(kTile >> 4) << 24);
    const uint64_t b_desc = desc_kmajor(smem_u32(q_op), C::kSbo, C::kLayout);
    for (int i = 0, stg = 0, ph = 0; i < my_tiles; ++i, stg = (stg + 1 == S ? 0 : stg + 1), ph ^= (stg == 0)) {
      const int sb = i & 1;                                  // stg = i % S, ph = (i / S) & 1, kept without divisions
      bool got = true;
      if (lane == 0) {
        got = mbar_wait(smem_u32(&bar_full[stg]), ph, &abort_flag, 2);
        if (got && i >= 2) got = mbar_wait(smem_u32(&bar_sempty[sb]), ((i >> 1) - 1) & 1, &abort_flag, 3);
      }
      if (!__all_sync(0xffffffffu, got)) break;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // cp.async data -> tensor-core reads
      tc_fence_after();
      if (warp == 0 && lane == 0) attn_event(p, 0, i);
      const uint8_t* st = stage0 + stg * C::kStageBytes;
      const uint8_t* ksf = st + C::kOffKsf;
      // K block scales of the tile -> scale set sb: lane l supplies rows l, l+32, l+64, l+96
      if constexpr (D == 128) {
        uint2 r0 = *reinterpret_cast<const uint2*>(ksf + (lane) * 8), r1 = *reinterpret_cast<const uint2*>(ksf + (lane + 32) * 8);
        uint2 r2 = *reinterpret_cast<const uint2*>(ksf + (lane + 64) * 8), r3 = *reinterpret_cast<const uint2*>(ksf + (lane + 96) * 8);
        const uint4 a[2] = {make_uint4(r0.x, r1.x, r2.x, r3.x), make_uint4(r0.y, r1.y, r2.y, r3.y)};
        tmem_st8(lane_base + kColSfa + sb * 16, a);
      } else {
        uint4 r0 = *reinterpret_cast<const uint4*>(ksf + (lane) * 16), r1 = *reinterpret_cast<const uint4*>(ksf + (lane + 32) * 16);
        uint4 r2 = *reinterpret_cast<const uint4*>(ksf + (lane + 64) * 16), r3 = *reinterpret_cast<const uint4*>(ksf + (lane + 96) * 16);
        const uint4 a[4] = {make_uint4(r0.x, r1.x, r2.x, r3.x), make_uint4(r0.y, r1.y, r2.y, r3.y),
                            make_uint4(r0.z, r1.z, r2.z, r3.z), make_uint4(r0.w, r1.w, r2.w, r3.w)};
        tmem_st16(lane_base + kColSfa + sb * 16, a);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 0) {
        tc_fence_after();
        if (elect_one()) {
          const uint64_t a_desc = desc_kmajor(smem_u32(st), C::kSbo, C::kLayout);
#pragma unroll
          for (int j = 0; j < C::kMma; ++j)
            mma_fp4<false>(tmem_base + kColS + sb * 16, a_desc + uint64_t(2 * j), b_desc + uint64_t(2 * j), idesc,
                           tmem_base + kColSfa + sb * 16 + 4 * j, tmem_base + kColSfb + 4 * j, j > 0 ? 1u : 0u);
          mma_commit(smem_u32(&bar_sfull[sb]));
        }
        __syncwarp();
        if (lane == 0) attn_event(p, 1, i);
      }
    }
  } else if (warp < kFirstCons) {
    // ============================================================ copy producers
    // Ampere-style 16-byte async copies, one per lane and instruction: with 16-token pages a tile is
    // 8 scattered slices x 4 arrays, far too many requests for the bulk-copy engine (measured: more
    // than 100 cycles of issue time per bulk copy), while a warp of cp.async moves 512 bytes per
    // instruction.  Producer warp w owns rows 32w..32w+31 of every tile (two page slices); the K
    // codes are written in the operand swizzle by address arithmetic.
    constexpr int kCpr = C::kRowBytes / 16;                    // 16-byte chunks per code row
    constexpr int kRowsPerIt = 32 / kCpr;                      // rows one warp instruction covers (8 or 4)
    constexpr int kIters = 32 / kRowsPerIt;                    // instructions per array and tile (4 or 8)
    const int pw = warp - kFront;
    // per-lane constants: row inside the instruction's row group, 16-byte chunk, scale row
    const int r_lane = lane / kCpr, chn = lane % kCpr;
    const int sf_row = D == 128 ? 2 * lane : lane;             // first row of this lane's 16 scale bytes
    const bool sf_lane = D == 128 ? lane < 16 : true;
    uint32_t k_dst[kIters];                                    // swizzled K offsets inside a stage
#pragma unroll
    for (int it = 0; it < kIters; ++it) k_dst[it] = swz_off<D>(32 * pw + it * kRowsPerIt + r_lane, chn * 16);
    const uint32_t v_dst0 = C::kOffV + (32 * pw + r_lane) * C::kRowBytes + chn * 16;
    const uint32_t sf_dst = (32 * pw + sf_row) * C::kSfPerRow;

    // block-table entry of slice `lane` (lanes 0 and 1) of a tile, fetched one tile ahead
    auto lookup = [&](int i) -> int {
      if (lane >= 2 || i >= my_tiles) return 0;
      const int t0 = (t_begin + i) * kTile + 32 * pw + lane * 16;
      return t0 < L ? __ldg(bt + (p.page_shift >= 0 ? t0 >> p.page_shift : t0 / p.page_size)) : 0;
    };
    int page_next = lookup(0);
    for (int i = 0, stg = 0, ph = 0; i < my_tiles; ++i, stg = (stg + 1 == S ? 0 : stg + 1), ph ^= (stg == 0)) {
      const int tok0 = (t_begin + i) * kTile + 32 * pw;
      const int rows = min(max(((L - tok0) + 15) & ~15, 0), 32);     // rows of this warp that exist (0, 16 or 32)
      int64_t page = page_next;
      page_next = lookup(i + 1);
      page = page < 0 ? 0 : (page >= p.num_pages ? p.num_pages - 1 : page);
      const int t0 = tok0 + lane * 16;
      const int in_page = p.page_shift >= 0 ? (t0 & (p.page_size - 1)) : t0 % p.page_size;
      const int64_t base_row = (page * p.hkv + hkv) * p.page_size + in_page;
      const int64_t base0 = __shfl_sync(0xffffffffu, base_row, 0), base1 = __shfl_sync(0xffffffffu, base_row, 1);
      bool free_ok = true;
      if (i >= S && lane == 0) free_ok = mbar_wait(smem_u32(&bar_empty[stg]), ph ^ 1, &abort_flag, 4);
      if (!__all_sync(0xffffffffu, free_ok)) break;
      const uint32_t st = smem_u32(stage0 + stg * C::kStageBytes);
      // rows 0-15 of this warp come from slice 0, rows 16-31 from slice 1
      const uint8_t* kg[2] = {p.k_data + base0 * C::kRowBytes + chn * 16, p.k_data + base1 * C::kRowBytes + chn * 16};
      const uint8_t* vg[2] = {p.v_data + base0 * C::kRowBytes + chn * 16, p.v_data + base1 * C::kRowBytes + chn * 16};
#pragma unroll
      for (int it = 0; it < kIters; ++it) {
        const int r = it * kRowsPerIt + r_lane;                // row inside this warp's 32
        if (it * kRowsPerIt < rows) {
          const int sl = (it * kRowsPerIt) >> 4;               // compile-time slice of the instruction
          const int off = (r & 15) * C::kRowBytes;
          cp_async16(st + k_dst[it], kg[sl] + off);
          cp_async16(st + v_dst0 + it * kRowsPerIt * C::kRowBytes, vg[sl] + off);
        }
      }
      if (sf_lane && sf_row < rows) {
        const int64_t br = (sf_row < 16 ? base0 : base1) + (sf_row & 15);
        cp_async16(st + C::kOffKsf + sf_dst, p.k_sf + br * C::kSfPerRow);
        cp_async16(st + C::kOffVsf + sf_dst, p.v_sf + br * C::kSfPerRow);
      }
      // every lane arrives once its own copies have landed (barrier count = producer lanes)
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&bar_full[stg])) : "memory");
      if (pw == 0 && lane == 0) attn_event(p, 2, i);
    }
  } else {
    // ============================================================ consumers
    const uint32_t lane_base = tmem_base + (uint32_t(cq * 32) << 16);
    float* my_s = sbuf + cw * 32 * 8;
    for (int i = 0, stg = 0, ph = 0; i < my_tiles; ++i, stg = (stg + 1 == S ? 0 : stg + 1), ph ^= (stg == 0)) {
      const int sb = i & 1;
      const int tile = t_begin + i;
      bool got = true;
      if (cw == 0 && lane == 0) attn_event(p, 6, i);
      if (lane == 0) {
        got = mbar_wait(smem_u32(&bar_sfull[sb]), (i >> 1) & 1, &abort_flag, 5);
        if (cw == 0) attn_event(p, 7, i);
        // the V codes and scales of the stage were written by the copy engine: observe its barrier too
        if (got) got = mbar_wait(smem_u32(&bar_full[stg]), ph, &abort_flag, 6);
      }
      if (!__all_sync(0xffffffffu, got)) break;
      tc_fence_after();
      if (cw == 0 && lane == 0) attn_event(p, 3, i);
      float r[16];
      tmem_ld16(lane_base + kColS + sb * 16, r);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_sempty[sb]));
      // fold the residue columns onto the base columns, move to the log2 domain, stage for the
      // fragment-order reads below: token `lane` of the quarter, 8 heads
      {
        float4 lo, hi;
        lo.x = (r[0] + r[8]) * p.score_scale_log2;  lo.y = (r[1] + r[9]) * p.score_scale_log2;
        lo.z = (r[2] + r[10]) * p.score_scale_log2; lo.w = (r[3] + r[11]) * p.score_scale_log2;
        hi.x = (r[4] + r[12]) * p.score_scale_log2; hi.y = (r[5] + r[13]) * p.score_scale_log2;
        hi.z = (r[6] + r[14]) * p.score_scale_log2; hi.w = (r[7] + r[15]) * p.score_scale_log2;
        if (D == 256 || (lane >> 4) == ch_half) {
          reinterpret_cast<float4*>(my_s + lane * 8)[0] = lo;
          reinterpret_cast<float4*>(my_s + lane * 8)[1] = hi;
        }
      }
      __syncwarp();
      if (cw == 0 && lane == 0) attn_event(p, 4, i);
      const uint8_t* st = stage0 + stg * C::kStageBytes;
#pragma unroll
      for (int c = 0; c < C::kChunksPerWarp; ++c) {
        const int tok_in_q = D == 128 ? 16 * ch_half : 16 * c;       // first token of the chunk inside the quarter
        const int tok_in_tile = 32 * cq + tok_in_q;
        const int valid = min(L - (tile * kTile + tok_in_tile), 16);
        if (valid <= 0) continue;
        float sv[4];
        sv[0] = my_s[(tok_in_q + 2 * tq) * 8 + nq];
        sv[1] = my_s[(tok_in_q + 2 * tq + 1) * 8 + nq];
        sv[2] = my_s[(tok_in_q + 2 * tq + 8) * 8 + nq];
        sv[3] = my_s[(tok_in_q + 2 * tq + 9) * 8 + nq];
        if (valid < 16) {
          if (2 * tq >= valid) sv[0] = -INFINITY;
          if (2 * tq + 1 >= valid) sv[1] = -INFINITY;
          if (8 + 2 * tq >= valid) sv[2] = -INFINITY;
          if (9 + 2 * tq >= valid) sv[3] = -INFINITY;
        }
        float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        if (mx > m_run + kLazyThreshold || m_run == -INFINITY) {
          const float f = fast_exp2(m_run - mx);                // 0 on the first chunk
          m_run = mx;
          l_run *= f;
#pragma unroll
          for (int j = 0; j < 8; ++j) { oacc[j][0] *= f; oacc[j][1] *= f; }
        }
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) pv[e] = fast_exp2(sv[e] - m_run);
        l_run += (pv[0] + pv[1]) + (pv[2] + pv[3]);
        uint32_t pa[4];
        pa[0] = h2_bits(__floats2half2_rn(pv[0], pv[1]));
        pa[1] = 0u;
        pa[2] = h2_bits(__floats2half2_rn(pv[2], pv[3]));
        pa[3] = 0u;
        // O += P . V for this warp's 64 output columns: lane (tq, nq) owns token rows
        // {2tq, 2tq+1, 2tq+8, 2tq+9} and the 8 columns 64 ce + 8 nq + j (half a scale block)
        const int col_byte0 = 32 * ce + nq * 4;
        const int sf_idx0 = 4 * ce + (nq >> 1);
        uint32_t vw[4];
        __half vs[4];
        const uint8_t* vrow = st + C::kOffV + (tok_in_tile + 2 * tq) * C::kRowBytes + col_byte0;
        const uint8_t* srow = st + C::kOffVsf + (tok_in_tile + 2 * tq) * C::kSfPerRow + sf_idx0;
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) {
          const int dr = (rr & 1) + (rr >> 1) * 8;              // rows 2tq, 2tq+1, 2tq+8, 2tq+9
          vw[rr] = *reinterpret_cast<const uint32_t*>(vrow + dr * C::kRowBytes);
          vs[rr] = e4m3_to_half(srow[dr * C::kSfPerRow]);
        }
        if (valid < 16) {                                       // rows past the sequence end hold stale bytes
#pragma unroll
          for (int rr = 0; rr < 4; ++rr)
            if (2 * tq + (rr & 1) + (rr >> 1) * 8 >= valid) { vw[rr] = 0u; vs[rr] = __half(0.f); }
        }
        const __half2 s01 = __halves2half2(vs[0], vs[1]);
        const __half2 s89 = __halves2half2(vs[2], vs[3]);
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          const int sh = j * 4;
          const uint32_t x0 = h2_bits(e2m1x2_to_half2((vw[0] >> sh) & 0xFFu));
          const uint32_t x1 = h2_bits(e2m1x2_to_half2((vw[1] >> sh) & 0xFFu));
          const uint32_t x8 = h2_bits(e2m1x2_to_half2((vw[2] >> sh) & 0xFFu));
          const uint32_t x9 = h2_bits(e2m1x2_to_half2((vw[3] >> sh) & 0xFFu));
          const uint32_t b0_lo = h2_bits(__hmul2(bits_h2(__byte_perm(x0, x1, 0x5410)), s01));
          const uint32_t b0_hi = h2_bits(__hmul2(bits_h2(__byte_perm(x0, x1, 0x7632)), s01));
          const uint32_t b1_lo = h2_bits(__hmul2(bits_h2(__byte_perm(x8, x9, 0x5410)), s89));
          const uint32_t b1_hi = h2_bits(__hmul2(bits_h2(__byte_perm(x8, x9, 0x7632)), s89));
          mma_f16(oacc[j], pa, b0_lo, b1_lo);
          mma_f16(oacc[j + 1], pa, b0_hi, b1_hi);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_empty[stg]));
      if (cw == 0 && lane == 0) attn_event(p, 5, i);
    }
  }

  // ---------------------------------------------------------------- merge the consumer warps
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  tc_fence_before();
  __syncthreads();                                           // pipeline memory is free now
  float* o_w = reinterpret_cast<float*>(stage0);              // [16 warps][8 heads][64 columns]
  float* m_w = o_w + kCons * 8 * kColsPerWarp;
  float* l_w = m_w + kCons * 8;
  if (warp >= kFirstCons) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // accumulator columns 2tq / 2tq+1 of n-tile j are columns 8 * (2tq) + j and 8 * (2tq+1) + j of the group
      o_w[(cw * 8 + nq) * kColsPerWarp + 8 * (2 * tq) + j] = oacc[j][0];
      o_w[(cw * 8 + nq) * kColsPerWarp + 8 * (2 * tq + 1) + j] = oacc[j][1];
    }
    if (tq == 0) {
      m_w[cw * 8 + nq] = m_run;
      l_w[cw * 8 + nq] = l_run;
    }
  }
  __syncthreads();
  const bool failed = abort_flag != 0;
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    const int e = d >> 6, dc = d & 63;
    // consumer warps that own column group e: index k = cw >> 2 (k & 1 = token half, k >> 1 = e for
    // head_dim 128; k = e for head_dim 256), all four quarters
    float mm = -INFINITY;
    for (int w = 0; w < kCons; ++w) {
      const int k = w >> 2;
      if ((D == 128 ? (k >> 1) : k) == e) mm = fmaxf(mm, m_w[w * 8 + g]);
    }
    float o = 0.f, l = 0.f;
    for (int w = 0; w < kCons; ++w) {
      const int k = w >> 2;
      if ((D == 128 ? (k >> 1) : k) != e) continue;
      const float mw = m_w[w * 8 + g];
      const float f = mw == -INFINITY ? 0.f : fast_exp2(mw - mm);
      o += f * o_w[(w * 8 + g) * kColsPerWarp + dc];
      l += f * l_w[w * 8 + g];
    }
    const int head = hkv * G + g;
    if (p.splits == 1) {
      const float rr = l > 0.f ? p.out_scale / l : 0.f;
      const int64_t oi = (int64_t(b) * p.hq + head) * D + d;
      if (p.out_nvfp4) sbuf[g * D + d] = o * rr;                 // quantised below, 16 values per thread
      else if (p.out_f32) static_cast<float*>(p.out)[oi] = o * rr;
      else static_cast<__nv_bfloat16*>(p.out)[oi] = __float2bfloat16_rn(o * rr);
    } else {
      const int64_t slot = (int64_t(split) * p.batch + b) * p.hq + head;
      p.o_part[slot * D + d] = o;
      if (d == 0) {
        p.l_part[slot] = l;
        p.m_part[slot] = mm;
      }
    }
  }
  if (failed && threadIdx.x == 0 && p.status) atomicExch(p.status, 1 + int(blockIdx.z) + (abort_flag << 16));
  __syncthreads();
  if (p.out_nvfp4 && p.splits == 1 && threadIdx.x < G * (D / 16)) {
    const int g = threadIdx.x / (D / 16), blk = threadIdx.x % (D / 16);
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = sbuf[g * D + blk * 16 + i];
    const int head = hkv * G + g, hidden = p.hq * D;
    store_nvfp4_out16(v, __ldg(p.out_gs), static_cast<uint8_t*>(p.out) + int64_t(b) * (hidden / 2), p.out_sf, b,
                      head * (D / 16) + blk, hidden);
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColsTc) : "memory");
  }
}

template <int D>
int launch_decode_tc(const AttnParams& p, cudaStream_t st) {
  using C = TCfg<D>;
  const int smem = kHeaderBytes + p.stages * C::kStageBytes + 1024;
  static bool attr_done[64] = {};                    // function attributes are per device
  int dev = 0;
  RI_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) dev = 0;
  if (!attr_done[dev]) {
    RI_CUDA(cudaFuncSetAttribute(resattn_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.splits, p.hkv, p.batch);
  cfg.blockDim = dim3(kThreadsTc);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cuda_status(cudaLaunchKernelEx(&cfg, resattn_tc_kernel<D>, p), "resattn decode launch");
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

// out[b, h, :] = sum_s 2^(m_s - m) o_s / sum_s 2^(m_s - m) l_s * out_scale, splits in order
__global__ void resattn_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ l_part,
                                     const float* __restrict__ m_part, void* __restrict__ out, int out_f32,
                                     int splits, int64_t rows, int d, float out_scale, int out_nvfp4,
                                     const float* __restrict__ out_gs, uint8_t* __restrict__ out_sf, int hq) {
  __shared__ float row_vals[256];
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t row = blockIdx.x;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, m_part[s * rows + row]);
  float l = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = m_part[s * rows + row];
    l += (ms == -INFINITY ? 0.f : fast_exp2(ms - mm)) * l_part[s * rows + row];
  }
  const float r = l > 0.f ? out_scale / l : 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = m_part[s * rows + row];
      if (ms != -INFINITY) o += fast_exp2(ms - mm) * o_part[(s * rows + row) * d + c];   // empty partials hold no data
    }
    if (out_nvfp4) row_vals[c] = o * r;
    else if (out_f32) static_cast<float*>(out)[row * d + c] = o * r;
    else static_cast<__nv_bfloat16*>(out)[row * d + c] = __float2bfloat16_rn(o * r);
  }
  if (out_nvfp4) {
    __syncthreads();
    if (threadIdx.x < d / 16) {
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = row_vals[threadIdx.x * 16 + i];
      const int b = int(row / hq), head = int(row % hq), hidden = hq * d;
      store_nvfp4_out16(v, __ldg(out_gs), static_cast<uint8_t*>(out) + int64_t(b) * (hidden / 2), out_sf, b,
                        head * (d / 16) + int(threadIdx.x), hidden);
    }
  }
}

}  // namespace
}  // namespace ri

using namespace ri;

extern "C" int64_t ri_resattn_workspace_bytes(int batch, int num_q_heads, int head_dim, int splits) {
  if (splits <= 1) return 0;
  const int64_t rows = int64_t(splits) * batch * num_q_heads;
  return rows * head_dim * 4 + 2 * rows * 4;
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
  RI_CHECK_ARG(head_dim == 128 || head_dim == 256, "ResAttn supports head_dim=128 or 256");
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
  p.batch = batch; p.hq = num_q_heads; p.hkv = num_kv_heads; p.group = group; p.page_size = page_size;
  p.page_shift = -1;
  for (int sft = 4; sft < 31; ++sft)
    if ((1 << sft) == page_size) p.page_shift = sft;
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
#ifdef RI_ATTN_PROFILE
  if (const char* e = getenv("RI_ATTN_TRACE_PTR")) p.trace = reinterpret_cast<long long*>(strtoull(e, nullptr, 16));
#endif
  p.stages = head_dim == 128 ? 8 : 4;
  if (splits > 1) {
    const int64_t need = ri_resattn_workspace_bytes(batch, num_q_heads, head_dim, splits);
    RI_CHECK_ARG(workspace != nullptr && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
                 "split-KV with %d splits needs a 16-byte aligned workspace of %lld bytes, got %lld", splits,
                 (long long)need, (long long)workspace_bytes);
    const int64_t rows = int64_t(splits) * batch * num_q_heads;
    p.o_part = static_cast<float*>(workspace);
    p.l_part = p.o_part + rows * head_dim;
    p.m_part = p.l_part + rows;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Both head dimensions run the kernel with both products on the tensor cores; RI_ATTN_PV=0 selects the
  // mma.sync P.V kernel for comparisons
  static const bool use_pv = [] { const char* e = getenv("RI_ATTN_PV"); return !(e && e[0] == '0'); }();
  s = head_dim == 128 ? (use_pv ? tcattn::launch_decode_pv<128>(p, st) : tcattn::launch_decode_tc<128>(p, st))
                      : (use_pv ? tcattn::launch_decode_pv<256>(p, st) : tcattn::launch_decode_tc<256>(p, st));
  if (s) return s;
  if (splits > 1) {
    const int64_t rows = int64_t(batch) * num_q_heads;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)rows);
    cfg.blockDim = dim3(head_dim <= 128 ? 128 : 256);
    cfg.stream = st;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cuda_status(cudaLaunchKernelEx(&cfg, resattn_merge_kernel, (const float*)p.o_part, (const float*)p.l_part,
                                          (const float*)p.m_part, p.out, p.out_f32, splits, rows, head_dim, out_scale, p.out_nvfp4,
                                          p.out_gs, p.out_sf, num_q_heads),
                       "resattn merge launch");
  }
  return RI_OK;
}
