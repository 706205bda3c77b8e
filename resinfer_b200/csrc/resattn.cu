// ResAttn: residue-compensated paged NVFP4-KV decode attention (one query token per sequence).
//
// HBM-bound streaming kernel.  One CTA per (KV split, KV head, sequence), four independent
// warps per CTA.  Each warp walks its own 16-token chunks of the sequence through a private ring
// of shared-memory stages that one lane fills with bulk async copies (cp.async.bulk +
// mbarrier::complete_tx) of the chunk's K codes, K scales, V codes and V scales -- 1-D TMA copies
// of whole page slices, nothing else touches HBM.  Per chunk:
//   * K and V nibbles are expanded to FP16 exactly (E2M1 x E4M3 fits FP16) and multiplied on
//     the legacy tensor-core path (mma.sync m16n8k16, FP32 accumulate);
//   * the 16 MMA rows hold the NVFP4 query in rows 0-7 and its NVFP4 residue in rows 8-15, so the
//     base and residue scores of one head land in the same thread and the fold is one add;
//   * online softmax with warp-shuffle row maxima and a lazy rescale (only when the maximum moves
//     by more than 2^8), row sums kept in unrounded FP32.
// The query is quantised in the CTA prologue with the same arithmetic as the grouped-Q quantiser
// (bit-identical codes).  Warps merge through shared memory; KV splits write (o, l, m) partials that
// a second kernel merges in split order (deterministic).
//
// Stands in for the reference's CuTeDSL decode kernel and its reducers (ShawRong/ResInfer
// csrc/resattn/kernel_paged_decode.py:722-2433, 2729-2861).
#include "common.cuh"
#include "resinfer_b200.h"

namespace ri {
namespace {

constexpr int kWarps = 4;
constexpr int kChunk = 16;                 // tokens per pipeline stage
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
  float score_scale_log2;                  // sm_scale * k_global_scale * log2(e)
  float out_scale;
  void* out;                               // [B, Hq, D] bf16 (or fp32 when out_f32)
  int out_f32;
  float* o_part; float* l_part; float* m_part;   // [splits, B, Hq, (D)]
  uint8_t* q_pack; uint8_t* q_sf;          // optional copies of the quantised query
  int splits, q_residue, stages;
  int32_t* status;
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

template <int D>
struct Cfg {
  static constexpr int kKSteps = D / 16;            // QK k-steps
  static constexpr int kNTiles = D / 8;             // PV n-tiles
  static constexpr int kRowBytes = D / 2;
  static constexpr int kSfPerRow = D / 16;
  static constexpr int kCodesBytes = kChunk * kRowBytes;
  static constexpr int kSfBytes = kChunk * kSfPerRow;
  static constexpr int kStageBytes = 2 * (kCodesBytes + kSfBytes);
  static constexpr int kQFragBytes = kKSteps * 32 * 16;
};

template <int D>
__global__ void __launch_bounds__(kWarps * 32) resattn_decode_kernel(const AttnParams p) {
  using C = Cfg<D>;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bars[kWarps][8];
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tq = lane & 3, nq = lane >> 2;
  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int G = p.group;

  uint4* q_frag = reinterpret_cast<uint4*>(smem);                       // [kKSteps][32] A fragments
  uint8_t* stage_base = smem + C::kQFragBytes + warp * p.stages * C::kStageBytes;

  if (threadIdx.x == 0) abort_flag = 0;
  if (lane == 0) {
    for (int s = 0; s < p.stages; ++s) mbar_init(smem_u32(&bars[warp][s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // zero the fragment area (rows of heads >= G and, without residue, rows 8-15 stay zero)
  for (int i = threadIdx.x; i < C::kQFragBytes / 16; i += blockDim.x) q_frag[i] = make_uint4(0, 0, 0, 0);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __syncthreads();

  // ---------------------------------------------------------------- query prologue
  // thread (g, blk) quantises one 16-block of head g to NVFP4 + NVFP4 residue (global scale 1)
  // and scatters the dequantised FP16 values into mma A-fragment order:
  //   value d of head g -> k-step s, lane g*4+tq, register {a0|a2} (base) / {a1|a3} (residue)
  //   with d = (D/4)*tq + 4*s + e, e in 0..3  (the same permutation is applied to K below)
  if (threadIdx.x < G * C::kSfPerRow) {
    const int g = threadIdx.x / C::kSfPerRow, blk = threadIdx.x % C::kSfPerRow;
    float v[16];
    load16(p.q + (int64_t(b) * p.hq + hkv * G + g) * D + blk * 16, v);
    BlockQ bq = quant_mext16(v, 1.0f, 1.0f);
    const float sfb = decode_e4m3(bq.sf), sfr = decode_e4m3(bq.sf_res);
    __half* qh = reinterpret_cast<__half*>(smem);
    const uint32_t bc[2] = {bq.base.x, bq.base.y}, rc[2] = {bq.res.x, bq.res.y};
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      float hb[8], hr[8];
      e2m1x8_to_float(bc[w], hb);
      e2m1x8_to_float(rc[w], hr);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int d = blk * 16 + w * 8 + i;
        const int t = d / (D / 4), within = d % (D / 4), s = within >> 2, e = within & 3;
        const int base_idx = ((s * 32 + g * 4 + t) * 4 + (e >> 1) * 2) * 2 + (e & 1);   // in halves
        qh[base_idx] = __float2half_rn(hb[i] * sfb);
        if (p.q_residue) qh[base_idx + 2] = __float2half_rn(hr[i] * sfr);               // a1 / a3
      }
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
  __syncthreads();

  // ---------------------------------------------------------------- this CTA's chunk range
  const int L = min(max(__ldg(p.seq_lens + b), 0), int(p.bt_stride) * p.page_size);
  const int n_chunks = (L + kChunk - 1) / kChunk;
  const int per_split = (n_chunks + p.splits - 1) / p.splits;
  const int c_begin = min(split * per_split, n_chunks);
  const int c_end = min(c_begin + per_split, n_chunks);
  const int my_chunks = c_end > c_begin + warp ? (c_end - c_begin - warp + kWarps - 1) / kWarps : 0;
  const int32_t* bt = p.block_tables + int64_t(b) * p.bt_stride;

  auto issue = [&](int i) {     // lane 0: fill stage i % stages with this warp's i-th chunk
    const int chunk = c_begin + warp + i * kWarps;
    const int t0 = chunk * kChunk;
    int64_t page = __ldg(bt + t0 / p.page_size);
    page = page < 0 ? 0 : (page >= p.num_pages ? p.num_pages - 1 : page);
    const int64_t row = (page * p.hkv + hkv) * p.page_size + (t0 % p.page_size);
    uint8_t* st = stage_base + (i % p.stages) * C::kStageBytes;
    const uint32_t bar = smem_u32(&bars[warp][i % p.stages]);
    mbar_expect_tx(bar, C::kStageBytes);
    bulk_load_1d(smem_u32(st), p.k_data + row * C::kRowBytes, C::kCodesBytes, bar);
    bulk_load_1d(smem_u32(st + C::kCodesBytes), p.v_data + row * C::kRowBytes, C::kCodesBytes, bar);
    bulk_load_1d(smem_u32(st + 2 * C::kCodesBytes), p.k_sf + row * C::kSfPerRow, C::kSfBytes, bar);
    bulk_load_1d(smem_u32(st + 2 * C::kCodesBytes + C::kSfBytes), p.v_sf + row * C::kSfPerRow, C::kSfBytes, bar);
  };
  if (lane == 0)
    for (int i = 0; i < min(my_chunks, p.stages); ++i) issue(i);

  // query fragments: registers for D = 128, re-read from shared memory for D = 256
  uint32_t qreg[D == 128 ? C::kKSteps : 1][4];
  if constexpr (D == 128) {
#pragma unroll
    for (int s = 0; s < C::kKSteps; ++s) {
      uint4 f = q_frag[s * 32 + lane];
      qreg[s][0] = f.x; qreg[s][1] = f.y; qreg[s][2] = f.z; qreg[s][3] = f.w;
    }
  }

  float oacc[C::kNTiles][4];
#pragma unroll
  for (int j = 0; j < C::kNTiles; ++j) oacc[j][0] = oacc[j][1] = oacc[j][2] = oacc[j][3] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;     // row nq (head g = nq), log2 domain
  bool alive = true;

  for (int i = 0; i < my_chunks && alive; ++i) {
    const int stg = i % p.stages;
    const int chunk = c_begin + warp + i * kWarps;
    const int t0 = chunk * kChunk;
    const int valid = min(L - t0, kChunk);
    // every lane polls the stage barrier; the warp takes one decision
    const bool got = mbar_wait(smem_u32(&bars[warp][stg]), (i / p.stages) & 1, &abort_flag);
    if (!__all_sync(0xffffffffu, got)) { alive = false; break; }
    const uint8_t* st = stage_base + stg * C::kStageBytes;
    const uint8_t* kc = st;
    const uint8_t* vc = st + C::kCodesBytes;
    const uint8_t* ksf = st + 2 * C::kCodesBytes;
    const uint8_t* vsf = ksf + C::kSfBytes;

    // ------------------------------------------------ S = K . (q + r)^T for 2 x 8 tokens
    float sacc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
      const int row = nt * 8 + nq;
      // this lane's quarter of the token row: D/4 codes = D/8 bytes, D/64 scale bytes
      constexpr int kWords = D / 32;                       // 32-bit words per lane
      uint32_t w[kWords];
      if constexpr (D == 128) {
        uint4 t = *reinterpret_cast<const uint4*>(kc + row * C::kRowBytes + tq * 16);
        w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
      } else {
        const uint4* src = reinterpret_cast<const uint4*>(kc + row * C::kRowBytes + tq * 32);
        uint4 t0v = src[0], t1v = src[1];
        w[0] = t0v.x; w[1] = t0v.y; w[2] = t0v.z; w[3] = t0v.w;
        w[4] = t1v.x; w[5] = t1v.y; w[6] = t1v.z; w[7] = t1v.w;
      }
      __half2 sc[D / 64];
#pragma unroll
      for (int u = 0; u < D / 64; ++u) {
        __half h = e4m3_to_half(ksf[row * C::kSfPerRow + tq * (D / 64) + u]);
        sc[u] = __half2(h, h);
      }
#pragma unroll
      for (int s = 0; s < C::kKSteps; ++s) {
        const uint32_t bits = (w[s >> 1] >> (16 * (s & 1))) & 0xFFFFu;   // 4 codes of this k-step
        const __half2 scale = sc[s >> 2];
        const uint32_t b0 = h2_bits(__hmul2(e2m1x2_to_half2(bits & 0xFFu), scale));
        const uint32_t b1 = h2_bits(__hmul2(e2m1x2_to_half2(bits >> 8), scale));
        if constexpr (D == 128) {
          mma_f16(sacc[nt], qreg[s], b0, b1);
        } else {
          uint4 f = q_frag[s * 32 + lane];
          const uint32_t a[4] = {f.x, f.y, f.z, f.w};
          mma_f16(sacc[nt], a, b0, b1);
        }
      }
    }
    // fold residue rows (8-15) onto base rows (0-7): both live in this thread
    float sv[4];
    sv[0] = (sacc[0][0] + sacc[0][2]) * p.score_scale_log2;   // token 2tq
    sv[1] = (sacc[0][1] + sacc[0][3]) * p.score_scale_log2;   // token 2tq+1
    sv[2] = (sacc[1][0] + sacc[1][2]) * p.score_scale_log2;   // token 8+2tq
    sv[3] = (sacc[1][1] + sacc[1][3]) * p.score_scale_log2;   // token 9+2tq
    if (valid < kChunk) {
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
      for (int j = 0; j < C::kNTiles; ++j) { oacc[j][0] *= f; oacc[j][1] *= f; }
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

    // ------------------------------------------------ O += P . V
    // lane (tq, nq) owns token rows {2tq, 2tq+1, 2tq+8, 2tq+9} and the D/8 head-dim columns
    // d = (D/8)*nq + j (one 16-wide (or two) scale block(s)); n-tile j, column nq <-> d
    constexpr int kVWords = D / 64;                         // 32-bit words per row per lane
    uint32_t vw[4][kVWords];
    __half vs[4][D / 128];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int row = 2 * tq + (r & 1) + (r >> 1) * 8;
      const bool ok = row < valid;
      if constexpr (D == 128) {
        uint2 t = ok ? *reinterpret_cast<const uint2*>(vc + row * C::kRowBytes + nq * 8) : make_uint2(0, 0);
        vw[r][0] = t.x; vw[r][1] = t.y;
      } else {
        uint4 t = ok ? *reinterpret_cast<const uint4*>(vc + row * C::kRowBytes + nq * 16) : make_uint4(0, 0, 0, 0);
        vw[r][0] = t.x; vw[r][1] = t.y; vw[r][2] = t.z; vw[r][3] = t.w;
      }
#pragma unroll
      for (int u = 0; u < D / 128; ++u)
        vs[r][u] = ok ? e4m3_to_half(vsf[row * C::kSfPerRow + nq * (D / 128) + u]) : __half(0.f);
    }
#pragma unroll
    for (int j = 0; j < C::kNTiles; j += 2) {
      const int word = j >> 3, sh = (j & 7) * 4;            // byte j/2 of the lane's row slice
      const int blk = j >> 4;                               // scale block inside the slice
      const __half2 s01 = __halves2half2(vs[0][blk], vs[1][blk]);
      const __half2 s89 = __halves2half2(vs[2][blk], vs[3][blk]);
      const uint32_t x0 = h2_bits(e2m1x2_to_half2((vw[0][word] >> sh) & 0xFFu));   // row 2tq  : d, d+1
      const uint32_t x1 = h2_bits(e2m1x2_to_half2((vw[1][word] >> sh) & 0xFFu));   // row 2tq+1
      const uint32_t x8 = h2_bits(e2m1x2_to_half2((vw[2][word] >> sh) & 0xFFu));
      const uint32_t x9 = h2_bits(e2m1x2_to_half2((vw[3][word] >> sh) & 0xFFu));
      // regroup (d, d+1) pairs of two tokens into (token, token+1) pairs of one column
      const uint32_t b0_lo = h2_bits(__hmul2(bits_h2(__byte_perm(x0, x1, 0x5410)), s01));
      const uint32_t b0_hi = h2_bits(__hmul2(bits_h2(__byte_perm(x0, x1, 0x7632)), s01));
      const uint32_t b1_lo = h2_bits(__hmul2(bits_h2(__byte_perm(x8, x9, 0x5410)), s89));
      const uint32_t b1_hi = h2_bits(__hmul2(bits_h2(__byte_perm(x8, x9, 0x7632)), s89));
      mma_f16(oacc[j], pa, b0_lo, b1_lo);
      mma_f16(oacc[j + 1], pa, b0_hi, b1_hi);
    }

    // stage consumed by every lane -> refill it
    __syncwarp();
    if (lane == 0 && i + p.stages < my_chunks) issue(i + p.stages);
  }

  // ---------------------------------------------------------------- merge the four warps
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  __syncthreads();                                           // pipeline memory is free now
  float* o_w = reinterpret_cast<float*>(smem + C::kQFragBytes);            // [warp][8][D]
  float* m_w = o_w + kWarps * 8 * D;                                          // [warp][8]
  float* l_w = m_w + kWarps * 8;
#pragma unroll
  for (int j = 0; j < C::kNTiles; ++j) {
    // accumulator columns 2tq / 2tq+1 of n-tile j are head-dim (D/8)*(2tq) + j and (D/8)*(2tq+1) + j
    o_w[(warp * 8 + nq) * D + (D / 8) * (2 * tq) + j] = oacc[j][0];
    o_w[(warp * 8 + nq) * D + (D / 8) * (2 * tq + 1) + j] = oacc[j][1];
  }
  if (tq == 0) {
    m_w[warp * 8 + nq] = m_run;
    l_w[warp * 8 + nq] = l_run;
  }
  __syncthreads();
  const bool failed = abort_flag != 0;
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, m_w[w * 8 + g]);
    float o = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = m_w[w * 8 + g];
      const float f = mw == -INFINITY ? 0.f : fast_exp2(mw - mm);
      o += f * o_w[(w * 8 + g) * D + d];
      l += f * l_w[w * 8 + g];
    }
    const int head = hkv * G + g;
    if (p.splits == 1) {
      const float r = l > 0.f ? p.out_scale / l : 0.f;
      const int64_t oi = (int64_t(b) * p.hq + head) * D + d;
      if (p.out_f32) static_cast<float*>(p.out)[oi] = o * r;
      else static_cast<__nv_bfloat16*>(p.out)[oi] = __float2bfloat16_rn(o * r);
    } else {
      const int64_t slot = (int64_t(split) * p.batch + b) * p.hq + head;
      p.o_part[slot * D + d] = o;
      if (d == 0) {
        p.l_part[slot] = l;
        p.m_part[slot] = mm;
      }
    }
  }
  if (failed && threadIdx.x == 0 && p.status) atomicExch(p.status, 1 + int(blockIdx.z));
  asm volatile("griddepcontrol.launch_dependents;");
}

// out[b, h, :] = sum_s 2^(m_s - m) o_s / sum_s 2^(m_s - m) l_s * out_scale, splits in order
__global__ void resattn_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ l_part,
                                     const float* __restrict__ m_part, void* __restrict__ out, int out_f32,
                                     int splits, int64_t rows, int d, float out_scale) {
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
      o += (ms == -INFINITY ? 0.f : fast_exp2(ms - mm)) * o_part[(s * rows + row) * d + c];
    }
    if (out_f32) static_cast<float*>(out)[row * d + c] = o * r;
    else static_cast<__nv_bfloat16*>(out)[row * d + c] = __float2bfloat16_rn(o * r);
  }
}

template <int D>
int launch_decode(const AttnParams& p, cudaStream_t st) {
  using C = Cfg<D>;
  const int merge_bytes = (kWarps * 8 * D + 2 * kWarps * 8) * 4;
  int pipe = kWarps * p.stages * C::kStageBytes;
  const int smem = C::kQFragBytes + (pipe > merge_bytes ? pipe : merge_bytes);
  static bool attr_done = false;
  if (!attr_done) {
    RI_CUDA(cudaFuncSetAttribute(resattn_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
    attr_done = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.splits, p.hkv, p.batch);
  cfg.blockDim = dim3(kWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cuda_status(cudaLaunchKernelEx(&cfg, resattn_decode_kernel<D>, p), "resattn decode launch");
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
                                 float score_scale, float out_scale, void* out, int out_dtype, uint8_t* q_pack,
                                 int64_t q_pack_bytes, uint8_t* q_sf, int64_t q_sf_bytes, int splits,
                                 void* workspace, int64_t workspace_bytes, int q_residue, int32_t* status,
                                 void* stream) {
  RI_CHECK_ARG(head_dim == 128 || head_dim == 256, "ResAttn supports head_dim=128 or 256");
  RI_CHECK_ARG(out_dtype == RI_DTYPE_BF16 || out_dtype == RI_DTYPE_F32, "output must be bf16");
  RI_CHECK_ARG(num_kv_heads > 0 && num_q_heads % num_kv_heads == 0, "H_q=%d must be divisible by H_kv=%d",
               num_q_heads, num_kv_heads);
  const int group = num_q_heads / num_kv_heads;
  RI_CHECK_ARG(group == 4 || group == 6 || group == 8,
               "decode residue Q8/Q16 supports logical GQA ratios (4, 6, 8), got %d", group);
  RI_CHECK_ARG(page_size >= 16 && page_size % 16 == 0, "page size must be a multiple of 16, got %d", page_size);
  RI_CHECK_ARG(batch >= 0 && num_pages > 0 && bt_stride >= 1, "bad batch / page pool / block table");
  RI_CHECK_ARG(splits >= 1 && splits <= 256, "splits must be in [1, 256]");
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
  p.score_scale_log2 = score_scale * kLog2e;
  p.out_scale = out_scale;
  p.out = out;
  p.out_f32 = out_dtype == RI_DTYPE_F32;
  p.q_pack = q_pack; p.q_sf = q_sf;
  p.splits = splits; p.q_residue = q_residue; p.status = status;
  p.stages = head_dim == 128 ? 6 : 4;
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
  s = head_dim == 128 ? launch_decode<128>(p, st) : launch_decode<256>(p, st);
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
                                          (const float*)p.m_part, p.out, p.out_f32, splits, rows, head_dim, out_scale),
                       "resattn merge launch");
  }
  return RI_OK;
}
