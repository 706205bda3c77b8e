// ResAttn decode with both products on the tensor cores (head_dim 128 and 256).  Included by resattn.cu inside
// namespace ri::<anon>::tcattn (it uses that file's AttnParams, cp_async16, swz_off, fast_exp2, ...).
//
//   S^T[128 tokens x 16] = K . Qpack^T     tcgen05.mma kind::mxf4nvf4.block_scale, K codes and E4M3 scales
//                                          as stored (rows 0-7 of Qpack: NVFP4 heads, rows 8-15: residues)
//   O^T[128 d x 16]     += V^T . P         tcgen05.mma kind::f16: V^T is the M-major A operand, written to
//                                          shared memory as FP16 (code x block scale, exact) by the
//                                          conversion warps; P (FP16) is the K-major B operand written
//                                          by the softmax warps; FP32 accumulator in tensor memory
//
// One CTA per (KV split, KV head, sequence), tiles of 128 tokens.  head_dim 128: two CTAs of 21 warps per SM;
// head_dim 256: one CTA of 29 warps (its FP16 V tile is 64 KB).  Roles:
//   softmax     eight warps, warp (q, hh): tokens 32 q .. 32 q + 31 of the tile (tensor-memory lane = token),
//               heads 4 hh .. 4 hh + 3.  The running maximum of a head is shared by the CTA and only raised
//               when a score exceeds it by more than 2^8 (then the accumulators in tensor memory are
//               rescaled); row sums stay per thread until the end.  (Four warps with eight heads per thread
//               measured 7-9 % slower: the softmax of a tile is the longest dependency chain of the CTA.)
//   MMA         one warp issues every MMA (scores of tile i+1 before the P.V of tile i), copies the K block
//               scales of a tile from shared to tensor memory (tcgen05.cp) and owns tensor memory
//   producers   four warps of cp.async: K codes and V codes in the operand swizzle of K, V scales as
//               stored, K scales in the layout of the tcgen05.cp 32x128b copy
//   conversion  8 / 16 warps: NVFP4 codes x E4M3 scale -> FP16, written in the 128-byte-swizzled M-major
//               operand layout; rows past the end of the sequence are written as zeros
// In every multi-warp role ONE lane polls the mbarriers and publishes its decision in shared memory;
// the other warps of the role wait on a named barrier.  Polling lanes in every warp took half of all
// issued instructions (measured: 1.6 -> 2.5 TB/s from this change alone).  Every mbarrier wait is
// bounded; the decision slot makes all warps of a role leave their loop together on expiry.

// O^T accumulators: the eight P.V MMAs of a tile (16 tokens each) add into eight different accumulators,
// 16 columns apart, which are summed at the end (head_dim 256: two sets, one per 128 output rows)
constexpr int kPvColO = 128;
constexpr int kPvOffMisc = 3072;                  // running maxima, rescale factors, flags
// P: K-major B operand without swizzle.  A core matrix is 8 rows (heads) x 16 bytes (8 tokens); the
// core matrices of consecutive 8-token groups are 144 bytes apart (not 128: the softmax warps then
// write without bank conflicts).  Two buffers of one 8-row group each, followed by a group of zeros
// that both use as rows 8-15.
constexpr int kPvPLbo = 144;
constexpr int kPvPGroup = 16 * kPvPLbo;           // 2304 bytes: one 8-row group over 128 tokens
constexpr int kPvOffP = 4096;
constexpr int kPvOffV = 11264;                    // [D/64 d-blocks][128 tokens][64 d] FP16, 128B swizzle, M-major
// head_dim 128: two CTAs of 21 warps per SM; head_dim 256: one CTA of 29 warps (the FP16 V tile is 64 KB)
template <int D, bool F8 = false>
struct PvCfg {
  static constexpr int kSoft = 8;                                     // softmax warps (4 heads per thread)
  static constexpr int kHpt = 32 / kSoft;                             // heads a softmax thread handles
  static constexpr int kProd = 4;                                     // copy producer warps, 128 / kProd rows of a tile each
  static constexpr int kConv = D == 128 ? 8 : 16;                     // conversion warps
  static constexpr int kVBufs = 2;                                    // expanded V tiles in flight
  static constexpr int kStages = F8 ? 3 : 2;                          // copy pipeline stages (the one-byte V tile leaves room for a third)
  static constexpr int kCtasPerSm = D == 128 ? 2 : 1;
  static constexpr int kDBlocks = D / 64;                             // 64-wide blocks of the head dimension
  static constexpr int kHalves = D / 128;                             // 128-row halves of O^T (M of one MMA)
  static constexpr int kAccs = F8 ? 4 : 8;                            // P.V MMAs (and accumulators) per tile and half: K = 32 / 16 tokens
  static constexpr int kVBytes = 128 * D * (F8 ? 1 : 2);
  static constexpr int kVStride = kVBytes;
  static constexpr int kHeaderBytes = kPvOffV + kVBufs * kVBytes;      // a multiple of 1024
  static constexpr int kThreads = (kSoft + 1 + kProd + kConv) * 32;
  static constexpr int kTmemCols = D == 128 ? 256 : 512;
  static constexpr int kSmemBytes = kHeaderBytes + kStages * TCfg<D>::kStageBytes + 1024;
};

__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_f8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// shared-memory matrix descriptor with explicit leading / stride byte offsets (sm_100 encoding)
__device__ __forceinline__ uint64_t desc_full(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type) {
  return uint64_t((saddr & 0x3FFFFu) >> 4) | (uint64_t(lbo_bytes >> 4) << 16) | (uint64_t(sbo_bytes >> 4) << 32) |
         (uint64_t(1) << 46) | (uint64_t(layout_type) << 61);
}
__device__ __forceinline__ void tmem_ld4f(uint32_t taddr, float (&v)[4]) {   // 32 lanes x 4 columns, waits for the data
  uint32_t r0, r1, r2, r3;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];\n\ttcgen05.wait::ld.sync.aligned;"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(taddr) : "memory");
  v[0] = __uint_as_float(r0); v[1] = __uint_as_float(r1); v[2] = __uint_as_float(r2); v[3] = __uint_as_float(r3);
}
__device__ __forceinline__ void tmem_st16f(uint32_t taddr, const float (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])) : "memory");
}

// Split-KV merge, fused into the decode kernel:
//   out = sum_s 2^(m_s - m) o_s / sum_s 2^(m_s - m) l_s * out_scale
// combined in split order, so the result does not depend on who merges or when.  Two carriers for the partials:
// global memory with tickets (merge_splits_last_cta) and the shared memory of a thread-block cluster
// (merge_splits_cluster).  Both do the same arithmetic in the same order, so they give the same bits; this is the
// body of the cluster form, with the loads as parameters.
// `scratch` is shared memory of this CTA: [0, 8 D) floats hold the output staging (or, in the cluster form, this
// CTA's own partial o), then 16 floats (the cluster form's l and m), then the weights [splits][8] and [8] 1 / l.
// The thread with index `first` (of `step` in all) handles the (head, column) pairs first, first + step, ...
constexpr int kMergeWeightsOff = 16;                         // floats between the o staging and the weights
template <int D, class LoadLM, class LoadO>
__device__ __forceinline__ void merge_partials(const AttnParams& p, int b, int hkv, float* scratch, int first, int step,
                                               LoadLM load_lm, LoadO load_o) {
  const int G = p.group;
  float* w_sh = scratch + 8 * D + kMergeWeightsOff;          // [splits][8] weights 2^(m_s - m), then [8] 1 / l
  float* r_sh = w_sh + p.splits * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < G) {                                            // one warp per head: maximum, weights, row sum
    // every lane takes the splits s = lane, lane + 32, ...: all loads of a pass are in flight together.  The
    // row sum is a fixed tree over the lanes (it depends on the split count only, never on arrival order).
    float mm = -INFINITY;
    for (int s = lane; s < p.splits; s += 32) {
      float ms, ls;
      load_lm(s, warp, ms, ls);
      mm = fmaxf(mm, ms);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
    float l = 0.f;
    for (int s = lane; s < p.splits; s += 32) {
      float ms, ls;
      load_lm(s, warp, ms, ls);
      const float w = ms == -INFINITY ? 0.f : fast_exp2(ms - mm);
      w_sh[s * 8 + warp] = w;
      l += w * ls;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) r_sh[warp] = l > 0.f ? p.out_scale / l : 0.f;
  }
  __syncthreads();
  for (int idx = first; idx < G * D; idx += step) {
    const int g = idx / D, c = idx - g * D;
    const int head = hkv * G + g;
    float o = 0.f;
    for (int s0 = 0; s0 < p.splits; s0 += 8) {               // eight loads in flight, then added in split order
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int s = s0 + j;
        v[j] = (s < p.splits && w_sh[s * 8 + g] != 0.f) ? load_o(s, g, c) : 0.f;   // empty partials hold no data
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j < p.splits) o += w_sh[(s0 + j) * 8 + g] * v[j];
    }
    const float v = o * r_sh[g];
    const int64_t oi = (int64_t(b) * p.hq + head) * D + c;
    if (p.out_nvfp4) scratch[g * D + c] = v;
    else if (p.out_f32) static_cast<float*>(p.out)[oi] = v;
    else static_cast<__nv_bfloat16*>(p.out)[oi] = __float2bfloat16_rn(v);
  }
}

// Global-memory carrier.  Every CTA of a (sequence, KV head) publishes its partial (o, l, m) and takes a ticket;
// the CTA that draws the last ticket (nobody waits for anybody) combines the partials of all splits.
// Returns true in the CTA that merged (the caller then packs the NVFP4 output if that is asked for).
// The same arithmetic in the same order as merge_partials, written out: sharing that body cost this hot
// instantiation register spills.
template <int D>
__device__ __forceinline__ bool merge_splits_last_cta(const AttnParams& p, int b, int hkv, float* scratch, int* flag_sh) {
  const int G = p.group;
  // every thread's partial stores are ordered before its arrival at the barrier; the ticket holder's fence
  // publishes them device-wide before the ticket and orders the merging CTA's reads after it
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* counter = p.split_counter + b * p.hkv + hkv;
    const int ticket = atomicAdd(counter, 1);
    const int last = ticket == p.splits - 1;
    if (last) *counter = 0;                                  // ready for the next call
    __threadfence();
    *flag_sh = last;
  }
  __syncthreads();
  if (!*flag_sh) return false;
  float* w_sh = scratch + 8 * D;                             // [splits][8] weights 2^(m_s - m), then [8] 1 / l
  float* r_sh = w_sh + p.splits * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < G) {                                            // one warp per head: maximum, weights, row sum
    const int head = hkv * G + warp;
    float mm = -INFINITY;
    for (int s = lane; s < p.splits; s += 32) mm = fmaxf(mm, __ldcg(p.m_part + (int64_t(s) * p.batch + b) * p.hq + head));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
    // every lane takes the splits s = lane, lane + 32, ...: all loads of a pass are in flight together.  The
    // row sum is a fixed tree over the lanes (it depends on the split count only, never on arrival order).
    float l = 0.f;
    for (int s = lane; s < p.splits; s += 32) {
      const int64_t slot = (int64_t(s) * p.batch + b) * p.hq + head;
      const float ms = __ldcg(p.m_part + slot), ls = __ldcg(p.l_part + slot);
      const float w = ms == -INFINITY ? 0.f : fast_exp2(ms - mm);
      w_sh[s * 8 + warp] = w;
      l += w * ls;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) r_sh[warp] = l > 0.f ? p.out_scale / l : 0.f;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, c = idx - g * D;
    const int head = hkv * G + g;
    const float* src = p.o_part + (int64_t(b) * p.hq + head) * D + c;      // split s lies s * stride further
    const int64_t stride = int64_t(p.batch) * p.hq * D;
    float o = 0.f;
    for (int s0 = 0; s0 < p.splits; s0 += 8) {               // eight loads in flight, then added in split order
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int s = s0 + j;
        v[j] = (s < p.splits && w_sh[s * 8 + g] != 0.f) ? __ldcg(src + s * stride) : 0.f;   // empty partials hold no data
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j < p.splits) o += w_sh[(s0 + j) * 8 + g] * v[j];
    }
    const float v = o * r_sh[g];
    const int64_t oi = (int64_t(b) * p.hq + head) * D + c;
    if (p.out_nvfp4) scratch[g * D + c] = v;
    else if (p.out_f32) static_cast<float*>(p.out)[oi] = v;
    else static_cast<__nv_bfloat16*>(p.out)[oi] = __float2bfloat16_rn(v);
  }
  __syncthreads();
  return true;
}

// Cluster carrier: the CTAs of a (sequence, KV head) form one thread-block cluster (cluster rank = split), every
// CTA leaves its partial in its own shared memory -- o at scratch[0, 8 D), l at [8 D, 8 D + 8), m behind it -- and
// after one cluster barrier each CTA combines a 1 / splits share of the (head, column) pairs, reading its peers'
// partials through distributed shared memory; a second barrier keeps every CTA's memory alive until its peers
// have read it.  No global round trip, no ticket, no workspace.  The barrier is the hardware's: every thread of
// every CTA of the cluster must reach both calls, which the kernel's two exits do unconditionally (all other
// waits of the kernel are bounded, so every CTA gets here).
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(const float* local, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}
template <int D>
__device__ __forceinline__ void merge_splits_cluster(const AttnParams& p, int b, int hkv, float* scratch, int split) {
  cluster_barrier();                                         // everybody's partial is in place
  const float* l_loc = scratch + 8 * D;
  merge_partials<D>(p, b, hkv, scratch, split * int(blockDim.x) + int(threadIdx.x), p.splits * int(blockDim.x),
      [=](int s, int g, float& ms, float& ls) {
        ls = ld_cluster_f32(l_loc + g, uint32_t(s));
        ms = ld_cluster_f32(l_loc + 8 + g, uint32_t(s));
      },
      [=](int s, int g, int c) { return ld_cluster_f32(scratch + g * D + c, uint32_t(s)); });
  cluster_barrier();                                         // nobody reads this CTA's partial any more
}

// 16-value blocks of the [heads][D] staging tile -> packed NVFP4 codes + block scales of sequence b
template <int D>
__device__ __forceinline__ void pack_nvfp4_output(const AttnParams& p, int b, int hkv, const float* stage_out) {
  const int G = p.group;
  if (threadIdx.x < G * (D / 16)) {
    const int g = threadIdx.x / (D / 16), blk = threadIdx.x % (D / 16);
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = stage_out[g * D + blk * 16 + i];
    const int head = hkv * G + g, hidden = p.hq * D;
    store_nvfp4_out16(v, __ldg(p.out_gs), static_cast<uint8_t*>(p.out) + int64_t(b) * (hidden / 2), p.out_sf, b,
                      head * (D / 16) + blk, hidden);
  }
}

// CL: the cluster reducer.  An instantiation of its own, so that the ticket form carries none of its code.
template <int D, bool F8, bool CL>
__global__ void __launch_bounds__(PvCfg<D, F8>::kThreads, PvCfg<D, F8>::kCtasPerSm)
resattn_pv_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                  const __grid_constant__ AttnParams p) {
  using C = TCfg<D>;
  using PC = PvCfg<D, F8>;
  constexpr int kPvAccs = PC::kAccs;
  constexpr int kPvConv = PC::kConv, kPvVBufs = PC::kVBufs, kPvStages = PC::kStages, kThreadsPv = PC::kThreads;
  constexpr int kPvTmemCols = PC::kTmemCols, kPvVStride = PC::kVStride, kPvHeaderBytes = PC::kHeaderBytes;
  constexpr int kPvSoft = PC::kSoft, kHpt = PC::kHpt, kPvProd = PC::kProd;
  constexpr int kPvMmaWarp = kPvSoft, kPvFirstProd = kPvSoft + 1, kPvFirstConv = kPvFirstProd + kPvProd;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kPvStages];
  __shared__ __align__(8) uint64_t bar_empty[kPvStages];
  __shared__ __align__(8) uint64_t bar_sfull[2], bar_vpready[2], bar_pvdone[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;
  __shared__ int merge_flag;
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* q_op = smem;                                        // [16][64 B] swizzled FP4 codes
  uint8_t* qsf_s = smem + 2048;                                // [16][8] E4M3 scales
  float* m_sh = reinterpret_cast<float*>(smem + kPvOffMisc);   // [8] running maxima (log2 domain)
  float* f_sh = m_sh + 8;                                      // [8] rescale factors of the current tile
  float* wmax = m_sh + 16;                                     // [4 warps][8] tile maxima
  volatile int* grow = reinterpret_cast<volatile int*>(m_sh + 48);   // [2] "a maximum moved" flag by tile parity
  float* red = m_sh + 64;                                      // [4 warps][8] row-sum reduction
  volatile int* soft_go = reinterpret_cast<volatile int*>(m_sh + 100);   // [3] decisions of the polling lanes
  volatile int* conv_go = reinterpret_cast<volatile int*>(m_sh + 104);   // [2]
  volatile int* prod_go = reinterpret_cast<volatile int*>(m_sh + 108);   // [2]
  uint8_t* stage0 = smem + kPvHeaderBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int G = p.group;
  constexpr int S = kPvStages;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int L = min(max(__ldg(p.seq_lens + b), 0), int(p.bt_stride) * p.page_size);
  const int n_tiles = (L + kTile - 1) / kTile;
  const int t_begin = min(split * p.tiles_per_split, n_tiles);
  const int t_end = min(t_begin + p.tiles_per_split, n_tiles);
  const int my_tiles = t_end - t_begin;
  if (my_tiles == 0 && p.splits > 1 && !(p.q_pack && split == 0)) {
    // nothing to read for this split: publish an empty partial and, if this CTA happens to draw the last
    // ticket, merge the others' (the whole CTA takes this branch together)
    float* scratch = reinterpret_cast<float*>(smem + kPvOffV);
    if constexpr (CL) {
      if (threadIdx.x < G) {
        scratch[8 * D + threadIdx.x] = 0.f;
        scratch[8 * D + 8 + threadIdx.x] = -INFINITY;
      }
      __syncthreads();
      merge_splits_cluster<D>(p, b, hkv, scratch, split);
    } else {
      if (threadIdx.x < G) {
        const int64_t slot = (int64_t(split) * p.batch + b) * p.hq + hkv * G + threadIdx.x;
        p.l_part[slot] = 0.f;
        p.m_part[slot] = -INFINITY;
      }
      if (merge_splits_last_cta<D>(p, b, hkv, scratch, &merge_flag) && p.out_nvfp4) pack_nvfp4_output<D>(p, b, hkv, scratch);
    }
    return;
  }
  const int32_t* bt = p.block_tables + int64_t(b) * p.bt_stride;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&bar_full[s]), kPvProd * 32);
      mbar_init(smem_u32(&bar_empty[s]), kPvConv + 1);         // conversion warps + the commit of the scores' MMAs
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_sfull[s]), 1);
      mbar_init(smem_u32(&bar_vpready[s]), kPvConv + kPvSoft);   // V tile converted and P written
      mbar_init(smem_u32(&bar_pvdone[s]), 1);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kPvMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"(kPvTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // zero the query operand, its scales, the shared scalars and both P buffers (rows 8-15 of P stay zero)
  for (int i = threadIdx.x; i < kPvOffV / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (threadIdx.x < 8) m_sh[threadIdx.x] = -INFINITY;

  // ---------------------------------------------------------------- query prologue
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
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp < kPvFirstProd || warp >= kPvFirstConv)
    asm volatile("bar.sync 2, %0;" ::"n"(kThreadsPv - kPvProd * 32) : "memory");

  float l_thr[kHpt];
#pragma unroll
  for (int h = 0; h < kHpt; ++h) l_thr[h] = 0.f;

  if (warp < kPvSoft) {
    // ============================================================ softmax warps
    // Warp (q, hh): tensor-memory quarter q = tokens 32 q .. 32 q + 31 of the tile, heads kHpt hh .. + kHpt - 1.
    // Only lane 0 of warp 0 polls mbarriers; the warps then meet on a named barrier, which costs the
    // waiting warps no issue slots.
    const int q = warp & 3, hh = warp >> 2, g0 = hh * kHpt;
    const uint32_t lane_base = tmem_base + (uint32_t(q * 32) << 16);
    if (hh == 0) {
#pragma unroll
      for (int j = 0; j < C::kMma; ++j) {
        uint4 w = make_uint4(0, 0, 0, 0);
        if (lane < 16) w.x = *reinterpret_cast<const uint32_t*>(qsf_s + lane * C::kSfPerRow + 4 * j);
        tmem_st4(lane_base + kColSfb + 4 * j, w);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    // the Q scales are in tensor memory: tell the MMA warp
    tc_fence_before();
    asm volatile("bar.sync 5, %0;" ::"n"(kPvSoft * 32 + 32) : "memory");
    for (int i = 0; i < my_tiles; ++i) {
      const int sb = i & 1;
      const int tile = t_begin + i;
      if (threadIdx.x == 0) {
        soft_go[sb] = mbar_wait(smem_u32(&bar_sfull[sb]), (i >> 1) & 1, &abort_flag, 5) ? 1 : 0;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kPvSoft * 32) : "memory");
      if (!soft_go[sb]) break;                                  // the same decision in all softmax warps
      tc_fence_after();
      float s[kHpt];
      bool mine_grows = false;
      {
        const bool valid = tile * kTile + 32 * q + lane < L;
        if constexpr (kHpt == 8) {
          float r[16];
          tmem_ld16(lane_base + kColS + sb * 16, r);
#pragma unroll
          for (int h = 0; h < 8; ++h) s[h] = valid ? (r[h] + r[8 + h]) * p.score_scale_log2 : -INFINITY;
        } else {
          float r0[4], r1[4];
          tmem_ld4f(lane_base + kColS + sb * 16 + g0, r0);
          tmem_ld4f(lane_base + kColS + sb * 16 + 8 + g0, r1);
#pragma unroll
          for (int h = 0; h < 4; ++h) s[h] = valid ? (r0[h] + r1[h]) * p.score_scale_log2 : -INFINITY;
        }
        tc_fence_before();
#pragma unroll
        for (int h = 0; h < kHpt; ++h) mine_grows |= s[h] > m_sh[g0 + h] + kLazyThreshold;   // also true while the maximum is -inf
        if (__any_sync(0xffffffffu, mine_grows) && lane == 0) grow[sb] = 1;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kPvSoft * 32) : "memory");
      if (grow[sb]) {
        // ---- a maximum moved (always on the first tile): exact tile maxima, rescale the accumulators
        float mx[kHpt];
#pragma unroll
        for (int h = 0; h < kHpt; ++h) {
          mx[h] = s[h];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], o));
        }
        if (lane == 0) {
#pragma unroll
          for (int h = 0; h < kHpt; ++h) wmax[q * 8 + g0 + h] = mx[h];
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kPvSoft * 32) : "memory");
        float f[kHpt];
#pragma unroll
        for (int h = 0; h < kHpt; ++h) {
          const int g = g0 + h;
          const float old = m_sh[g];
          const float nw = fmaxf(fmaxf(old, fmaxf(wmax[g], wmax[8 + g])), fmaxf(wmax[16 + g], wmax[24 + g]));
          f[h] = old == -INFINITY ? 0.f : fast_exp2(old - nw);
          l_thr[h] *= f[h];
          mx[h] = nw;
        }
        if (i > 0) {
          // the P.V of the previous tile must have landed before the accumulators are rescaled in place
          bool got = true;
          if (lane == 0) got = mbar_wait(smem_u32(&bar_pvdone[(i - 1) & 1]), ((i - 1) >> 1) & 1, &abort_flag, 7);
          if (__all_sync(0xffffffffu, got)) {
            tc_fence_after();
#pragma unroll 1
            for (int a = 0; a < kPvAccs * PC::kHalves; ++a) {
              if constexpr (kHpt == 8) {
                float o[16];
                tmem_ld16(lane_base + kPvColO + 16 * a, o);
#pragma unroll
                for (int h = 0; h < 8; ++h) o[h] *= f[h];
                tmem_st16f(lane_base + kPvColO + 16 * a, o);
              } else {                                          // this warp's four heads = four columns of the accumulator
                float o[4];
                tmem_ld4f(lane_base + kPvColO + 16 * a + g0, o);
                tmem_st4(lane_base + kPvColO + 16 * a + g0,
                         make_uint4(__float_as_uint(o[0] * f[0]), __float_as_uint(o[1] * f[1]),
                                    __float_as_uint(o[2] * f[2]), __float_as_uint(o[3] * f[3])));
              }
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
          }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kPvSoft * 32) : "memory");   // everybody has read the old maxima
        if (q == 0) {
#pragma unroll
          for (int h = 0; h < kHpt; ++h)
            if (lane == h) m_sh[g0 + h] = mx[h];
        }
        if (threadIdx.x == 8) grow[sb] = 0;
        asm volatile("bar.sync 1, %0;" ::"n"(kPvSoft * 32) : "memory");
      }
      // ---- probabilities of this thread's token, FP16, into the K-major B operand of the P.V MMAs.
      // (The P buffer is free: the commit behind s_full(i) was issued by the same thread after the P.V
      // MMAs of tile i-2, so having seen it means those have read the buffer.)
      {
        const int t = 32 * q + lane;
        if constexpr (F8) {
          // E4M3 probabilities (the reference's choice, csrc/resattn/kernel_paged_decode.py:1958-1963); the row
          // sums keep the unrounded values, as there.  A core matrix of the 8-bit K-major operand is 8 heads x
          // 16 tokens; the core matrices of consecutive 16-token groups are kPvPLbo bytes apart.
          uint8_t* pb = smem + kPvOffP + sb * kPvPGroup + (t >> 4) * kPvPLbo + (t & 15) + g0 * 16;
          float pv[kHpt];
#pragma unroll
          for (int h = 0; h < kHpt; ++h) {
            pv[h] = fast_exp2(s[h] - m_sh[g0 + h]);            // 0 for tokens past the end (s = -inf)
            l_thr[h] += pv[h];
          }
#pragma unroll
          for (int h = 0; h < kHpt; h += 2) {
            uint16_t two;                                      // low byte: first operand of the pair
            asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(two) : "f"(pv[h + 1]), "f"(pv[h]));
            pb[h * 16] = uint8_t(two & 0xFF);
            pb[(h + 1) * 16] = uint8_t(two >> 8);
          }
        } else {
        __half* pb = reinterpret_cast<__half*>(smem + kPvOffP + sb * kPvPGroup + (t >> 3) * kPvPLbo) + (t & 7) + g0 * 8;
#pragma unroll
        for (int h = 0; h < kHpt; ++h) {
          const float pv = fast_exp2(s[h] - m_sh[g0 + h]);     // 0 for tokens past the end (s = -inf)
          l_thr[h] += pv;
          pb[h * 8] = __float2half_rn(pv);
        }
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_vpready[sb]));
    }
  } else if (warp == kPvMmaWarp) {
    // ============================================================ MMA issuer
    // One thread issues everything, the scores of tile i+1 before the P.V of tile i.  (Two issuing
    // warps measured 4-7 % slower, twice, and with one the commit behind s_full(i) also covers the P.V of tile i-2.)
    const uint32_t idesc_qk = (1u << 7) | (1u << 10) | (uint32_t(16 >> 3) << 17) | (uint32_t(kTile >> 4) << 24);
    // kind::f16: FP32 accumulate (bits 4-5 = 1), FP16 x FP16, A M-major (bit 15), B K-major, N = 16, M = 128
    const uint32_t idesc_pv = (1u << 4) | (1u << 15) | (uint32_t(16 >> 3) << 17) | (uint32_t(128 >> 4) << 24);
    const uint64_t bq_desc = desc_kmajor(smem_u32(q_op), C::kSbo, C::kLayout);
    bool alive = true;
    asm volatile("bar.sync 5, %0;" ::"n"(kPvSoft * 32 + 32) : "memory");   // the Q scales are in tensor memory
    // Scores of tile i.  Its S buffer and scale set were last used by tile i-2, whose softmax finished
    // before the P.V of tile i-2 was issued (by this thread, earlier).
    auto issue_qk = [&](int i) {
      const int stg = i % S, sb = i & 1;
      bool got = true;
      if (lane == 0) got = mbar_wait(smem_u32(&bar_full[stg]), (i / S) & 1, &abort_flag, 3);
      if (!__all_sync(0xffffffffu, got)) { alive = false; return; }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // cp.async data -> tensor-core reads
      tc_fence_after();
      if (elect_one()) {
        const uint32_t st_addr = smem_u32(stage0 + stg * C::kStageBytes);
        const uint64_t a_desc = desc_kmajor(st_addr, C::kSbo, C::kLayout);
        // K block scales: the producers store them as [64-column group][32 rows][4 quarters][4 bytes],
        // the layout of one 32x128b copy per MMA
#pragma unroll
        for (int j = 0; j < C::kMma; ++j)
          tmem_cp_sf(tmem_base + kColSfa + sb * 16 + 4 * j, desc_sf(st_addr + C::kOffKsf + j * 512));
#pragma unroll
        for (int j = 0; j < C::kMma; ++j)
          mma_fp4<false>(tmem_base + kColS + sb * 16, a_desc + uint64_t(2 * j), bq_desc + uint64_t(2 * j), idesc_qk,
                         tmem_base + kColSfa + sb * 16 + 4 * j, tmem_base + kColSfb + 4 * j, j > 0 ? 1u : 0u);
        mma_commit(smem_u32(&bar_sfull[sb]));
        mma_commit(smem_u32(&bar_empty[stg]));                 // the K codes of the stage have been read
      }
      __syncwarp();
    };
    auto issue_pv = [&](int i) -> bool {
      const int vb = i & 1;
      bool got = true;
      if (lane == 0) got = mbar_wait(smem_u32(&bar_vpready[vb]), (i >> 1) & 1, &abort_flag, 9);
      if (!__all_sync(0xffffffffu, got)) return false;
      tc_fence_after();
      if (elect_one()) {
        // A = V^T: M-major, 128-byte swizzle: 64-d blocks 16 KB apart (leading offset), 8-token groups 1 KB apart
        const uint32_t va = smem_u32(smem + kPvOffV + (kPvVBufs == 2 ? vb * kPvVStride : 0));
        // B = P: K-major, no swizzle: 8-token core matrices kPvPLbo apart along K; rows 8-15 are the zero group
        const uint32_t pa = smem_u32(smem + kPvOffP + vb * kPvPGroup);
        const uint32_t p_sbo = (2 - vb) * kPvPGroup;
        if constexpr (F8) {
          // kind::f8f6f4, E4M3 x E4M3, K = 32 tokens per instruction: A = one 128-byte row per token (128 d),
          // 8-token groups 1 KB apart; B = two 16-token core matrices per instruction
          const uint32_t idesc_pv8 = (1u << 4) | (1u << 15) | (uint32_t(16 >> 3) << 17) | (uint32_t(128 >> 4) << 24);
#pragma unroll
          for (int hf = 0; hf < PC::kHalves; ++hf)
#pragma unroll
            for (int k32 = 0; k32 < kTile / 32; ++k32)
              mma_f8_ss(tmem_base + kPvColO + 16 * (hf * kPvAccs + k32),
                        desc_full(va + hf * 16384 + k32 * 4096, 16384, 1024, 2),
                        desc_full(pa + k32 * 2 * kPvPLbo, kPvPLbo, p_sbo, 0), idesc_pv8, i > 0 ? 1u : 0u);
        } else {
#pragma unroll
        for (int hf = 0; hf < PC::kHalves; ++hf)
#pragma unroll
          for (int k16 = 0; k16 < kTile / 16; ++k16)
            mma_f16_ss(tmem_base + kPvColO + 16 * (hf * kPvAccs + k16),
                       desc_full(va + hf * 2 * 16384 + k16 * 2048, 16384, 1024, 2),
                       desc_full(pa + k16 * 2 * kPvPLbo, kPvPLbo, p_sbo, 0), idesc_pv, i > 0 ? 1u : 0u);
        }
        mma_commit(smem_u32(&bar_pvdone[vb]));
      }
      __syncwarp();
      return true;
    };
    if (my_tiles > 0) issue_qk(0);
    for (int i = 0; i < my_tiles && alive; ++i) {
      if (i + 1 < my_tiles) issue_qk(i + 1);
      if (!alive || !issue_pv(i)) break;
    }
  } else if (warp < kPvFirstConv) {
    // ============================================================ copy producers
    constexpr int kCpr = C::kRowBytes / 16;
    constexpr int kRowsPerIt = 32 / kCpr;
    constexpr int kRowsW = kTile / kPvProd;                    // rows of a tile per producer warp (32 or 16)
    constexpr int kIters = kRowsW / kRowsPerIt;
    const int pw = warp - kPvFirstProd;
    const int r_lane = lane / kCpr, chn = lane % kCpr;
    const int sf_row = D == 128 ? 2 * lane : lane;             // first row of this lane's 16 scale bytes
    const bool sf_lane = D == 128 ? lane < kRowsW / 2 : lane < kRowsW;
    uint32_t k_dst[kIters];
#pragma unroll
    for (int it = 0; it < kIters; ++it) k_dst[it] = swz_off<D>(kRowsW * pw + it * kRowsPerIt + r_lane, chn * 16);
    const uint32_t sf_dst = (kRowsW * pw + sf_row) * C::kSfPerRow;
    auto lookup = [&](int i) -> int {
      if (lane >= kRowsW / 16 || i >= my_tiles) return 0;
      const int t0 = (t_begin + i) * kTile + kRowsW * pw + lane * 16;
      return t0 < L ? __ldg(bt + (p.page_shift >= 0 ? t0 >> p.page_shift : t0 / p.page_size)) : 0;
    };
    int page_next = lookup(0);
    for (int i = 0, stg = 0, ph = 0; i < my_tiles; ++i, stg = (stg + 1 == S ? 0 : stg + 1), ph ^= (stg == 0)) {
      const int tok0 = (t_begin + i) * kTile + kRowsW * pw;
      const int rows = min(max(((L - tok0) + 15) & ~15, 0), kRowsW);
      int64_t page = page_next;
      page_next = lookup(i + 1);
      page = page < 0 ? 0 : (page >= p.num_pages ? p.num_pages - 1 : page);
      const int t0 = tok0 + lane * 16;
      const int in_page = p.page_shift >= 0 ? (t0 & (p.page_size - 1)) : t0 % p.page_size;
      // a page holds [Hkv, page_size] rows of codes (and of scales); pages lie code_page_stride (sf_page_stride)
      // bytes apart, which is the dense distance for a pool of its own and the whole interleaved page for a
      // cache that keeps K codes | K scales | V codes | V scales together
      const int in_row = hkv * p.page_size + in_page;
      const int pg0 = __shfl_sync(0xffffffffu, int(page), 0), pg1 = __shfl_sync(0xffffffffu, int(page), 1);
      const int in0 = __shfl_sync(0xffffffffu, in_row, 0), in1 = __shfl_sync(0xffffffffu, in_row, 1);
      const int64_t code0 = pg0 * p.code_page_stride + int64_t(in0) * C::kRowBytes;
      const int64_t code1 = pg1 * p.code_page_stride + int64_t(in1) * C::kRowBytes;
      const int64_t sf0 = pg0 * p.sf_page_stride + int64_t(in0) * C::kSfPerRow;
      const int64_t sf1 = pg1 * p.sf_page_stride + int64_t(in1) * C::kSfPerRow;
      if (i >= S) {                                            // one lane polls, the four warps meet on a named barrier
        if (pw == 0 && lane == 0) prod_go[i & 1] = mbar_wait(smem_u32(&bar_empty[stg]), ph ^ 1, &abort_flag, 4) ? 1 : 0;
        asm volatile("bar.sync 4, %0;" ::"n"(kPvProd * 32) : "memory");
        if (!prod_go[i & 1]) break;
      }
      const uint32_t st = smem_u32(stage0 + stg * C::kStageBytes);
      if (p.tma_pages) {
        // Pages of 128 tokens (or a multiple): the K codes, the V codes and the V scales of a tile are three
        // contiguous blocks of the pool.  One thread fetches them with the copy engine: the two code blocks
        // as tiled loads that write the operand swizzle, the scales as one bulk copy.  The tile's rows
        // past the end of the sequence belong to the same page, so whole blocks are always fetched.
        if (pw == 0 && lane == 0) {
          const uint32_t full = smem_u32(&bar_full[stg]);
          mbar_expect_tx(full, 2 * C::kKBytes + C::kSfBytes);
          tma_load_3d(st, &k_map, 0, in0, pg0, full);
          tma_load_3d(st + C::kOffV, &v_map, 0, in0, pg0, full);
          bulk_load_1d(st + C::kOffVsf, p.v_sf + sf0, C::kSfBytes, full);
        }
      } else {
        const uint8_t* kg[2] = {p.k_data + code0 + chn * 16, p.k_data + code1 + chn * 16};
        const uint8_t* vg[2] = {p.v_data + code0 + chn * 16, p.v_data + code1 + chn * 16};
#pragma unroll
        for (int it = 0; it < kIters; ++it) {
          const int r = it * kRowsPerIt + r_lane;
          if (it * kRowsPerIt < rows) {
            const int sl = (it * kRowsPerIt) >> 4;
            const int off = (r & 15) * C::kRowBytes;
            cp_async16(st + k_dst[it], kg[sl] + off);
            cp_async16(st + C::kOffV + k_dst[it], vg[sl] + off);
          }
        }
        if (sf_lane && sf_row < rows) {
          cp_async16(st + C::kOffVsf + sf_dst, p.v_sf + (sf_row < 16 ? sf0 : sf1) + (sf_row & 15) * C::kSfPerRow);
        }
      }
      if (lane < rows) {                                       // K scales of token kRowsW pw + lane, 4 bytes per MMA
        const uint8_t* src = p.k_sf + (lane < 16 ? sf0 : sf1) + (lane & 15) * C::kSfPerRow;
        const int tk = kRowsW * pw + lane;
        const uint32_t dst = st + C::kOffKsf + (tk & 31) * 16 + (tk >> 5) * 4;
#pragma unroll
        for (int j = 0; j < C::kMma; ++j)
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 512 * j), "l"(src + 4 * j) : "memory");
      }
      // every producer thread arrives once per tile, when its own cp.async copies have landed; the thread
      // that armed the barrier for the copy engine's bytes has arrived with that instruction already
      if (!(p.tma_pages && pw == 0 && lane == 0))
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&bar_full[stg])) : "memory");
    }
  } else {
    // ============================================================ V conversion warps
    // warp c: tokens 32 (c / blocks) .. +31, d-block c % blocks (64 head-dim values = 32 code bytes = 4 scale blocks)
    const int cv = warp - kPvFirstConv;
    const int tok = 32 * (cv / PC::kDBlocks) + lane, dblk = cv % PC::kDBlocks;
    for (int i = 0, stg = 0, ph = 0; i < my_tiles; ++i, stg = (stg + 1 == S ? 0 : stg + 1), ph ^= (stg == 0)) {
      const int vb = i & 1;
      if (cv == 0 && lane == 0) {                              // one lane polls, the eight warps meet on a named barrier
        bool got = mbar_wait(smem_u32(&bar_full[stg]), ph, &abort_flag, 6);
        if (kPvVBufs == 2) {
          if (got && i >= 2) got = mbar_wait(smem_u32(&bar_pvdone[vb]), ((i >> 1) - 1) & 1, &abort_flag, 11);
        } else {
          if (got && i >= 1) got = mbar_wait(smem_u32(&bar_pvdone[vb ^ 1]), ((i - 1) >> 1) & 1, &abort_flag, 11);
        }
        conv_go[vb] = got ? 1 : 0;
      }
      asm volatile("bar.sync 3, %0;" ::"n"(kPvConv * 32) : "memory");
      if (!conv_go[vb]) break;
      const uint8_t* st = stage0 + stg * C::kStageBytes;
      const bool valid = (t_begin + i) * kTile + tok < L;
      uint4 c0 = make_uint4(0, 0, 0, 0), c1 = c0;
      uint32_t sfw = 0;
      if (valid) {
        // the producers store the V rows with the swizzle of the K operand (conflict-free 16-byte reads)
        const uint8_t* row = st + C::kOffV + tok * C::kRowBytes;
        const int sw = D == 128 ? (tok >> 1) & 3 : tok & 7;
        c0 = *reinterpret_cast<const uint4*>(row + (((2 * dblk) ^ sw) << 4));
        c1 = *reinterpret_cast<const uint4*>(row + (((2 * dblk + 1) ^ sw) << 4));
        sfw = *reinterpret_cast<const uint32_t*>(st + C::kOffVsf + tok * C::kSfPerRow + dblk * 4);
      }
      // The codes and scales are in registers: give the stage back before converting, so that its
      // refill (about 2600 cycles of memory latency) starts a conversion earlier.  (The arrive is a
      // release; __syncwarp orders the other lanes' loads before it.)
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_empty[stg]));
      const uint32_t words[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};   // 8 codes (= 8 d) per word
      // the four block scales of this thread's 64 values as FP16 pairs (s, s)
      uint32_t sc2[4];
      {
        uint32_t lo, hi;                                       // (s0, s1), (s2, s3) as FP16 pairs
        asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
            : "=r"(lo), "=r"(hi) : "r"(sfw));
        sc2[0] = __byte_perm(lo, 0, 0x1010); sc2[1] = __byte_perm(lo, 0, 0x3232);
        sc2[2] = __byte_perm(hi, 0, 0x1010); sc2[3] = __byte_perm(hi, 0, 0x3232);
      }
      if constexpr (F8) {
        // E4M3 V (the reference's choice, csrc/resattn/qmul4.py:45): code x block scale is exact in FP16 and is
        // rounded to E4M3 (nearest even, saturating).  One 128-byte row per token holds 128 head-dim values; this
        // thread's 64 values are the four 16-byte chunks (dblk & 1) * 4 .. + 3, one per scale block.
        const uint32_t row0 = smem_u32(smem + kPvOffV + (kPvVBufs == 2 ? vb * kPvVStride : 0) + (dblk >> 1) * 16384 +
                                       (tok >> 3) * 1024 + (tok & 7) * 128);
#pragma unroll
        for (int blk = 0; blk < 4; ++blk) {
          const __half2 s2 = bits_h2(sc2[blk]);
          uint32_t o[4];
#pragma unroll
          for (int hw = 0; hw < 2; ++hw) {
            uint32_t h0, h1, h2, h3;
            asm("{\n\t.reg .b8 a, b, c, d;\n\tmov.b32 {a, b, c, d}, %4;\n\t"
                "cvt.rn.f16x2.e2m1x2 %0, a;\n\tcvt.rn.f16x2.e2m1x2 %1, b;\n\t"
                "cvt.rn.f16x2.e2m1x2 %2, c;\n\tcvt.rn.f16x2.e2m1x2 %3, d;\n\t}"
                : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3) : "r"(words[2 * blk + hw]));
            const uint32_t p0 = h2_bits(__hmul2(bits_h2(h0), s2)), p1 = h2_bits(__hmul2(bits_h2(h1), s2));
            const uint32_t p2 = h2_bits(__hmul2(bits_h2(h2), s2)), p3 = h2_bits(__hmul2(bits_h2(h3), s2));
            asm("{\n\t.reg .b16 a, b, c, d;\n\t"
                "cvt.rn.satfinite.e4m3x2.f16x2 a, %2;\n\tcvt.rn.satfinite.e4m3x2.f16x2 b, %3;\n\t"
                "cvt.rn.satfinite.e4m3x2.f16x2 c, %4;\n\tcvt.rn.satfinite.e4m3x2.f16x2 d, %5;\n\t"
                "mov.b32 %0, {a, b};\n\tmov.b32 %1, {c, d};\n\t}"
                : "=r"(o[2 * hw]), "=r"(o[2 * hw + 1]) : "r"(p0), "r"(p1), "r"(p2), "r"(p3));
          }
          const uint32_t chunk = uint32_t(((dblk & 1) * 4 + blk) ^ (tok & 7));
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row0 + (chunk << 4)), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
        }
      } else {
      // destination row of this token in the swizzled M-major tile; chunk w goes to (w ^ (tok & 7)) << 4,
      // which is an XOR on the address because the row is 128-byte aligned
      const uint32_t dst0 = smem_u32(smem + kPvOffV + (kPvVBufs == 2 ? vb * kPvVStride : 0) + dblk * 16384 +
                                     (tok >> 3) * 1024 + (tok & 7) * 128) | ((tok & 7) << 4);
#pragma unroll
      for (int w8 = 0; w8 < 8; ++w8) {                         // one 16-byte chunk = 8 FP16 per code word
        uint32_t h0, h1, h2, h3;
        asm("{\n\t.reg .b8 a, b, c, d;\n\tmov.b32 {a, b, c, d}, %4;\n\t"
            "cvt.rn.f16x2.e2m1x2 %0, a;\n\tcvt.rn.f16x2.e2m1x2 %1, b;\n\t"
            "cvt.rn.f16x2.e2m1x2 %2, c;\n\tcvt.rn.f16x2.e2m1x2 %3, d;\n\t}"
            : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3) : "r"(words[w8]));
        const __half2 s2 = bits_h2(sc2[w8 >> 1]);
        const uint32_t o0 = h2_bits(__hmul2(bits_h2(h0), s2)), o1 = h2_bits(__hmul2(bits_h2(h1), s2));
        const uint32_t o2 = h2_bits(__hmul2(bits_h2(h2), s2)), o3 = h2_bits(__hmul2(bits_h2(h3), s2));
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst0 ^ (w8 << 4)), "r"(o0), "r"(o1), "r"(o2), "r"(o3) : "memory");
      }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&bar_vpready[vb]));
      }
    }
  }

  // ---------------------------------------------------------------- output
  // thread (softmax warp q, lane) owns head-dim columns 128 half + 32 q + lane of all heads
  float* red_l = red;
  bool have_o = false;
  float o_acc[8];
#pragma unroll
  for (int h = 0; h < 8; ++h) o_acc[h] = 0.f;
  auto load_half = [&](int hf) {          // sum of the eight accumulators of output rows 128 hf .. 128 hf + 127
    const uint32_t lane_base = tmem_base + (uint32_t(warp * 32) << 16);
    tc_fence_after();
#pragma unroll 1
    for (int a = 0; a < kPvAccs; ++a) {
      float o[16];
      tmem_ld16(lane_base + kPvColO + 16 * (hf * kPvAccs + a), o);
#pragma unroll
      for (int h = 0; h < 8; ++h) o_acc[h] += o[h];
    }
  };
  if (warp < kPvSoft) {
    if (warp < 4 && my_tiles > 0) {                            // the first four softmax warps write the output
      bool got = true;
      if (lane == 0) got = mbar_wait(smem_u32(&bar_pvdone[(my_tiles - 1) & 1]), ((my_tiles - 1) >> 1) & 1, &abort_flag, 12);
      have_o = __all_sync(0xffffffffu, got);
      if (have_o) load_half(0);
    }
#pragma unroll
    for (int h = 0; h < kHpt; ++h) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) l_thr[h] += __shfl_xor_sync(0xffffffffu, l_thr[h], o);
    }
    if (lane == 0) {
#pragma unroll
      for (int h = 0; h < kHpt; ++h) red_l[(warp & 3) * 8 + (warp >> 2) * kHpt + h] = l_thr[h];
    }
  }
  tc_fence_before();
  __syncthreads();
  const bool failed = abort_flag != 0;
  float* stage_out = reinterpret_cast<float*>(smem + kPvOffV);      // [8 heads][D] for the NVFP4 output path
  if (warp < 4) {
#pragma unroll
    for (int hf = 0; hf < PC::kHalves; ++hf) {
      if (hf > 0) {
#pragma unroll
        for (int h = 0; h < 8; ++h) o_acc[h] = 0.f;
        if (have_o) load_half(hf);
      }
      const int d = 128 * hf + 32 * warp + lane;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        if (g >= G) break;
        const float l = (red_l[g] + red_l[8 + g]) + (red_l[16 + g] + red_l[24 + g]);
        const int head = hkv * G + g;
        if (p.splits == 1) {
          const float rr = l > 0.f ? p.out_scale / l : 0.f;
          const int64_t oi = (int64_t(b) * p.hq + head) * D + d;
          if (p.out_nvfp4) stage_out[g * D + d] = o_acc[g] * rr;
          else if (p.out_f32) static_cast<float*>(p.out)[oi] = o_acc[g] * rr;
          else static_cast<__nv_bfloat16*>(p.out)[oi] = __float2bfloat16_rn(o_acc[g] * rr);
        } else if constexpr (CL) {
          stage_out[g * D + d] = o_acc[g];
          if (d == 0) {
            stage_out[8 * D + g] = l;
            stage_out[8 * D + 8 + g] = my_tiles > 0 ? m_sh[g] : -INFINITY;
          }
        } else {
          const int64_t slot = (int64_t(split) * p.batch + b) * p.hq + head;
          p.o_part[slot * D + d] = o_acc[g];
          if (d == 0) {
            p.l_part[slot] = l;
            p.m_part[slot] = my_tiles > 0 ? m_sh[g] : -INFINITY;
          }
        }
      }
    }
  }
  if (failed && threadIdx.x == 0 && p.status) atomicExch(p.status, 1 + int(blockIdx.z) + (abort_flag << 16));
  __syncthreads();
  // every CTA takes its ticket, also one whose waits expired (the status word flags that call), so that
  // the counters are back at zero when the grid has finished
  bool pack = p.out_nvfp4 && p.splits == 1;
  if (p.splits > 1) {
    if constexpr (CL) merge_splits_cluster<D>(p, b, hkv, stage_out, split);
    else pack = merge_splits_last_cta<D>(p, b, hkv, stage_out, &merge_flag) && p.out_nvfp4;
  }
  if (pack) pack_nvfp4_output<D>(p, b, hkv, stage_out);
  if (warp == kPvMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kPvTmemCols) : "memory");
  }
}

// 3-D byte tensor over a code pool: [pages, rows of a page = heads * page_size, D/2 bytes], pages `page_stride`
// bytes apart; box = one 128-token tile; swizzle = the operand swizzle of the scores' MMA (64 bytes for head_dim
// 128, 128 bytes for 256)
template <int D>
int make_pool_map(CUtensorMap* map, const uint8_t* base, int64_t pages, int64_t page_rows, int64_t page_stride) {
  EncodeTiledFn fn;
  int s = get_encode_fn(&fn);
  if (s) return s;
  cuuint64_t dims[3] = {cuuint64_t(D / 2), cuuint64_t(page_rows), cuuint64_t(pages)};
  cuuint64_t strides[2] = {cuuint64_t(D / 2), cuuint64_t(page_stride)};
  cuuint32_t box[3] = {cuuint32_t(D / 2), cuuint32_t(kTile), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, D == 128 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed for the KV pool with CUresult %d (base %p, %lld pages of %lld rows, "
              "%lld bytes apart)", (int)r, base, (long long)pages, (long long)page_rows, (long long)page_stride);
    return RI_ERR_ARG;
  }
  return RI_OK;
}

// A cluster launch places the CTAs of a cluster on as few SMs as their resources allow, two per SM for head_dim
// 128, where they then share the conversion pipes.  A grid that has an SM for every CTA asks for this much
// shared memory instead, which makes every CTA take an SM of its own.
constexpr int kSpreadSmemBytes = 120 * 1024;

// Launch attributes of the instantiations of one (head_dim, format) on the current device, set once per device
// (also callable ahead of the first launch: ri_resattn_prepare).
template <int D, bool F8>
int prepare_decode_pv() {
  using PC = PvCfg<D, F8>;
  static bool attr_done[64] = {};
  int dev = 0;
  RI_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) dev = 0;
  if (!attr_done[dev]) {
    RI_CUDA(cudaFuncSetAttribute(resattn_pv_kernel<D, F8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PC::kSmemBytes));
    RI_CUDA(cudaFuncSetAttribute(resattn_pv_kernel<D, F8, false>, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
    RI_CUDA(cudaFuncSetAttribute(resattn_pv_kernel<D, F8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 PC::kSmemBytes > kSpreadSmemBytes ? PC::kSmemBytes : kSpreadSmemBytes));
    RI_CUDA(cudaFuncSetAttribute(resattn_pv_kernel<D, F8, true>, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
    RI_CUDA(cudaFuncSetAttribute(resattn_pv_kernel<D, F8, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));   // clusters of 16
    attr_done[dev] = true;
  }
  return RI_OK;
}

template <int D, bool F8>
int launch_decode_pv(const AttnParams& p, cudaStream_t st) {
  using PC = PvCfg<D, F8>;
  {
    int s = prepare_decode_pv<D, F8>();
    if (s) return s;
  }
  CUtensorMap k_map{}, v_map{};
  if (p.tma_pages) {
    const int64_t page_rows = int64_t(p.hkv) * p.page_size;
    int s = make_pool_map<D>(&k_map, p.k_data, p.num_pages, page_rows, p.code_page_stride);
    if (s) return s;
    s = make_pool_map<D>(&v_map, p.v_data, p.num_pages, page_rows, p.code_page_stride);
    if (s) return s;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.splits, p.hkv, p.batch);
  cfg.blockDim = dim3(PC::kThreads);
  cfg.dynamicSmemBytes = PC::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2] = {};
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (p.cluster_merge) {                                     // the splits of a (sequence, KV head) form one cluster
    if (int64_t(p.splits) * p.hkv * p.batch <= p.sm_count && PC::kSmemBytes < kSpreadSmemBytes)
      cfg.dynamicSmemBytes = kSpreadSmemBytes;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = p.splits;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
    static int fits[64][17] = {};                             // per device and cluster size: 0 unknown, 1 fits, -1 does not
    int dev = 0;
    RI_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) dev = 0;
    int& fit = fits[dev][p.splits];
    if (fit == 0) {
      int clusters = 0;
      RI_CUDA(cudaOccupancyMaxActiveClusters(&clusters, resattn_pv_kernel<D, F8, true>, &cfg));
      fit = clusters >= 1 ? 1 : -1;
    }
    if (fit < 0) {
      set_error("this device cannot co-schedule a cluster of %d decode CTAs: use the ticket reducer", p.splits);
      return RI_ERR_ARG;
    }
  }
  if (p.cluster_merge)
    return cuda_status(cudaLaunchKernelEx(&cfg, resattn_pv_kernel<D, F8, true>, k_map, v_map, p), "resattn decode launch");
  return cuda_status(cudaLaunchKernelEx(&cfg, resattn_pv_kernel<D, F8, false>, k_map, v_map, p), "resattn decode launch");
}
