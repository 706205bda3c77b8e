// Block-scaled FP4 GEMM on the Blackwell tensor cores (tcgen05), used by MEXT and KEXT.
//
//   out[M, N] = alpha * act . W^T      act: FP4 codes of the tokens (+ residue), W: FP4 weights
//
// The weight is the 128-row MMA-A operand, the tokens are the MMA-N operand (16..256 columns), so
// decode-sized batches do not waste tensor-core rows and the kernel is a weight-streaming kernel:
// every weight byte is pulled through a TMA pipeline exactly once.
//   * operands: TMA (cp.async.bulk.tensor, 128B-swizzled K-major tiles of 256 FP4 = 128 bytes),
//     no cluster multicast anywhere;
//   * block scales: 1-D bulk copies of the 512-byte 128x4 chunks into shared memory, moved to tensor
//     memory by four scale warps with wide tcgen05.st (one warp per 32-lane quarter);
//   * MMA: tcgen05.mma kind::mxf4nvf4.block_scale (block16 / UE4M3 for NVFP4) or kind::mxf4
//     (block32 / UE8M0 for MXFP4), issued by one elected thread, FP32 accumulators in tensor memory;
//   * residue fold: row_pair activations put base / residue in adjacent accumulator columns that
//     the epilogue adds; concat_k activations issue two MMA groups per W tile into one accumulator
//     (W is read once, unlike a K loop over 2K);
//   * work: the (output tile, K tile) units form one list that a persistent grid cuts into ranges --
//     whole tiles, even K splits or ragged ranges, chosen by a measured cost model.  K-split tiles
//     exchange FP32 partials through a caller workspace; the contributor that arrives last (atomic
//     ticket, nobody waits) sums them in CTA order, so the result is deterministic.
// Warp roles (12 warps): warp 0 = weight TMA producer, warp 10 = activation TMA producer, warp 11 =
// producer of the activation scales, warp 1 = MMA issuer (owns tensor memory), warps 2-5 = epilogue,
// warps 6-9 = scale warps.  Every mbarrier
// wait is bounded: on expiry the kernel records a status word, stops issuing and tears down normally.
//
// Stands in for the reference's CuTeDSL Fold kernel (ShawRong/ResInfer
// csrc/common/fold/sm10x/kernel_sm100_fold.py) and the library GEMM of its KEXT route.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "resinfer_b200.h"
#include "tc05.cuh"

namespace ri {
namespace {

constexpr int kTileW = 128;       // weight rows per CTA (MMA M)
constexpr int kTileKBytes = 128;  // 256 FP4 per K tile
constexpr int kMmaPerTile = 4;    // 4 x K64 instructions per K tile
constexpr int kThreads = 384;       // 12 warps: W producer, MMA, 4 epilogue, 4 scale, activation producer, activation-scale producer
constexpr int kTmemCols = 512;
constexpr int kSfCol = 256;        // first tensor-memory column of the block-scale sets
constexpr int kMaxSfSets = 10;      // = kMaxStages: one scale set per pipeline stage when tensor memory allows
constexpr int kMaxStages = 10;
constexpr int kMaxDynSmem = 227 * 1024 - 2048;    // 227 KB per CTA minus the static barriers / flags
constexpr int kArMaxRanks = 8;                    // ranks of the fused all-reduce
constexpr int64_t kArPairBytesMax = 2 << 20;      // fused all-reduce: up to this many bytes per rank go out as (value, call) pairs
constexpr int kEpiStageBytes = 8 * 1024;          // epilogue staging: 16 token pairs x 128 outputs x 4 bytes

struct GemmParams {
  int m, n, k;                  // tokens, weight rows, weight K (elements)
  int fmt, layout;
  int n_tile;                   // accumulator columns per CTA
  int tok_per_tile;             // tokens per CTA tile
  int act_rows;                 // rows of the activation operand (M or 2M)
  int k_tiles;
  int tiles, tok_tiles;         // output tiles (weight tiles x token tiles)
  long long units;              // tiles * k_tiles
  int grid, tile_granular;      // persistent CTAs; ranges cut at tile boundaries only
  int stages;
  int sf_sets, sf_set_cols;     // scale sets in tensor memory: 16 columns for W + the activation's
  int chunks;                   // 512-byte scale chunks per K tile (4 NVFP4, 2 MXFP4)
  int act_row_tiles;            // 128-row scale tiles the activation buffer holds
  int64_t w_sf_tile_stride;     // bytes between 128-row tiles of the weight scales
  int64_t act_sf_tile_stride;
  int act_res_chunk0;           // concat_k: first chunk of the residue half
  int act_res_col0;             // concat_k: byte column of the residue half
  const uint8_t* w_sf;
  const uint8_t* act_sf;
  const float* alpha;
  int n_alpha;
  void* out;
  int out_fp16;                 // 0 bf16, 1 fp16, 2 fp32
  int64_t out_stride;
  float* ws_partial;
  int* ws_counter;
  int32_t* status;
  // shared memory carve-up
  int smem_act_off, smem_sfa_off, smem_sfb_off, stage_bytes;
  int map3;                     // 512-element stages: the tensor maps are 3-D (128 B, rows, 256-element sub-tiles), one copy per stage
  long long* trace;             // development builds: [grid][8] nanosecond stamps
  // Fused all-reduce over peer memory (ri_fp4_gemm_allreduce).  Every rank owns an "inbox" with one area per
  // source rank.  The CTA that completes an output tile goes over the tile twice.  First pass: the BF16 tile is
  // stored into this rank's area of every PEER's inbox (plain stores that cross NVLink without waiting for
  // anything) and the tile is announced to the peers.  After the (bounded) wait for their announcements of the
  // same tile, second pass: the tile is formed again from tensor memory / the K-split partials, the peers'
  // tiles are read from the local inbox, everything is added in rank order in FP32 and written to ar_out.
  // This rank's own tile never travels through memory.
  uint16_t* ar_push[kArMaxRanks];      // where this rank's partial goes in rank r's inbox ([ar_rank] is unused)
  const uint4* ar_pull[kArMaxRanks];   // rank r's area of this rank's inbox (local memory)
  uint32_t* ar_flags[kArMaxRanks];     // rank r's flag array, [tile][kArMaxRanks] call numbers
  uint32_t* ar_epoch;                  // local: fused calls completed so far, per tile
  uint32_t* ar_state;                  // local: [0] launches completed so far, [1] CTA ticket of the running launch
  void* ar_out;
  int64_t ar_out_stride;
  long long ar_wait_ns;
  int ar_ll;                           // 1: small tiles travel as (value, call number) pairs and nobody fences (see ar_tile_vectors)
  int ar_rank, ar_world;
};

using namespace tc;

// ---------------------------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------------------------
// Work decomposition ("stream-K"): the K tiles of all output tiles form one linear list of units,
// unit u = (output tile u / KT, K tile u % KT).  The grid is persistent, one CTA per SM, and CTA c
// owns the contiguous unit range [start(c), start(c+1)), so every SM streams the same number of
// weight bytes whatever the number of output tiles is.  A range that covers only part of a tile's K
// yields an FP32 partial in the workspace; the CTA that delivers the last part of a tile (atomic
// ticket, nobody waits) adds the parts in CTA order and writes the tile.  A CTA writes at most two
// partials (its first and its last segment): slot 2c+1 when it is the first contributor of the tile,
// slot 2c otherwise.
// Development builds (-DRI_GEMM_TRACE) record nanosecond stamps of the phases of every CTA.
__device__ __forceinline__ void stamp(const GemmParams& p, int slot) {
#ifdef RI_GEMM_TRACE
  if (p.trace) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    p.trace[blockIdx.x * 8 + slot] = (long long)t;
  }
#endif
}
// per-unit event times of the first two CTAs (development builds): row `ev`, first 24 units
__device__ __forceinline__ void trace_ev(const GemmParams& p, int ev, int unit) {
#ifdef RI_GEMM_TRACE
  if (p.trace && blockIdx.x < 2 && unit < 24) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    p.trace[8 * 296 + (blockIdx.x * 8 + ev) * 24 + unit] = (long long)t;
  }
#endif
}
__device__ __forceinline__ long long range_start(const GemmParams& p, int c) {
  if (p.tile_granular) return ((long long)c * p.tiles / p.grid) * p.k_tiles;
  return (long long)c * p.units / p.grid;
}
__device__ __forceinline__ int cta_of_unit(const GemmParams& p, long long u) {
  if (p.tile_granular) return int((((u / p.k_tiles) + 1) * p.grid - 1) / p.tiles);
  return int(((u + 1) * p.grid - 1) / p.units);
}

// Position of a role in its CTA's unit list, advanced without divisions: output tile, K tile,
// pipeline stage and scale set with their mbarrier phase parities.
struct Walk {
  int tile, kt, stage, set, it;
  uint32_t stage_par, set_par;
  __device__ __forceinline__ void init(const GemmParams& p, long long u) {
    tile = int(u / p.k_tiles);
    kt = int(u % p.k_tiles);
    stage = set = it = 0;
    stage_par = set_par = 0;
  }
  __device__ __forceinline__ void next(const GemmParams& p) {
    if (++kt == p.k_tiles) { kt = 0; ++tile; }
    if (++stage == p.stages) { stage = 0; stage_par ^= 1; }
    if (++set == p.sf_sets) { set = 0; set_par ^= 1; }
    ++it;
  }
};

// Fused all-reduce, the hand-shake for one output tile, run by the four epilogue warps (threads 64..191) once
// this rank's tile has been stored into every peer's inbox.  Thread r of the first warp handles rank r: one
// system-scope release store of this tile's call number into that rank's flag array (the release covers the
// whole CTA's tile stores, which the barrier before it ordered ahead of this thread), then a wait, for at most
// ar_wait_ns, until that rank has announced the same call number here.  A CTA meets its tiles in increasing
// order and announces each before it waits, so the ranks cannot block each other in a cycle.  If a peer never
// arrives, *ar_ok is cleared and the status word says which one.
// A function of its own, not inlined: its registers are allocated apart from the kernel's main loops.
__device__ __noinline__ void ar_exchange_tile(const GemmParams& p, int* ar_ok, uint32_t ar_call, int flag_tile) {
  const int et = int(threadIdx.x) - 64;
  if (et == 0) *ar_ok = 1;
  asm volatile("bar.sync 1, 128;" ::: "memory");        // every thread's stores of the tile are behind it
  if (et < p.ar_world && et != p.ar_rank) {
    // (selected with compile-time indices: a run-time index would move the kernel arguments to local memory)
    uint32_t* flags_peer = p.ar_flags[0];
    uint32_t* flags_here = p.ar_flags[0];
#pragma unroll
    for (int r = 1; r < kArMaxRanks; ++r) {
      if (r == et) flags_peer = p.ar_flags[r];
      if (r == p.ar_rank) flags_here = p.ar_flags[r];
    }
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags_peer + flag_tile * kArMaxRanks + p.ar_rank),
                 "r"(ar_call) : "memory");
    const uint32_t* theirs = flags_here + flag_tile * kArMaxRanks + et;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (uint32_t spin = 0;; ++spin) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(theirs) : "memory");
      if (int32_t(seen - ar_call) >= 0) break;
      if ((spin & 63u) == 63u) {
        unsigned long long t1;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
        if ((long long)(t1 - t0) > p.ar_wait_ns) {
          *ar_ok = 0;
          if (p.status) atomicExch(p.status, 0x40000000 | (et << 8) | p.ar_rank);
          break;
        }
      }
    }
  }
  if (et == 0) p.ar_epoch[flag_tile] = ar_call;
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

// Fused all-reduce, the two vectors (tokens tok and tok + 1, eight outputs each) that one thread of the copy-out
// holds.  First pass (phase 1): store them into this rank's area of every peer's inbox.  Second pass (phase 2):
// read the peers' vectors from the local inbox (four ranks' loads in flight), add all ranks in rank order in FP32
// with this rank's BF16 values in its place, write BF16 to ar_out; a missing peer (ok == 0) leaves this rank's
// own values.
// Small tiles (p.ar_ll) use a protocol without fences or flag arrays: every 32-bit word of a vector travels as
// an 8-byte pair (word, call number) -- an aligned 8-byte store arrives whole -- so the reader simply polls the
// pairs of its own vector until all four carry this call's number (bounded like every other wait).  Twice the
// bytes, one NVLink crossing of latency.  The call number counts the launches on this set of inboxes, so data
// left over from earlier calls (at least two calls old: the inboxes alternate) never matches.
// Not inlined, for the same reason as ar_exchange_tile.
__device__ __forceinline__ void ll_store(uint8_t* dst, uint4 t, uint32_t call) {
  asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(t.x), "r"(call), "r"(t.y), "r"(call) : "memory");
  asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 16), "r"(t.z), "r"(call), "r"(t.w), "r"(call) : "memory");
}
// polls one vector's four pairs; false if they did not all arrive in time
__device__ __forceinline__ bool ll_load(const uint8_t* src, uint32_t call, long long wait_ns, uint4* out) {
  uint4 a, b;
  unsigned long long t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(src) : "memory");
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(src + 16) : "memory");
    if (a.y == call && a.w == call && b.y == call && b.w == call) break;
    if ((spin & 63u) == 0u) {
      unsigned long long t1;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
      if (spin == 0) t0 = t1;
      else if ((long long)(t1 - t0) > wait_ns) return false;
    }
  }
  *out = make_uint4(a.x, a.z, b.x, b.z);
  return true;
}
__device__ __noinline__ void ar_tile_vectors(const GemmParams& p, int phase, int ok, uint32_t call, uint4 t0, uint4 t1,
                                             int64_t eoff, int64_t out_off, bool second) {
  const bool ll = p.ar_ll != 0;
  if (phase == 1) {
#pragma unroll
    for (int r = 0; r < kArMaxRanks; ++r) {
      if (r < p.ar_world && r != p.ar_rank) {
        if (ll) {
          uint8_t* dst = reinterpret_cast<uint8_t*>(p.ar_push[r]) + 4 * eoff;
          ll_store(dst, t0, call);
          if (second) ll_store(dst + 4 * p.out_stride, t1, call);
        } else {
          *reinterpret_cast<uint4*>(p.ar_push[r] + eoff) = t0;
          if (second) *reinterpret_cast<uint4*>(p.ar_push[r] + eoff + p.out_stride) = t1;
        }
      }
    }
    return;
  }
  float a0s[8], a1s[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { a0s[e] = 0.f; a1s[e] = 0.f; }
#pragma unroll
  for (int r0 = 0; r0 < kArMaxRanks; r0 += 4) {
    if (r0 < p.ar_world) {
      uint4 la[4], lb[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        la[q] = make_uint4(0u, 0u, 0u, 0u);
        lb[q] = make_uint4(0u, 0u, 0u, 0u);
        if (ok && r0 + q < p.ar_world && r0 + q != p.ar_rank) {
          if (ll) {
            const uint8_t* src = reinterpret_cast<const uint8_t*>(p.ar_pull[r0 + q]) + 4 * eoff;
            bool got = ll_load(src, call, p.ar_wait_ns, &la[q]);
            if (got && second) got = ll_load(src + 4 * p.out_stride, call, p.ar_wait_ns, &lb[q]);
            if (!got) {
              ok = 0;                                        // the rest of this thread's vector: own values only
              if (p.status) atomicExch(p.status, 0x40000000 | ((r0 + q) << 8) | p.ar_rank);
            }
          } else {
            const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.ar_pull[r0 + q]) + eoff);
            asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(la[q].x), "=r"(la[q].y), "=r"(la[q].z), "=r"(la[q].w) : "l"(src));
            if (second)
              asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(lb[q].x), "=r"(lb[q].y), "=r"(lb[q].z), "=r"(lb[q].w) : "l"(src + (p.out_stride >> 3)));
          }
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (r0 + q < p.ar_world) {
          const bool mine_r = r0 + q == p.ar_rank;
          const uint32_t wa[4] = {mine_r ? t0.x : la[q].x, mine_r ? t0.y : la[q].y, mine_r ? t0.z : la[q].z, mine_r ? t0.w : la[q].w};
          const uint32_t wb[4] = {mine_r ? t1.x : lb[q].x, mine_r ? t1.y : lb[q].y, mine_r ? t1.z : lb[q].z, mine_r ? t1.w : lb[q].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            a0s[2 * e] += __uint_as_float(wa[e] << 16);
            a0s[2 * e + 1] += __uint_as_float(wa[e] & 0xFFFF0000u);
            a1s[2 * e] += __uint_as_float(wb[e] << 16);
            a1s[2 * e + 1] += __uint_as_float(wb[e] & 0xFFFF0000u);
          }
        }
      }
    }
  }
  uint4 o0 = t0, o1 = t1;                                    // a peer is missing: this rank's own values
  if (ok) {
    uint32_t* w0 = &o0.x;
    uint32_t* w1 = &o1.x;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat162 h0 = __floats2bfloat162_rn(a0s[2 * e], a0s[2 * e + 1]);
      const __nv_bfloat162 h1 = __floats2bfloat162_rn(a1s[2 * e], a1s[2 * e + 1]);
      w0[e] = *reinterpret_cast<const uint32_t*>(&h0);
      w1[e] = *reinterpret_cast<const uint32_t*>(&h1);
    }
  }
  uint16_t* fin = static_cast<uint16_t*>(p.ar_out) + out_off;
  *reinterpret_cast<uint4*>(fin) = o0;
  if (second) *reinterpret_cast<uint4*>(fin + p.ar_out_stride) = o1;
}

// ---- helpers of the two-CTA variant (a cluster of two CTAs works on one 256-row weight tile)
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {      // every thread of both CTAs
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the mbarrier at the same shared-memory offset in the leader CTA (rank 0) of the pair.  From
// the other CTA this is a relaxed arrive: the default release at cluster scope costs about 1 us per call
// (measured), which the scale warps would pay for every K tile, and nothing needs it here -- what the
// arrive announces are tensor-memory stores and loads that this thread has already waited for
// (tcgen05.wait), not generic-proxy writes.
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar, int rank) {
  if (rank == 0) {
    mbar_arrive(bar);
    return;
  }
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(bar), "r"(0));
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
// completion of this thread's earlier MMAs -> the mbarrier at this offset in BOTH CTAs of the pair
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
template <bool MX>
__device__ __forceinline__ void mma_fp4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  if constexpr (MX) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
  }
}
// Bounded wait on a barrier that the other CTA of the pair completes (its arrives, or the leader's
// multicast commits).  Polls without a suspend-time hint: a thread put to sleep by the hinted form was
// woken late when the completing arrive came from the other SM (measured: about 1.5 us per K tile).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int site) {
  long long t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((spin & 255u) == 255u) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitLimitCycles) { *abort_flag = site; return false; }
    }
  }
}
template <bool PAIR>
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag, int site) {
  if constexpr (PAIR) return mbar_wait_cluster(bar, parity, abort_flag, site);
  else return mbar_wait(bar, parity, abort_flag, site);
}

// PAIR = false: one CTA per 128-row weight tile (all plans, K splits included).
// PAIR = true: clusters of two CTAs, tcgen05.mma.cta_group::2.  A pair owns 256 weight rows and n_tile token
// columns: CTA r loads weight rows 128 r .. of the pair's tile and HALF of the activation tile (rows
// n_tile / 2 * r ..) with its own plain TMA loads -- no multicast -- so an SM takes in half as many
// activation bytes per weight byte; the MMA of the leader CTA (rank 0) reads both halves and writes 128
// accumulator rows in each CTA's tensor memory; each CTA writes its own 128 output features.  Block
// scales: every CTA loads the scales of its own weight rows and of ALL token columns.  Only whole tiles
// (no K split).  Cross-CTA signals: the scale warps of both CTAs arrive on the leader's scale barrier (an
// arrival implies that CTA's stage has landed), the leader's commits arrive on the barriers of both CTAs,
// both epilogues arrive on the leader's accumulator-free barrier.
// KS = K tiles of 256 FP4 that make up one pipeline stage (1 or 2).  What a stage costs is mostly the hand-shakes
// around it -- a turn of the producers, the scale warps and the MMA warp takes 0.4 - 0.45 us whatever the stage
// holds (traced; the kernel took the same time with the weight loads left out) -- so with few token columns, where
// shared and tensor memory have the room, a stage carries 512 elements of K: two 128-byte-swizzled sub-tiles per
// operand, eight scale chunks, eight MMAs, one round of barriers.
template <bool MX, bool PAIR, bool AR = false, int KS = 1>
__global__ void __launch_bounds__(kThreads, 1)
fp4_gemm_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap act_map,
                const __grid_constant__ GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kMaxStages];
  __shared__ __align__(8) uint64_t bar_empty[kMaxStages];
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];
  __shared__ __align__(8) uint64_t bar_sf_full[kMaxSfSets];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int abort_flag;
  __shared__ int is_last_cta;
  __shared__ int acc_ok;
  __shared__ int ar_ok;

  // dynamic shared memory is only guaranteed 16-byte aligned: round up to the 1024-byte swizzle atom
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // stays a shared-space pointer

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = PAIR ? int(cluster_rank()) : 0;          // CTA of the pair; rank 0 issues the MMAs
  const int cta = PAIR ? int(blockIdx.x >> 1) : int(blockIdx.x);   // index of the unit range (pairs share one)
  if (threadIdx.x == 0) stamp(p, 0);
  const long long u_begin = range_start(p, cta);
  const long long u_end = range_start(p, cta + 1);
  const bool kcat = p.layout == RI_GEMM_CONCAT_K;
  const int halves = kcat ? 2 : 1;
  const int row_tiles = (p.n_tile + 127) / 128;             // scale row tiles per activation tile
  static_assert(KS == 1 || !PAIR, "two-CTA tiles keep 256-element stages");
  constexpr int kKTile = 256 * KS;                           // elements of K per stage
  constexpr int kMmas = kMmaPerTile * KS;                    // K64 instructions per stage
  constexpr int kWSub = kTileW * kTileKBytes;                // bytes of one 256-element weight sub-tile
  constexpr int kSfaCols = 16 * KS;                          // tensor-memory columns of a stage's weight scales
  const int act_sub_bytes = (PAIR ? p.n_tile / 2 : p.n_tile) * kTileKBytes;   // activation rows this CTA loads, one sub-tile
  const int act_tile_bytes = act_sub_bytes * KS;             // ... per stage and half
  const int nbuf = p.n_tile <= 128 ? 2 : 1;                  // accumulator buffers in tensor memory

  // Set-up.  Warp 0 (the weight producer) initialises the barriers and only *arrives* at the set-up
  // barrier, so its first loads are in flight while warp 1 allocates tensor memory; the dependent
  // kernel of the stream may be scheduled from here on (it waits for this grid before it touches
  // anything this grid writes).
  uint32_t tmem_base = 0;
  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&w_map)) : "memory");
      for (int s = 0; s < p.stages; ++s) {
        mbar_init(smem_u32(&bar_full[s]), 1);
        mbar_init(smem_u32(&bar_empty[s]), 1);
      }
      for (int b = 0; b < 2; ++b) {
        mbar_init(smem_u32(&bar_acc_full[b]), 1);
        mbar_init(smem_u32(&bar_acc_empty[b]), PAIR ? 2 : 1);   // pair: the epilogues of both CTAs
      }
      for (int s = 0; s < kMaxSfSets; ++s) {
        mbar_init(smem_u32(&bar_sf_full[s]), PAIR ? 8 : 4);     // one arrival per scale warp (of both CTAs)
      }
      abort_flag = 0;
      is_last_cta = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __threadfence_block();
    asm volatile("bar.arrive 2, %0;" ::"n"(kThreads) : "memory");
  } else {
    if (warp == 1) {
      if constexpr (PAIR) {       // one warp of each CTA of the pair executes the pair allocation
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
      } else {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
      }
    }
    if (warp == 10 && lane == 0)
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&act_map)) : "memory");
    tc_fence_before();
    asm volatile("bar.sync 2, %0;" ::"n"(kThreads) : "memory");
    tc_fence_after();
    tmem_base = tmem_base_slot;
  }
  // pair: the barriers of both CTAs exist before anybody signals across the pair
  if constexpr (PAIR) cluster_sync_all();
  if (threadIdx.x == 32) stamp(p, 1);

  if (warp == 0 || warp >= 10) {
    // ------------------------------------------------------------------ TMA producers
    // Three issuing threads in three warps.  Issuing a copy occupies the issuing warp for 0.15-0.3 us
    // (measured), so a thread that issued all four to six copies of a K tile paced the whole pipeline;
    // in different warps the issue costs overlap.  Warp 0 arms the barrier and loads the weight tile and
    // its scales, warp 10 loads the activation tile(s), warp 11 the activation scales.
    const bool w_role = warp == 0;
    const bool act_tile_role = warp == 10;
    if (lane == 0) {
      const uint32_t sf_stride = p.chunks * 512;           // bytes of a full tile's scale chunks
      const int n_units = int(u_end - u_begin);
      Walk w;
      w.init(p, u_begin);
      int cur_tile = -1, w_tile = 0, tok_tile = 0, first_row_tile = 0, valid_row_tiles = 0;
      bool w_sf_valid = true;                                // pair: the odd last tile has no second half
      const uint8_t* w_sf_tile = nullptr;
      if (!w_role) asm volatile("griddepcontrol.wait;" ::: "memory");   // activations come from the previous kernel
      for (int i = 0; i < n_units; ++i, w.next(p)) {
        if (w.tile != cur_tile) {
          cur_tile = w.tile;
          w_tile = cur_tile / p.tok_tiles;
          tok_tile = cur_tile - w_tile * p.tok_tiles;
          if constexpr (PAIR) w_tile = 2 * w_tile + rank;     // this CTA's 128 rows of the pair's 256
          w_sf_valid = w_tile * kTileW < p.n;
          first_row_tile = (tok_tile * p.n_tile) >> 7;
          valid_row_tiles = 0;
          for (int t = 0; t < row_tiles; ++t)
            if (first_row_tile + t < p.act_row_tiles) ++valid_row_tiles;
          w_sf_tile = p.w_sf + int64_t(w_tile) * p.w_sf_tile_stride;
        }
        // the last K tile may hold fewer K64 steps: copy only the scale chunks that exist
        const int rem = p.k - w.kt * kKTile;
        const int n_mma = rem >= kKTile ? kMmas : rem >> 6;
        const uint32_t sf_bytes = uint32_t(MX ? (n_mma + 1) >> 1 : n_mma) * 512;
        if (w.it >= p.stages) {
          if (!wait_bar<PAIR>(smem_u32(&bar_empty[w.stage]), w.stage_par ^ 1, &abort_flag, w_role ? 1 : 2)) break;
        }
        uint8_t* st = smem + w.stage * p.stage_bytes;
        const uint32_t full = smem_u32(&bar_full[w.stage]);
        trace_ev(p, w_role ? 0 : (act_tile_role ? 1 : 7), i);
        if (w_role) {
          const uint32_t tx = KS * kWSub + (w_sf_valid ? sf_bytes : 0u) +
                              halves * (act_tile_bytes + valid_row_tiles * sf_bytes);
          mbar_expect_tx(full, tx);
          if (KS > 1 && p.map3) {                             // all sub-tiles with one copy: issuing a copy is what costs
            tma_load_3d(smem_u32(st), &w_map, 0, w_tile * kTileW, w.kt * KS, full);
          } else {
#pragma unroll
            for (int sub = 0; sub < KS; ++sub)                // rows past N and columns past K read as zero
              tma_load_2d(smem_u32(st + sub * kWSub), &w_map, (w.kt * KS + sub) * kTileKBytes, w_tile * kTileW, full);
          }
          if (w_sf_valid) bulk_load_1d(smem_u32(st + p.smem_sfa_off), w_sf_tile + w.kt * sf_stride, sf_bytes, full);
        } else {
          for (int h = 0; h < halves; ++h) {
            if (act_tile_role) {
              if (KS > 1 && p.map3) {                         // (one half only with a 3-D map)
                tma_load_3d(smem_u32(st + p.smem_act_off), &act_map, 0, tok_tile * p.n_tile, w.kt * KS, full);
                continue;
              }
#pragma unroll
              for (int sub = 0; sub < KS; ++sub)
                tma_load_2d(smem_u32(st + p.smem_act_off + h * act_tile_bytes + sub * act_sub_bytes), &act_map,
                            (w.kt * KS + sub) * kTileKBytes + h * p.act_res_col0,
                            tok_tile * p.n_tile + (PAIR ? rank * (p.n_tile / 2) : 0), full);
              continue;
            }
            for (int t = 0; t < row_tiles; ++t) {
              if (first_row_tile + t >= p.act_row_tiles) continue;
              const uint8_t* src = p.act_sf + int64_t(first_row_tile + t) * p.act_sf_tile_stride +
                                   (w.kt * p.chunks + h * p.act_res_chunk0) * 512;
              bulk_load_1d(smem_u32(st + p.smem_sfb_off + (h * row_tiles + t) * sf_stride), src, sf_bytes, full);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (!PAIR || rank == 0) {   // the whole warp walks the loop (converged); one elected lane issues the tcgen05 instructions
      // (a single thread walking the loop alone measured 3-6 % slower)
      // instruction descriptor: E2M1 x E2M1, K-major A and B, M = 128, N = n_tile
      const uint32_t idesc_base = (1u << 7) | (1u << 10) | (uint32_t(p.n_tile >> 3) << 17) |
                                  (MX ? (1u << 23) : 0u) | (uint32_t((PAIR ? 2 * kTileW : kTileW) >> 4) << 24);
      bool ok = true;
      const int n_units = int(u_end - u_begin);
      const uint32_t smem_addr0 = smem_u32(smem);
      const int act_sub_units = act_sub_bytes >> 4;           // an activation sub-tile in descriptor units
      const bool sets_per_stage = p.sf_sets == p.stages;
      Walk w;
      w.init(p, u_begin);
      int seg = 0, i = 0;
      while (i < n_units && ok) {
        const int buf = nbuf == 2 ? (seg & 1) : 0;
        if (seg >= nbuf) {                          // the epilogue must have drained this buffer
          const bool got = wait_bar<PAIR>(smem_u32(&bar_acc_empty[buf]), ((seg / nbuf) - 1) & 1, &abort_flag, 3);
          if (!__all_sync(0xffffffffu, got)) { ok = false; break; }       // warp-uniform decision
          tc_fence_after();
        }
        const uint32_t d_tmem = tmem_base + buf * p.n_tile;
        uint32_t accumulate = 0;
        for (;;) {                                  // K tiles of this segment (same output tile)
          // The scale warps have put this K tile's block scales into scale set `set` of tensor memory (pair: the
          // scale warps of both CTAs).  They waited for the stage's data before they read its scales, so their
          // arrival also tells that the stage has landed -- here and in the other CTA of a pair.  Only when scale
          // sets are recycled faster than stages (sets < stages) is the stage's own barrier looked at as well.
          bool got = sets_per_stage || wait_bar<PAIR>(smem_u32(&bar_full[w.stage]), w.stage_par, &abort_flag, 4);
          got = got && wait_bar<PAIR>(smem_u32(&bar_sf_full[w.set]), w.set_par, &abort_flag, 5);
          if (!__all_sync(0xffffffffu, got)) { ok = false; break; }       // warp-uniform decision
          tc_fence_after();
          if (w.it == 0 && lane == 0) stamp(p, 3);
          if (lane == 0) trace_ev(p, 2, i);
          const bool leader = elect_one();
          const uint32_t st_addr = smem_addr0 + uint32_t(w.stage * p.stage_bytes);
          const int rem = p.k - w.kt * kKTile;
          const int n_mma = rem >= kKTile ? kMmas : rem >> 6;
          const uint32_t sfa_col = tmem_base + kSfCol + w.set * p.sf_set_cols;
          const uint32_t sfb_col = sfa_col + kSfaCols;
          // descriptors: the start address field counts 16-byte units, so the K64 steps of a sub-tile (32 bytes
          // apart) and the sub-tiles of a stage are constant offsets from the stage's first descriptor
          const uint64_t a_desc0 = desc_sw128(st_addr);
          for (int h = 0; h < halves; ++h) {
            const uint64_t b_desc0 = desc_sw128(st_addr + uint32_t(p.smem_act_off + h * act_tile_bytes));
#pragma unroll
            for (int j = 0; j < kMmas; ++j) {
              if (j >= n_mma) break;
              const uint64_t a_desc = a_desc0 + uint64_t((j >> 2) * (kWSub >> 4) + (j & 3) * 2);
              const uint64_t b_desc = b_desc0 + uint64_t((j >> 2) * act_sub_units + (j & 3) * 2);
              // NVFP4: one chunk per instruction; MXFP4: one chunk per two instructions, the second
              // uses scale bytes 2-3 of each column (scale-factor id 2)
              const int c = MX ? (j >> 1) : j;
              const uint32_t sf_id = MX ? uint32_t((j & 1) * 2) : 0u;
              const uint32_t idesc = idesc_base | (sf_id << 4) | (sf_id << 29);
              if (leader) {
                if constexpr (PAIR)
                  mma_fp4_pair<MX>(d_tmem, a_desc, b_desc, idesc,
                                   sfa_col + 4 * c, sfb_col + ((h * p.chunks + c) * row_tiles) * 4, accumulate);
                else
                  mma_fp4<MX>(d_tmem, a_desc, b_desc, idesc,
                              sfa_col + 4 * c, sfb_col + ((h * p.chunks + c) * row_tiles) * 4, accumulate);
              }
              accumulate = 1;
            }
          }
          if (leader) {                               // frees the stage (and, later, its scale set); pair: in both CTAs
            if constexpr (PAIR) mma_commit_pair(smem_u32(&bar_empty[w.stage]));
            else mma_commit(smem_u32(&bar_empty[w.stage]));
          }
          __syncwarp();
          if (lane == 0) trace_ev(p, 3, i);
          const bool tile_done = w.kt == p.k_tiles - 1;
          w.next(p);
          ++i;
          if (tile_done || i == n_units) break;
        }
        if (ok && elect_one()) {                    // this segment's accumulator is complete
          if constexpr (PAIR) mma_commit_pair(smem_u32(&bar_acc_full[buf]));
          else mma_commit(smem_u32(&bar_acc_full[buf]));
        }
        __syncwarp();
        ++seg;
      }
      if (lane == 0) {
        stamp(p, 4);
      }
    }
  } else {
    // ------------------------------------------------------ epilogue (warps 2..5), scales (warps 6..9)
    // a warp touches tensor-memory lanes 32*(warp%4)..+31; each role walks the list of segments in a loop of its own (separate loops keep the registers of one role
    // out of the other's way: values that are live in a shared loop get spilled into the per-K-tile path)
    const bool scale_role = warp >= 6;
    const int quarter = warp & 3;
    const int n_units = int(u_end - u_begin);
    Walk w;
    w.init(p, u_begin);
    int i = 0;
    if (scale_role) {
      // ---- scale duty: copy the block scales of every K tile from shared memory into a scale set of
      // tensor memory.  The 512-byte chunk of (128 rows x 4 k-groups) is laid out so that lane l reads
      // 16 bytes = the 4 columns of rows l, l+32, l+64, l+96; every warp writes the same 32 x 4 columns
      // into its own quarter (the MMA expects them replicated).
      bool scale_alive = true;
      const uint32_t sf_stride = p.chunks * 512;
      const uint32_t q_lane = uint32_t(quarter * 32) << 16;
      int lag_stage = 0;
      uint32_t lag_par = 0;
      {
        for (; i < n_units; ++i, w.next(p)) {
          if (!scale_alive) continue;
          const int rem = p.k - w.kt * kKTile;
          const int n_mma = rem >= kKTile ? kMmas : rem >> 6;
          const int n_chunks = MX ? (n_mma + 1) >> 1 : n_mma;
          bool got = wait_bar<PAIR>(smem_u32(&bar_full[w.stage]), w.stage_par, &abort_flag, 6);
          if (got && p.sf_sets < p.stages && w.it >= p.sf_sets) {
            // fewer scale sets than stages: before a set is reused the MMAs of unit (it - sf_sets) must have
            // completed, which is what the commit on that unit's stage barrier reports.  (With one set per
            // stage the arrival of the stage's data already implies it: the stage was refilled only after
            // that commit.)
            got = wait_bar<PAIR>(smem_u32(&bar_empty[lag_stage]), lag_par, &abort_flag, 7);
            if (++lag_stage == p.stages) { lag_stage = 0; lag_par ^= 1; }
          }
          if (!__all_sync(0xffffffffu, got)) { scale_alive = false; continue; }
          tc_fence_after();
          if (warp == 6 && lane == 0) trace_ev(p, 4, i);
          const uint8_t* st = smem + w.stage * p.stage_bytes;
          const uint32_t col0 = tmem_base + q_lane + kSfCol + w.set * p.sf_set_cols;
          const uint8_t* sfa_src = st + p.smem_sfa_off + lane * 16;
          const uint8_t* sfb_src = st + p.smem_sfb_off + lane * 16;
          if (KS > 1 && n_chunks == p.chunks) {
            // 512- / 1024-element stages (one scale row tile, no two-CTA tiles): groups of four chunks = 16 columns
            constexpr int kGroups = (MX ? 2 : 4) * KS / 4;
#pragma unroll
            for (int g = 0; g < kGroups; ++g) {
              uint4 a[4];
#pragma unroll
              for (int c = 0; c < 4; ++c) a[c] = *reinterpret_cast<const uint4*>(sfa_src + (g * 4 + c) * 512);
              tmem_st16(col0 + g * 16, a);
            }
            for (int h = 0; h < halves; ++h) {
#pragma unroll
              for (int g = 0; g < kGroups; ++g) {
                uint4 b[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) b[c] = *reinterpret_cast<const uint4*>(sfb_src + h * sf_stride + (g * 4 + c) * 512);
                tmem_st16(col0 + kSfaCols + (h * p.chunks + g * 4) * 4, b);
              }
            }
          } else if (n_chunks == p.chunks) {
            // full K tile: 16-byte chunk slices are fetched first, then written with wide stores
            // (4 chunks = 16 columns per instruction; MXFP4 has 2 chunks = 8 columns)
            if constexpr (MX) {
              uint4 a[2] = {*reinterpret_cast<const uint4*>(sfa_src), *reinterpret_cast<const uint4*>(sfa_src + 512)};
              tmem_st8(col0, a);
              for (int g8 = 0; g8 < halves * row_tiles; ++g8) {       // column order (h, c, t): pairs of chunks
                const int h = g8 / row_tiles, tt = g8 % row_tiles;
                // with two row tiles the column order interleaves them: c0t0 c0t1 c1t0 c1t1
                if (row_tiles == 1) {
                  const uint8_t* s0 = sfb_src + h * sf_stride;
                  uint4 b[2] = {*reinterpret_cast<const uint4*>(s0), *reinterpret_cast<const uint4*>(s0 + 512)};
                  tmem_st8(col0 + 16 + h * 8, b);
                } else {
                  const int c = tt;                                    // one chunk, both row tiles
                  const uint8_t* s0 = sfb_src + (h * 2) * sf_stride + c * 512;
                  uint4 b[2] = {*reinterpret_cast<const uint4*>(s0), *reinterpret_cast<const uint4*>(s0 + sf_stride)};
                  tmem_st8(col0 + 16 + (h * 2 + c) * 8, b);
                }
              }
            } else {
              uint4 a[4];
#pragma unroll
              for (int c = 0; c < 4; ++c) a[c] = *reinterpret_cast<const uint4*>(sfa_src + c * 512);
              tmem_st16(col0, a);
              if (row_tiles == 1) {
                for (int h = 0; h < halves; ++h) {
                  uint4 b[4];
#pragma unroll
                  for (int c = 0; c < 4; ++c) b[c] = *reinterpret_cast<const uint4*>(sfb_src + h * sf_stride + c * 512);
                  tmem_st16(col0 + 16 + h * 16, b);
                }
              } else {
                for (int h = 0; h < halves; ++h)
                  for (int cp = 0; cp < 2; ++cp) {                     // chunk pair: c, t order = c0t0 c0t1 c1t0 c1t1
                    uint4 b[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                      b[q] = *reinterpret_cast<const uint4*>(sfb_src + (h * 2 + (q & 1)) * sf_stride + (cp * 2 + (q >> 1)) * 512);
                    tmem_st16(col0 + 16 + (h * 4 + cp * 2) * 8, b);
                  }
              }
            }
          } else {
            for (int c = 0; c < n_chunks; ++c) {
              tmem_st4(col0 + 4 * c, *reinterpret_cast<const uint4*>(sfa_src + c * 512));
              for (int h = 0; h < halves; ++h)
                for (int t = 0; t < row_tiles; ++t)
                  tmem_st4(col0 + kSfaCols + ((h * p.chunks + c) * row_tiles + t) * 4,
                           *reinterpret_cast<const uint4*>(sfb_src + (h * row_tiles + t) * sf_stride + c * 512));
            }
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          tc_fence_before();
          if (warp == 6 && lane == 0) trace_ev(p, 5, i);
          if (lane == 0) {
            if constexpr (PAIR) mbar_arrive_leader(smem_u32(&bar_sf_full[w.set]), rank);   // the leader's barrier
            else mbar_arrive(smem_u32(&bar_sf_full[w.set]));
          }
          if (warp == 6 && lane == 0) trace_ev(p, 6, i);
        }
      }
    } else {
    const int row_in_tile = quarter * 32 + lane;
    const bool pair = p.layout == RI_GEMM_ROW_PAIR;
    const int64_t tile_elems = int64_t(kTileW) * p.n_tile;
    int seg = 0;
    const int esz = p.out_fp16 == 2 ? 4 : 2;                  // output element size
    const bool out_vec = ((reinterpret_cast<uintptr_t>(p.out) | uintptr_t(p.out_stride * esz)) & 15) == 0;
    uint8_t* epi_stage = smem + p.stages * p.stage_bytes;     // kEpiStageBytes behind the pipeline stages
    // global scales may come from the kernel before this one; fetch them while the main loop runs
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float a0 = p.alpha ? __ldg(p.alpha) : 1.0f;
    const float a1 = (p.alpha && p.n_alpha > 1) ? __ldg(p.alpha + 1) : a0;
    uint32_t ar_launch_call = 0;                               // launches on these inboxes so far, plus one
    if constexpr (AR) {
      if (p.ar_ll) ar_launch_call = p.ar_state[0] + 1;        // (the launch before this one has completed: see the wait above)
    }
    while (i < n_units) {
      const int tile = w.tile;
      const long long tile_begin = (long long)tile * p.k_tiles, tile_end = tile_begin + p.k_tiles;
      const int seg_units = min(p.k_tiles - w.kt, n_units - i);          // K tiles of this segment
      const bool complete = seg_units == p.k_tiles;
      const int buf = nbuf == 2 ? (seg & 1) : 0;
      for (int j = 0; j < seg_units; ++j, ++i) w.next(p);
      // ---- epilogue duty for the segment
      // one thread waits for the accumulator so that all four warps take the same decision
      const int c_first = cta_of_unit(p, tile_begin), c_last = cta_of_unit(p, tile_end - 1);
      if (warp == 2 && lane == 0) {
        // K-split tile: have all the other contributors delivered already?  (Usually true for a CTA's
        // last segment: the rest of that tile was another CTA's first piece of work.)  Then this CTA
        // is the one that finishes the tile and its own part never has to leave the SM.
        int others = -1;
        if (!complete) {
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(others) : "l"(p.ws_counter + tile) : "memory");
        }
        acc_ok = wait_bar<PAIR>(smem_u32(&bar_acc_full[buf]), (seg / nbuf) & 1, &abort_flag, 8) ? 1 : 0;
        is_last_cta = (!complete && others == c_last - c_first) ? 2 : 0;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!acc_ok) break;
      tc_fence_after();
      const bool finish_now = is_last_cta == 2;
      if (seg == 0 && threadIdx.x == 64) stamp(p, 5);
      const int tok_tile = tile % p.tok_tiles;
      const int w_tile = PAIR ? 2 * (tile / p.tok_tiles) + rank : tile / p.tok_tiles;
      const int n_row0 = w_tile * kTileW;
      const int tok0 = tok_tile * p.tok_per_tile;
      const uint32_t t_lane = tmem_base + buf * p.n_tile + (uint32_t(quarter * 32) << 16);
      float* mine = p.ws_partial + (int64_t(cta) * 2 + (cta == c_first ? 1 : 0)) * tile_elems;
      // fused all-reduce: this tile's call number (per tile with the flag protocol, per launch with the pairs)
      uint32_t ar_call = 0;
      if constexpr (AR) {
        if (p.ar_ll) ar_call = ar_launch_call;
        else if (n_row0 < p.n) ar_call = p.ar_epoch[w_tile * p.tok_tiles + tok_tile] + 1;
      }

      // Output of one chunk of 32 accumulator columns (16 tokens with the row_pair layout, 32
      // otherwise).  A thread owns one output column n (its weight row) and `ntok` token values.
      // 16-bit outputs go through shared memory so that the global stores are 16-byte vectors along
      // n: two tokens are packed into one 32-bit word, word [token pair][n]; a thread of the
      // copy-out reads 8 words of a pair row and writes one vector for each of the two tokens.
      // FP32 output (a debugging format) is stored element by element.
      auto emit_chunk = [&](const float (&v)[32], int c0, int cols, int phase) {
        const int ntok = pair ? cols >> 1 : cols;
        const int tokc0 = tok0 + (pair ? c0 >> 1 : c0);
        float o[32];
        if (pair) {
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = p.n_alpha > 1 ? a0 * v[2 * j] + a1 * v[2 * j + 1] : a0 * (v[2 * j] + v[2 * j + 1]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = a0 * v[j];
        }
        if (esz == 4) {
          const int n = n_row0 + row_in_tile;
          if (n < p.n) {
            float* dst = static_cast<float*>(p.out) + int64_t(tokc0) * p.out_stride + n;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < ntok && tokc0 + j < p.m) dst[int64_t(j) * p.out_stride] = o[j];
          }
          return;
        }
        uint32_t* stage32 = reinterpret_cast<uint32_t*>(epi_stage);
        const int npair = (ntok + 1) >> 1;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          if (i < npair) {
            uint32_t wv;
            if (p.out_fp16) {
              const __half2 h = __floats2half2_rn(o[2 * i], o[2 * i + 1]);
              wv = *reinterpret_cast<const uint32_t*>(&h);
            } else {
              const __nv_bfloat162 h = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
              wv = *reinterpret_cast<const uint32_t*>(&h);
            }
            stage32[i * kTileW + row_in_tile] = wv;
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // copy-out: thread -> (pair row, vector of 8 outputs); 16 vectors per token row of the tile
        const int et = int(threadIdx.x) - 64;
        for (int pr = et >> 4; pr < npair; pr += 8) {
          const int vc = et & 15;
          const int n0 = n_row0 + vc * 8;
          const int tok = tokc0 + 2 * pr;
          if (tok >= p.m || n0 >= p.n) continue;
          const uint4 lo4 = *reinterpret_cast<const uint4*>(stage32 + pr * kTileW + vc * 8);
          const uint4 hi4 = *reinterpret_cast<const uint4*>(stage32 + pr * kTileW + vc * 8 + 4);
          uint4 t0, t1;                                       // token `tok` (low halves), token `tok + 1` (high halves)
          t0.x = __byte_perm(lo4.x, lo4.y, 0x5410); t0.y = __byte_perm(lo4.z, lo4.w, 0x5410);
          t0.z = __byte_perm(hi4.x, hi4.y, 0x5410); t0.w = __byte_perm(hi4.z, hi4.w, 0x5410);
          t1.x = __byte_perm(lo4.x, lo4.y, 0x7632); t1.y = __byte_perm(lo4.z, lo4.w, 0x7632);
          t1.z = __byte_perm(hi4.x, hi4.y, 0x7632); t1.w = __byte_perm(hi4.z, hi4.w, 0x7632);
          uint16_t* dst = static_cast<uint16_t*>(p.out) + int64_t(tok) * p.out_stride + n0;
          const bool second = tok + 1 < p.m && 2 * pr + 1 < ntok;
          if constexpr (AR) {
            if (phase) {                                           // (the host checked the vector alignment)
              ar_tile_vectors(p, phase, p.ar_ll ? 1 : ar_ok, ar_call, t0, t1, int64_t(tok) * p.out_stride + n0,
                              int64_t(tok) * p.ar_out_stride + n0, second);
              continue;
            }
          }
          if (out_vec && n0 + 8 <= p.n) {
            *reinterpret_cast<uint4*>(dst) = t0;
            if (second) *reinterpret_cast<uint4*>(dst + p.out_stride) = t1;
          } else {
            const uint32_t a[4] = {t0.x, t0.y, t0.z, t0.w}, bq[4] = {t1.x, t1.y, t1.z, t1.w};
            const int cnt = min(8, p.n - n0);
            for (int e = 0; e < cnt; ++e) {
              dst[e] = uint16_t(a[e >> 1] >> ((e & 1) * 16));
              if (second) dst[p.out_stride + e] = uint16_t(bq[e >> 1] >> ((e & 1) * 16));
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");      // the stage is reused by the next chunk
      };

      // A tile that is finished here goes through its chunks once -- or, with the fused all-reduce, twice
      // (store to the peers, hand-shake, form again and add the peers' tiles).
      const bool ar_tile = AR && n_row0 < p.n;
      for (int phase = (ar_tile && (complete || finish_now)) ? 1 : 0;;) {
      for (int c0 = 0; c0 < p.n_tile; c0 += 32) {
        const int cols = min(32, p.n_tile - c0);               // 32, or 16 for the last chunk
        float v[32];
        if (cols == 32) {
          tmem_ld32(t_lane + c0, v);
        } else {
          float lo[16];
          tmem_ld16(t_lane + c0, lo);
#pragma unroll
          for (int j = 0; j < 16; ++j) { v[j] = lo[j]; v[16 + j] = 0.f; }
        }
        if (finish_now) {
          // sum in CTA order, this CTA's part straight from tensor memory (same order and values as
          // the reduction below, so the result does not depend on which path ran)
          float s[32];
#pragma unroll
          for (int q = 0; q < 32; ++q) s[q] = 0.f;
          const int64_t off = int64_t(c0) * kTileW + row_in_tile;
          for (int cc = c_first; cc <= c_last; ++cc) {
            if (cc == cta) {
#pragma unroll
              for (int q = 0; q < 32; ++q) s[q] += v[q];
            } else {
              const float* s0 = p.ws_partial + (int64_t(cc) * 2 + (cc == c_first ? 1 : 0)) * tile_elems + off;
              float fa[32];
#pragma unroll
              for (int q = 0; q < 32; ++q) fa[q] = q < cols ? __ldcg(s0 + q * kTileW) : 0.f;
#pragma unroll
              for (int q = 0; q < 32; ++q) s[q] += fa[q];
            }
          }
          emit_chunk(s, c0, cols, phase);
        } else if (!complete) {
          // partial tile, column-major [n_tile][128]: a warp writes one full 128-byte line per column
          float* dst = mine + int64_t(c0) * kTileW + row_in_tile;
#pragma unroll
          for (int j = 0; j < 32; ++j) if (j < cols) __stcg(dst + j * kTileW, v[j]);
        } else {
          emit_chunk(v, c0, cols, phase);
        }
      }
      if (phase != 1) break;
      if constexpr (AR) {
        if (!p.ar_ll) ar_exchange_tile(p, &ar_ok, ar_call, w_tile * p.tok_tiles + tok_tile);
      }
      phase = 2;
      }
      // the accumulator buffer has been read: hand it back to the MMA warp
      tc_fence_before();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        if constexpr (PAIR) mbar_arrive_leader(smem_u32(&bar_acc_empty[buf]), rank);   // the leader issues the next tile's MMAs
        else mbar_arrive(smem_u32(&bar_acc_empty[buf]));
        if (finish_now) {
          p.ws_counter[tile] = 0;                  // everybody else has arrived: ready for the next call
        } else if (!complete) {
          // the barrier above ordered every thread's partial stores before this thread; the fence
          // publishes them device-wide before the ticket, and orders the reads after it
          __threadfence();
          const int ticket = atomicAdd(p.ws_counter + tile, 1);
          const int last = ticket == c_last - c_first;
          if (last) p.ws_counter[tile] = 0;        // ready for the next call
          is_last_cta = last;
          __threadfence();
        }
      }
      if (!complete && !finish_now) {
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) stamp(p, 2);
        if (is_last_cta) {
          // add the parts in CTA order (deterministic), 32 columns at a time with the loads of two
          // contributors in flight together, then write the chunk like a complete tile's
          for (int phase = ar_tile ? 1 : 0;;) {
          for (int c0 = 0; c0 < p.n_tile; c0 += 32) {
            const int cols = min(32, p.n_tile - c0);
            float s[32];
#pragma unroll
            for (int q = 0; q < 32; ++q) s[q] = 0.f;
            const int64_t off = int64_t(c0) * kTileW + row_in_tile;
            for (int cc = c_first; cc <= c_last; cc += 2) {
              const float* s0 = p.ws_partial + (int64_t(cc) * 2 + (cc == c_first ? 1 : 0)) * tile_elems + off;
              const bool two = cc + 1 <= c_last;
              const float* s1 = p.ws_partial + (int64_t(two ? cc + 1 : cc) * 2) * tile_elems + off;
              float fa[32], fb[32];
#pragma unroll
              for (int q = 0; q < 32; ++q) fa[q] = q < cols ? __ldcg(s0 + q * kTileW) : 0.f;
#pragma unroll
              for (int q = 0; q < 32; ++q) fb[q] = (two && q < cols) ? __ldcg(s1 + q * kTileW) : 0.f;
#pragma unroll
              for (int q = 0; q < 32; ++q) s[q] += fa[q];
#pragma unroll
              for (int q = 0; q < 32; ++q) s[q] += fb[q];
            }
            emit_chunk(s, c0, cols, phase);
          }
          if (phase != 1) break;
          if constexpr (AR) {
            if (!p.ar_ll) ar_exchange_tile(p, &ar_ok, ar_call, w_tile * p.tok_tiles + tok_tile);
          }
          phase = 2;
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");    // is_last_cta is reused by the next segment
      }
      ++seg;
    }
    if (threadIdx.x == 64) stamp(p, 6);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) stamp(p, 7);
  if constexpr (AR) {
    // the last CTA to get here closes the call: the next launch on these inboxes reads the new count
    if (p.ar_ll && threadIdx.x == 0) {
      const uint32_t t = atomicAdd(p.ar_state + 1, 1u);
      if (t == gridDim.x - 1) {
        p.ar_state[1] = 0;
        __threadfence();
        *reinterpret_cast<volatile uint32_t*>(p.ar_state) = *reinterpret_cast<volatile uint32_t*>(p.ar_state) + 1;
      }
    }
  }
  if (abort_flag) {
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, 1 + (int)blockIdx.x + (abort_flag << 16));   // CTA and wait site
    __nanosleep(1000000);                          // let copies that are still in flight land
  }
  if constexpr (PAIR) {
    // neither CTA frees tensor memory or leaves while its partner may still signal it or read its tiles
    cluster_sync_all();
    if (warp == 1) {
      tc_fence_after();
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
  } else if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
// 2-D byte tensor [rows, row_bytes] (row stride `stride` bytes) with a [box_rows, 128 B] box,
// 128-byte swizzle, zero fill outside.
int make_map(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t stride,
             uint32_t box_rows) {
  EncodeTiledFn fn;
  int s = get_encode_fn(&fn);
  if (s) return s;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {stride};
  cuuint32_t box[2] = {kTileKBytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (base %p, row_bytes %llu, rows %llu, stride %llu, box_rows %u)",
              (int)r, base, (unsigned long long)row_bytes, (unsigned long long)rows, (unsigned long long)stride, box_rows);
    return RI_ERR_ARG;
  }
  return RI_OK;
}

// The same bytes as a 3-D tensor [row_bytes / 128 sub-tiles, rows, 128 B] with a [2, box_rows, 128 B] box: one copy
// brings two consecutive 128-byte-swizzled K sub-tiles of the same rows, laid out one after the other in shared
// memory exactly as two copies of the 2-D box would.  row_bytes must be a multiple of 128 (every sub-tile whole).
// Returns RI_ERR_UNSUPPORTED, without touching the error text, if the driver does not take the map.
int make_map_subtiles(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t stride,
                      uint32_t box_rows, uint32_t sub_tiles) {
  EncodeTiledFn fn;
  int s = get_encode_fn(&fn);
  if (s) return s;
  cuuint64_t dims[3] = {kTileKBytes, rows, row_bytes / kTileKBytes};
  cuuint64_t strides[2] = {stride, kTileKBytes};
  cuuint32_t box[3] = {kTileKBytes, box_rows, sub_tiles};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? RI_OK : RI_ERR_UNSUPPORTED;
}

// Pairs (clusters of two CTAs with the kernel's shared-memory footprint) that can be resident at once,
// per device; 0 = not asked yet (then SMs / 2 is assumed).  Filled by ri_fp4_gemm before it plans.
int g_pair_slots[64] = {};
int g_plan_device = 0;
constexpr int kKs2MaxCols = 128;   // widest activation tile that gets 512-element stages
#ifdef RI_GEMM_FORCE_KS           // development builds: 1 / 2 forces the stage size where the shape allows it
constexpr int g_force_ks = RI_GEMM_FORCE_KS;
#else
constexpr int g_force_ks = 0;
#endif

struct Plan {
  int n_tile, tok_per_tile, tok_tiles, w_tiles, k_tiles, tiles, stages;
  long long units;
  int grid, tile_granular;      // persistent CTAs (pair plans: pairs) and how their unit ranges are cut
  int pair;                     // two-CTA tiles of 256 weight rows (cta_group::2), whole tiles only
  int ks;                       // 256-element K tiles per pipeline stage (1 or 2)
  int chunks, stage_bytes, smem_act_off, smem_sfa_off, smem_sfb_off, smem_total;
};

// Measured choices for the projection shapes of the benchmark model on a 148-SM part (NVFP4 and MXFP4,
// row_pair activations; sweep over splits 1, 2, 3, 4, 6 per (shape, M) under CUDA graphs with rotating
// weight copies): weight rows, K, largest M of the bucket, `splits` value of the fastest plan.  Shapes that
// are not listed use the cost model below, which reproduces these rows to within 2 %.  Stands where the
// reference keys tile and cluster shapes on M (csrc/common/fold/sm10x/tactics.py:14-87).
struct Tactic { int n, k, m_max, splits; };
constexpr Tactic kTactics[] = {
    {10240, 5120, 128, 1},                          // qkv: 80 whole tiles; K splits over all SMs measured 13-70 % slower
    {5120, 8192, 16, 3}, {5120, 8192, 128, 2},      // o: 40 tiles x 3 K slices up to 16 tokens, x 2 above
    {51200, 5120, 128, 1},                          // gate_up: whole tiles (K splits within 1 % up to 8 tokens, 4-17 % slower above)
    {5120, 25600, 128, 3},                          // down: 40 tiles x 3 K slices (ragged ranges over all SMs 3-10 % slower)
};

// `splits`: 1 = ranges are cut at output-tile boundaries only (no K split, no workspace);
// 0 = choose (stream-K over all SMs unless the tiles already balance); s > 1 = stream-K over
// min(tiles * s, SMs) CTAs; -2 = two-CTA tiles where the shape allows them (256 accumulator columns),
// else as 1.
int make_plan(int m, int n, int k, int fmt, int layout, int splits, int sm_count, Plan* pl) {
  if (splits == 0 && sm_count == 148 && layout == RI_GEMM_ROW_PAIR) {
    for (const Tactic& t : kTactics)
      if (t.n == n && t.k == k && m <= t.m_max) {
        splits = t.splits;
        break;
      }
  }
  const int act_rows = layout == RI_GEMM_ROW_PAIR ? 2 * m : m;
  const int halves_c = layout == RI_GEMM_CONCAT_K ? 2 : 1;
  pl->w_tiles = (n + kTileW - 1) / kTileW;
  // Stages of 512 elements of K while the activation tile has at most 128 columns: the scale sets then still fit
  // tensor memory beside two accumulator buffers (four sets of 64 columns, two of 96 with the concat_k layout) and
  // two to four stages of 48-108 KB fit shared memory -- a shallow pipeline, but depth is not what limits these
  // launches (four stages measured the same as eight): the per-stage hand-shakes are, see the kernel.  Measured
  // against 256-element stages: 8-17 % less time up to 64 tokens, 3-14 % at 64, 8 % at 128 (concat_k) on three
  // of the four benchmark shapes and 2 % more on the fourth.
  pl->ks = (g_force_ks == 1 || (act_rows + 15) / 16 * 16 > kKs2MaxCols || k < 1024) ? 1 : 2;
  if (halves_c == 2 && k > 8192) pl->ks = 1;      // two stages of 108 KB lose on long K (measured, K = 25600: +10 %)
  // (1024-element stages were built and measured too: two stages fit, and the launch is 5 % slower)
  pl->k_tiles = (k + 256 * pl->ks - 1) / (256 * pl->ks);
  pl->pair = 0;
  pl->chunks = (fmt == RI_FMT_NVFP4 ? 4 : 2) * pl->ks;
  // accumulator columns per CTA: one tile for up to `cap` activation rows, tiles of `cap` rows above.
  // Plans that split K use cap 128 (smaller FP32 partials, double-buffered accumulators), others 256.
  auto geometry = [&](int cap) {
    pl->n_tile = act_rows <= cap ? (act_rows + 15) / 16 * 16 : cap;
    if (pl->n_tile < 16) pl->n_tile = 16;
    pl->tok_per_tile = layout == RI_GEMM_ROW_PAIR ? pl->n_tile / 2 : pl->n_tile;
    pl->tok_tiles = (act_rows + pl->n_tile - 1) / pl->n_tile;
    pl->tiles = pl->w_tiles * pl->tok_tiles;
    pl->units = (long long)pl->tiles * pl->k_tiles;
  };
  // Plan choice for splits == 0: a cost model fitted to measurements on B200 (microseconds).
  //   * an SM pulls weight bytes (HBM) at about 58 GB/s while up to ~96 CTAs stream and 44 GB/s when
  //     all SMs do (the HBM ceiling is shared), and activation tiles (L2) at about 120 GB/s;
  //   * a plan that splits K pays for the exchange of FP32 partials: about 3 us + 0.04 us per
  //     accumulator column when every CTA owns one even slice of one tile, 4 us + 0.06 us per column
  //     for ragged ranges (more contributors per tile, two partials per CTA);
  //   (constants re-fitted with 512-element stages on the tensor-parallel shards of the benchmark shapes at
  //   M = 1, 16, 64: the plan chosen is within 6 % of the best of splits 1..4 on all 36 cases, 0.4 % on average;
  //   the constants of the 256-element kernel, 42 / 35 GB/s and 2 + 0.02 / 3 + 0.05 us, lost 7 % on average there)
  //   * the output pass costs about 0.75 us per 32 accumulator columns.
  // Candidates: whole tiles per CTA; even K splits s = 2 .. SMs / tiles; ragged ranges on every SM.
  const double w_unit_kb = (pl->ks * kTileW * kTileKBytes + pl->chunks * 512) / 1024.0;
  auto act_unit_kb = [&](int n_tile) { return halves_c * (pl->ks * n_tile * kTileKBytes + pl->chunks * 512 * ((n_tile + 127) / 128)) / 1024.0; };
  auto stream_us = [&](double units_per_cta, int ctas, int n_tile) {
    const double rate = ctas <= 96 ? 58.0 : 44.0;
    return units_per_cta * (w_unit_kb / rate + act_unit_kb(n_tile) / 120.0);     // KB / (GB/s) = us
  };
  auto epi_us = [&](int n_tile) { return 0.75 * ((n_tile + 31) / 32); };
  // two-CTA tiles: 256 weight rows x 256 accumulator columns per pair, (SMs / 2) pairs at a time
  auto pair_geometry = [&]() {
    geometry(256);
    pl->pair = 1;
    pl->tiles = ((pl->w_tiles + 1) / 2) * pl->tok_tiles;
    pl->units = (long long)pl->tiles * pl->k_tiles;
    pl->tile_granular = 1;
    const int slots = g_pair_slots[g_plan_device] > 0 ? g_pair_slots[g_plan_device] : sm_count / 2;
    pl->grid = pl->tiles < slots ? pl->tiles : slots;
  };
  auto pair_eligible = [&]() {
    geometry(256);
    return pl->n_tile == 256 && pl->w_tiles >= 2 && sm_count >= 2;
  };
  if (splits == 1 || (splits == -2 && !pair_eligible())) {
    geometry(256);
    pl->tile_granular = 1;
    pl->grid = pl->tiles < sm_count ? pl->tiles : sm_count;
  } else if (splits == -2) {
    pair_geometry();
  } else if (splits <= 0) {
    geometry(256);
    const int grid_t = pl->tiles < sm_count ? pl->tiles : sm_count;
    const double waves = double((pl->tiles + grid_t - 1) / grid_t);
    // (with two accumulator buffers the output pass of a tile runs under the next tile's K loop: only the
    // last one is exposed)
    double best = stream_us(waves * pl->k_tiles, grid_t, pl->n_tile) + (pl->n_tile <= 128 ? 1.0 : waves) * epi_us(pl->n_tile);
    int best_split = 1;                                   // 1 = whole tiles, -1 = ragged ranges, s > 1 = even split
    geometry(128);
    if (pl->units >= 2) {
      for (int s = 2; s * pl->tiles <= sm_count && s <= pl->k_tiles; ++s) {
        const double upc = double((pl->k_tiles + s - 1) / s);
        const double c = stream_us(upc, s * pl->tiles, pl->n_tile) + epi_us(pl->n_tile) + 3.0 + 0.04 * pl->n_tile;
        if (c < best) { best = c; best_split = s; }
      }
      long long g = sm_count;
      if (pl->units / 2 < g) g = pl->units / 2;                 // at least two K tiles per CTA
      if (g > 0 && pl->tiles % g != 0) {
        const double c = stream_us(double(pl->units) / g, int(g), pl->n_tile) + epi_us(pl->n_tile) + 4.0 + 0.06 * pl->n_tile;
        if (c < best) { best = c; best_split = -1; }
      }
    }
    if (pair_eligible() && pl->tok_tiles >= 2) {
      // a CTA of a pair takes in half of the activation tile per weight tile; measured: no gain while all
      // tokens fit one tile (the K loop is short and latency-bound either way), 10-20 % with several tiles
      const int pair_tiles = ((pl->w_tiles + 1) / 2) * pl->tok_tiles;
      const int slots = g_pair_slots[g_plan_device] > 0 ? g_pair_slots[g_plan_device] : sm_count / 2;
      const int grid_p = pair_tiles < slots ? pair_tiles : slots;
      const double waves_p = double((pair_tiles + grid_p - 1) / grid_p);
      const double act_kb = halves_c * (128 * kTileKBytes + pl->chunks * 512 * 2) / 1024.0;
      const double rate = 2 * grid_p <= 96 ? 58.0 : 44.0;
      const double c = waves_p * pl->k_tiles * (w_unit_kb / rate + act_kb / 120.0) + waves_p * epi_us(256) + 1.0;
      if (c < best) { best = c; best_split = -2; }
    }
    if (best_split == -2) {
      pair_geometry();
    } else if (best_split == 1) {
      geometry(256);
      pl->tile_granular = 1;
      pl->grid = grid_t;
    } else if (best_split > 1) {
      geometry(128);
      pl->tile_granular = 0;
      pl->grid = best_split * pl->tiles;
    } else {
      geometry(128);
      pl->tile_granular = 0;
      long long g = sm_count;
      if (pl->units / 2 < g) g = pl->units / 2;
      pl->grid = int(g);
    }
  } else {
    geometry(128);
    pl->tile_granular = 0;
    long long g = (long long)pl->tiles * splits;
    if (g > sm_count) g = sm_count;
    if (g > pl->units) g = pl->units;
    pl->grid = int(g);
  }
  if (!pl->tile_granular && pl->grid <= pl->tiles && pl->tiles % pl->grid == 0) pl->tile_granular = 1;
  const int halves = layout == RI_GEMM_CONCAT_K ? 2 : 1;
  const int row_tiles = (pl->n_tile + 127) / 128;
  const int sf_bytes = pl->chunks * 512;
  pl->smem_act_off = pl->ks * kTileW * kTileKBytes;
  pl->smem_sfa_off = pl->smem_act_off + halves * pl->ks * (pl->pair ? pl->n_tile / 2 : pl->n_tile) * kTileKBytes;
  pl->smem_sfb_off = pl->smem_sfa_off + sf_bytes;
  int stage = pl->smem_sfb_off + halves * row_tiles * sf_bytes;
  pl->stage_bytes = (stage + 1023) / 1024 * 1024;
  const int budget = kMaxDynSmem - 1024 - kEpiStageBytes;   // 1 KB of slack to align the tiles to 1024 bytes
  int stages = budget / pl->stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return RI_ERR_UNSUPPORTED;
  pl->stages = stages;
  pl->smem_total = stages * pl->stage_bytes + kEpiStageBytes + 1024;
  return RI_OK;
}

int64_t partial_bytes(const Plan& pl) {
  return pl.tile_granular ? 0 : int64_t(pl.grid) * 2 * kTileW * pl.n_tile * 4;
}

#ifdef RI_GEMM_TRACE
long long* g_trace = nullptr;
#endif

}  // namespace
}  // namespace ri

using namespace ri;

#ifdef RI_GEMM_TRACE
extern "C" void ri_fp4_gemm_set_trace(int64_t* device_buffer) { g_trace = reinterpret_cast<long long*>(device_buffer); }
#endif

extern "C" int64_t ri_fp4_gemm_counter_bytes(int m, int n) {
  (void)m;
  // one ticket per output tile; sized for the smallest tile the planner uses
  const int64_t w_tiles = (int64_t(n) + kTileW - 1) / kTileW;
  const int64_t tok_tiles = (2 * int64_t(m) + 127) / 128;
  return (w_tiles * tok_tiles * 4 + 255) / 256 * 256;
}

extern "C" int ri_fp4_gemm_auto_splits(int m, int n, int k, int fmt, int layout) {
  if (m <= 0) return 1;
  DeviceInfo di;
  int sms = 148;                                   // planning without a visible device assumes a B200
  if (device_info(&di) == 0) sms = di.sm_count;
  Plan pl;
  if (make_plan(m, n, k, fmt, layout, 0, sms, &pl)) return -1;
  return pl.tile_granular ? 1 : (pl.grid + pl.tiles - 1) / pl.tiles + (pl.grid % pl.tiles ? 1 : 0);
}

extern "C" int64_t ri_fp4_gemm_workspace_bytes(int m, int n, int k, int fmt, int layout, int splits) {
  if (splits == 1 || m <= 0) return 0;
  // The plan depends on the SM count.  The size returned covers the plan of the device in use (when one
  // is visible) and the plan of a full 148-SM part, so that a launch never finds the workspace short.
  DeviceInfo di;
  int counts[2] = {148, 148};
  if (device_info(&di) == 0) counts[1] = di.sm_count;
  int64_t partial = 0;
  for (int i = 0; i < 2; ++i) {
    Plan pl;
    if (make_plan(m, n, k, fmt, layout, splits, counts[i], &pl)) return -1;
    if (pl.tile_granular) continue;
    const int sms = counts[i] > 148 ? counts[i] : 148;     // room for a grid of every SM, whatever the planner picks
    const int64_t bytes = int64_t(sms) * 2 * kTileW * pl.n_tile * 4;
    if (bytes > partial) partial = bytes;
  }
  return partial ? ri_fp4_gemm_counter_bytes(m, n) + partial : 0;
}

extern "C" int ri_fp4_gemm_allreduce_uses_pairs(int m, int n, int world);

namespace ri {
namespace {
// the ranks of a fused all-reduce (ri_fp4_gemm_allreduce); null for a plain launch
struct ArArgs {
  void* const* rank_inboxes;
  int64_t inbox_area;                  // BF16 elements between the areas of consecutive source ranks
  void* const* rank_flags;
  void* tile_calls;
  int64_t max_tiles;
  int rank, world;
  void* reduced_out;
  int64_t reduced_row_stride;
};

int gemm_launch(const uint8_t* act, int64_t act_row_bytes, const uint8_t* act_sf,
                int64_t act_sf_bytes, const uint8_t* w, int64_t w_row_bytes,
                const uint8_t* w_sf, int64_t w_sf_bytes, const float* alpha, int n_alpha,
                void* out, int out_dtype, int64_t out_row_stride, int m, int n, int k,
                int fmt, int layout, int splits, void* workspace, int64_t workspace_bytes,
                int32_t* status, int enable_pdl, void* stream, const ArArgs* ar) {
  RI_CHECK_ARG(fmt == RI_FMT_NVFP4 || fmt == RI_FMT_MXFP4, "unknown FP4 format: %d", fmt);
  RI_CHECK_ARG(layout >= RI_GEMM_PLAIN && layout <= RI_GEMM_CONCAT_K, "unknown activation layout %d", layout);
  RI_CHECK_ARG(m >= 0 && n > 0 && k > 0, "positive dimensions required");
  RI_CHECK_ARG(k % (fmt == RI_FMT_NVFP4 ? 64 : 128) == 0, "K must be a multiple of %d (got %d)",
               fmt == RI_FMT_NVFP4 ? 64 : 128, k);
  RI_CHECK_ARG(layout != RI_GEMM_CONCAT_K || k % 256 == 0, "the concat_k layout needs K %% 256 == 0 (got %d)", k);
  RI_CHECK_ARG(out_dtype == RI_DTYPE_BF16 || out_dtype == RI_DTYPE_FP16 || out_dtype == RI_DTYPE_F32,
               "output must be bf16 or fp16");
  RI_CHECK_ARG(out_row_stride >= n, "output row stride smaller than N");
  RI_CHECK_ARG(w_row_bytes >= k / 2 && w_row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
               "weight rows must be 16-byte aligned with stride >= K/2 (stride %lld)", (long long)w_row_bytes);
  const int vec = fmt == RI_FMT_NVFP4 ? 16 : 32;
  const int act_rows = layout == RI_GEMM_ROW_PAIR ? 2 * m : m;
  const int64_t act_cols = layout == RI_GEMM_CONCAT_K ? int64_t(k) : k / 2;       // bytes
  const int act_k_total = layout == RI_GEMM_CONCAT_K ? 2 * k : k;
  RI_CHECK_ARG(act_row_bytes >= act_cols && act_row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(act) & 15) == 0,
               "activation must be compact 16-byte aligned rows of %lld bytes; got stride %lld",
               (long long)act_cols, (long long)act_row_bytes);
  RI_CHECK_ARG(n_alpha >= 0 && n_alpha <= 2 && (n_alpha < 2 || layout == RI_GEMM_ROW_PAIR),
               "a separate residue alpha needs the row_pair layout");
  RI_CHECK_ARG(fmt == RI_FMT_NVFP4 || alpha == nullptr, "MXFP4 has no global scale");
  const int64_t w_chunks = (int64_t(k) + 4 * vec - 1) / (4 * vec);
  const int64_t act_chunks = (int64_t(act_k_total) + 4 * vec - 1) / (4 * vec);
  const int64_t need_wsf = ((int64_t(n) + 127) / 128) * w_chunks * 512;
  const int64_t act_row_tiles = (int64_t(act_rows) + 127) / 128;
  RI_CHECK_ARG(w_sf_bytes >= need_wsf, "expected a 128x4 weight scale buffer of %lld bytes, got %lld",
               (long long)need_wsf, (long long)w_sf_bytes);
  RI_CHECK_ARG(act_sf_bytes >= act_row_tiles * act_chunks * 512,
               "expected a 128x4 activation scale buffer of %lld bytes, got %lld",
               (long long)(act_row_tiles * act_chunks * 512), (long long)act_sf_bytes);
  RI_CHECK_ARG((reinterpret_cast<uintptr_t>(w_sf) & 15) == 0 && (reinterpret_cast<uintptr_t>(act_sf) & 15) == 0,
               "scale buffers must be 16-byte aligned");
  if (m == 0) return RI_OK;

  DeviceInfo di;
  int s = device_info(&di);
  if (s) return s;
  g_plan_device = di.ordinal;
  if (g_pair_slots[di.ordinal] == 0) {
    // how many two-CTA clusters of this kernel the device holds at once (GPC shapes decide, not SMs / 2 alone)
    RI_CUDA(cudaFuncSetAttribute(fp4_gemm_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem));
    cudaLaunchConfig_t q{};
    q.gridDim = dim3(2 * di.sm_count);
    q.blockDim = dim3(kThreads);
    q.dynamicSmemBytes = kMaxDynSmem;
    cudaLaunchAttribute ca{};
    ca.id = cudaLaunchAttributeClusterDimension;
    ca.val.clusterDim.x = 2; ca.val.clusterDim.y = 1; ca.val.clusterDim.z = 1;
    q.attrs = &ca;
    q.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, fp4_gemm_kernel<false, true>, &q) != cudaSuccess || clusters <= 0) {
      (void)cudaGetLastError();
      clusters = di.sm_count / 2;
    }
    g_pair_slots[di.ordinal] = clusters;
  }
  Plan pl;
  s = make_plan(m, n, k, fmt, layout, splits, di.sm_count, &pl);
  if (s) {
    set_error("no tile plan for M=%d N=%d K=%d", m, n, k);
    return s;
  }
  float* ws_partial = nullptr;
  int* ws_counter = nullptr;
  if (!pl.tile_granular) {
    const int64_t counter_bytes = ri_fp4_gemm_counter_bytes(m, n);
    const int64_t partial = partial_bytes(pl);
    RI_CHECK_ARG(workspace != nullptr && workspace_bytes >= counter_bytes + partial,
                 "the K-split plan (%d CTAs over %d tiles) needs a workspace of %lld bytes, got %lld", pl.grid,
                 pl.tiles, (long long)(counter_bytes + partial), (long long)workspace_bytes);
    RI_CHECK_ARG((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "workspace must be 256-byte aligned");
    RI_CHECK_ARG(int64_t(pl.tiles) * 4 <= counter_bytes, "internal: counter area too small");
    ws_counter = static_cast<int*>(workspace);
    ws_partial = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + counter_bytes);
  }

  CUtensorMap w_map, act_map;
  int map3 = 0;
  if (pl.ks > 1 && k % 256 == 0 && act_cols == k / 2) {       // every 128-byte sub-tile whole: one copy per stage and operand
    map3 = make_map_subtiles(&w_map, w, uint64_t(k / 2), uint64_t(n), uint64_t(w_row_bytes), kTileW, pl.ks) == RI_OK &&
           make_map_subtiles(&act_map, act, uint64_t(act_cols), uint64_t(act_rows), uint64_t(act_row_bytes),
                             uint32_t(pl.n_tile), pl.ks) == RI_OK;
  }
  if (!map3) {
    s = make_map(&w_map, w, uint64_t(k / 2), uint64_t(n), uint64_t(w_row_bytes), kTileW);
    if (s) return s;
    s = make_map(&act_map, act, uint64_t(act_cols), uint64_t(act_rows), uint64_t(act_row_bytes),
                 uint32_t(pl.pair ? pl.n_tile / 2 : pl.n_tile));
    if (s) return s;
  }

  GemmParams p{};
  p.m = m; p.n = n; p.k = k; p.fmt = fmt; p.layout = layout;
  p.n_tile = pl.n_tile; p.tok_per_tile = pl.tok_per_tile; p.act_rows = act_rows;
  p.k_tiles = pl.k_tiles; p.tiles = pl.tiles; p.tok_tiles = pl.tok_tiles; p.units = pl.units;
  p.grid = pl.grid; p.tile_granular = pl.tile_granular;
  p.stages = pl.stages; p.chunks = pl.chunks;
  {
    const int halves_h = layout == RI_GEMM_CONCAT_K ? 2 : 1;
    const int row_tiles_h = (pl.n_tile + 127) / 128;
    p.sf_set_cols = 16 * pl.ks + pl.chunks * halves_h * row_tiles_h * 4;
    // one scale set per pipeline stage if tensor memory has room for at least two (the scale warps then
    // need no second wait per K tile); the stage count is trimmed to the sets that fit
    const int sets_max = (kTmemCols - kSfCol) / p.sf_set_cols;
    if (sets_max >= 2) {
      if (p.stages > sets_max) p.stages = sets_max;
      if (p.stages > kMaxSfSets) p.stages = kMaxSfSets;
      p.sf_sets = p.stages;
    } else {
      p.sf_sets = 1;
    }
  }
  p.act_row_tiles = int(act_row_tiles);
  p.w_sf_tile_stride = w_chunks * 512;
  p.act_sf_tile_stride = act_chunks * 512;
  p.act_res_chunk0 = int(k / (4 * vec));
  p.act_res_col0 = k / 2;
  p.w_sf = w_sf; p.act_sf = act_sf; p.alpha = alpha; p.n_alpha = alpha ? (n_alpha > 0 ? n_alpha : 1) : 0;
  p.out = out; p.out_fp16 = out_dtype == RI_DTYPE_F32 ? 2 : (out_dtype == RI_DTYPE_FP16 ? 1 : 0); p.out_stride = out_row_stride;
  p.ws_partial = ws_partial; p.ws_counter = ws_counter; p.status = status;
  p.smem_act_off = pl.smem_act_off; p.smem_sfa_off = pl.smem_sfa_off; p.smem_sfb_off = pl.smem_sfb_off;
  p.stage_bytes = pl.stage_bytes;
  p.map3 = map3;
#ifdef RI_GEMM_TRACE
  p.trace = g_trace;
#endif
  if (ar) {
    // flag entries are indexed by (128-row weight tile, token tile); a two-CTA plan rounds the weight tiles up to pairs
    const int64_t w_tiles_flag = pl.pair ? 2 * ((int64_t(n) + 2 * kTileW - 1) / (2 * kTileW)) : (int64_t(n) + kTileW - 1) / kTileW;
    RI_CHECK_ARG(w_tiles_flag * pl.tok_tiles <= ar->max_tiles,
                 "the fused all-reduce needs %lld tile flags, the flag arrays hold %lld",
                 (long long)(w_tiles_flag * pl.tok_tiles), (long long)ar->max_tiles);
    for (int r = 0; r < ar->world; ++r) {
      // an area holds inbox_area elements of 4 bytes (room for the pairs); plain BF16 tiles use its first half
      p.ar_push[r] = reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(ar->rank_inboxes[r]) + int64_t(ar->rank) * ar->inbox_area * 4);
      p.ar_pull[r] = reinterpret_cast<const uint4*>(static_cast<uint8_t*>(ar->rank_inboxes[ar->rank]) + int64_t(r) * ar->inbox_area * 4);
      p.ar_flags[r] = static_cast<uint32_t*>(ar->rank_flags[r]);
    }
    p.ar_epoch = static_cast<uint32_t*>(ar->tile_calls);
    p.ar_state = p.ar_epoch + ar->max_tiles;            // two words behind the per-tile counts
    // small partials travel as (value, call number) pairs: twice the bytes, no fences
    p.ar_ll = ri_fp4_gemm_allreduce_uses_pairs(m, n, ar->world);
    p.ar_out = ar->reduced_out;
    p.ar_out_stride = ar->reduced_row_stride;
    p.ar_wait_ns = peer_wait_ns();
    p.ar_rank = ar->rank;
    p.ar_world = ar->world;
  }

  const bool mxk = fmt == RI_FMT_MXFP4;
  auto kernel = pl.pair ? (mxk ? fp4_gemm_kernel<true, true> : fp4_gemm_kernel<false, true>)
                        : (mxk ? fp4_gemm_kernel<true, false> : fp4_gemm_kernel<false, false>);
  if (ar)                                           // the variant whose epilogue sums over the ranks
    kernel = pl.pair ? (mxk ? fp4_gemm_kernel<true, true, true> : fp4_gemm_kernel<false, true, true>)
                     : (mxk ? fp4_gemm_kernel<true, false, true> : fp4_gemm_kernel<false, false, true>);
  if (pl.ks == 2) {                                 // 512-element stages (never with two-CTA tiles)
    kernel = mxk ? fp4_gemm_kernel<true, false, false, 2> : fp4_gemm_kernel<false, false, false, 2>;
    if (ar) kernel = mxk ? fp4_gemm_kernel<true, false, true, 2> : fp4_gemm_kernel<false, false, true, 2>;
  }
  static bool attr_set[64][2][2][2][5] = {};        // function attributes are per device
  if (!attr_set[di.ordinal][fmt][pl.pair][ar ? 1 : 0][pl.ks]) {
    RI_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem));
    attr_set[di.ordinal][fmt][pl.pair][ar ? 1 : 0][pl.ks] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pl.pair ? 2 * pl.grid : pl.grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = pl.smem_total;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attrs[2]{};
  int n_attrs = 0;
  if (enable_pdl) {
    attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
    ++n_attrs;
  }
  if (pl.pair) {                                    // the two CTAs of a pair form a cluster
    attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
    attrs[n_attrs].val.clusterDim.x = 2;
    attrs[n_attrs].val.clusterDim.y = 1;
    attrs[n_attrs].val.clusterDim.z = 1;
    ++n_attrs;
  }
  cfg.attrs = n_attrs ? attrs : nullptr;
  cfg.numAttrs = n_attrs;
  return cuda_status(cudaLaunchKernelEx(&cfg, kernel, w_map, act_map, p), "fp4 gemm launch");
}
}  // namespace
}  // namespace ri

extern "C" int ri_fp4_gemm(const uint8_t* act, int64_t act_row_bytes, const uint8_t* act_sf,
                           int64_t act_sf_bytes, const uint8_t* w, int64_t w_row_bytes,
                           const uint8_t* w_sf, int64_t w_sf_bytes, const float* alpha, int n_alpha,
                           void* out, int out_dtype, int64_t out_row_stride, int m, int n, int k,
                           int fmt, int layout, int splits, void* workspace, int64_t workspace_bytes,
                           int32_t* status, int enable_pdl, void* stream) {
  return ri::gemm_launch(act, act_row_bytes, act_sf, act_sf_bytes, w, w_row_bytes, w_sf, w_sf_bytes, alpha, n_alpha, out,
                         out_dtype, out_row_stride, m, n, k, fmt, layout, splits, workspace, workspace_bytes, status,
                         enable_pdl, stream, nullptr);
}

extern "C" int64_t ri_fp4_gemm_allreduce_tiles(int m, int n) {
  // an upper bound of the (weight tile, token tile) pairs of any plan for the shape, weight tiles rounded to pairs
  const int64_t w_tiles = 2 * ((int64_t(n) + 2 * ri::kTileW - 1) / (2 * ri::kTileW));
  const int64_t tok_tiles = (2 * int64_t(m < 1 ? 1 : m) + 15) / 16;
  return w_tiles * tok_tiles;
}
extern "C" int ri_fp4_gemm_allreduce_uses_pairs(int m, int n, int world) {
  return int64_t(world - 1) * m * n * 4 <= ri::kArPairBytesMax ? 1 : 0;
}
extern "C" int64_t ri_fp4_gemm_allreduce_flag_bytes(int64_t max_tiles) { return max_tiles * ri::kArMaxRanks * 4; }
extern "C" int64_t ri_fp4_gemm_allreduce_call_bytes(int64_t max_tiles) { return (max_tiles + 2) * 4; }

extern "C" int ri_fp4_gemm_allreduce(const uint8_t* act, int64_t act_row_bytes, const uint8_t* act_sf,
                                     int64_t act_sf_bytes, const uint8_t* w, int64_t w_row_bytes,
                                     const uint8_t* w_sf, int64_t w_sf_bytes, const float* alpha, int n_alpha,
                                     int64_t partial_row_stride, int m, int n, int k, int fmt, int layout, int splits,
                                     void* workspace, int64_t workspace_bytes, int32_t* status, int enable_pdl,
                                     void* stream, void* const* rank_inboxes, int64_t inbox_area,
                                     void* const* rank_flags, void* tile_calls, int64_t max_tiles, int rank, int world,
                                     void* reduced_out, int64_t reduced_row_stride) {
  using namespace ri;
  RI_CHECK_ARG(world >= 2 && world <= kArMaxRanks && rank >= 0 && rank < world, "bad rank %d / world %d (2..%d ranks)",
               rank, world, kArMaxRanks);
  RI_CHECK_ARG(rank_inboxes && rank_flags && tile_calls && reduced_out && max_tiles > 0, "null argument");
  for (int r = 0; r < world; ++r)
    RI_CHECK_ARG(rank_inboxes[r] && rank_flags[r] && (reinterpret_cast<uintptr_t>(rank_inboxes[r]) & 15) == 0,
                 "rank %d: buffers must be mapped and 16-byte aligned", r);
  RI_CHECK_ARG(n % 8 == 0 && partial_row_stride % 8 == 0 && partial_row_stride >= n && reduced_row_stride % 8 == 0 &&
                   reduced_row_stride >= n && inbox_area % 8 == 0 && (reinterpret_cast<uintptr_t>(reduced_out) & 15) == 0,
               "the fused all-reduce moves 16-byte vectors: N, the row strides and the inbox areas must be multiples of 8");
  RI_CHECK_ARG(inbox_area >= int64_t(m) * partial_row_stride, "an inbox area of %lld elements is too small for [%d, %lld]",
               (long long)inbox_area, m, (long long)partial_row_stride);
  ArArgs ar{rank_inboxes, inbox_area, rank_flags, tile_calls, max_tiles, rank, world, reduced_out, reduced_row_stride};
  void* own_area = static_cast<uint8_t*>(rank_inboxes[rank]) + int64_t(rank) * inbox_area * 4;
  return gemm_launch(act, act_row_bytes, act_sf, act_sf_bytes, w, w_row_bytes, w_sf, w_sf_bytes, alpha, n_alpha, own_area,
                     RI_DTYPE_BF16, partial_row_stride, m, n, k, fmt, layout, splits, workspace, workspace_bytes, status,
                     enable_pdl, stream, &ar);
}
