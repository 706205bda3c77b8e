// One-shot all-reduce of small BF16 tensors over peer memory (NVLink), for the row-parallel linears of a
// tensor-parallel decode step: the partial outputs are at most a few MB, so a ring or tree collective is
// all latency.  Every rank keeps its partial in a buffer that the other ranks of the node have mapped
// (CUDA IPC); one kernel per rank tells the peers "my partial of call number e is in place" with a
// system-scope store into their flag arrays, waits (bounded) until every peer has said the same, then
// sums the partials of all ranks with plain peer loads, in rank order, FP32 accumulation, and writes
// the BF16 result to local memory.  The sum is bit-identical on every rank.
//
// No multicast, no multimem, no NCCL.  Only ranks on DIFFERENT GPUs ever wait for each other.
// The reference leaves this step to vLLM's tensor-parallel linear layers (its linear methods,
// quant/vllm_integration/linear_method_v2.py and linear_method_mxfp4.py, return the rank-local partial
// from `apply`; the all-reduce follows in vLLM's RowParallelLinear).
#include "common.cuh"
#include "resinfer_b200.h"

namespace ri {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kArThreads = 512;

struct PeerArParams {
  const uint4* data[kMaxRanks];     // rank r's partial (this process's mapping of it)
  uint32_t* flags[kMaxRanks];       // rank r's flag array [kMaxRanks] (this process's mapping of it)
  uint4* out;                       // local result
  uint32_t* state;                  // local: [0] calls completed so far, [1] block ticket, [2] block ticket of the slice pass
  int32_t* status;
  int64_t n16;                      // 16-byte units (8 BF16 values) to reduce
  long long wait_ns;                // how long a block waits for the peers before it gives up
  int two_shot;                     // sum a slice per rank and exchange the sums (large partials on many ranks)
  int rank, world;
};

__device__ __forceinline__ long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return (long long)t;
}

__device__ __forceinline__ void add8(float (&acc)[8], uint4 v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] += __uint_as_float(w[i] << 16);
    acc[2 * i + 1] += __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

// the BF16 sum of one 16-byte vector over all ranks, rank order, FP32; all loads in flight together (a peer load
// is a 2 - 3 us round trip)
__device__ __forceinline__ uint4 sum_over_ranks(const PeerArParams& p, int64_t i) {
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  uint4 v[kMaxRanks];
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r) {
    if (r < p.world)
      asm volatile("ld.global.cv.v4.u32 {%0, %1, %2, %3}, [%4];"     // never from a stale line of this GPU's caches
                   : "=r"(v[r].x), "=r"(v[r].y), "=r"(v[r].z), "=r"(v[r].w) : "l"(p.data[r] + i));
  }
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r)
    if (r < p.world) add8(acc, v[r]);
  uint4 o;
  uint32_t* ow = &o.x;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    ow[j] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return o;
}

// threads 0 .. world-1 of a block: wait until rank `threadIdx.x` has stored `epoch` into flag slot `slot` of this
// rank's flag array; false (and the status word set) if that takes longer than p.wait_ns
__device__ __forceinline__ void wait_for_peers(const PeerArParams& p, uint32_t epoch, int slot, int* ok) {
  if (threadIdx.x < p.world) {
    const int r = threadIdx.x;
    const uint32_t* mine = p.flags[p.rank] + slot * kMaxRanks + r;
    const long long t0 = global_ns();
    for (uint32_t spin = 0;; ++spin) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (int32_t(seen - epoch) >= 0) break;
      if ((spin & 255u) == 255u && global_ns() - t0 > p.wait_ns) {
        *ok = 0;
        if (p.status) atomicExch(p.status, 0x40000000 | (r << 8) | p.rank);    // which peer never arrived
        break;
      }
    }
  }
}

__global__ void __launch_bounds__(kArThreads, 2) peer_allreduce_kernel(const PeerArParams p) {
  __shared__ int ok;
  __shared__ int last_block;
  // launched with programmatic stream serialisation: the partial is the previous kernel's output
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(p.state) + 1;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  // The partial was written by the previous kernel of this stream.  Block 0 announces it to every rank (this one
  // included; the release store orders the partial ahead of the flag) ...
  if (blockIdx.x == 0 && threadIdx.x < p.world)
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[threadIdx.x] + p.rank), "r"(epoch) : "memory");
  // ... and every block waits until every rank has announced this call, for at most p.wait_ns.
  wait_for_peers(p, epoch, 0, &ok);
  __syncthreads();
  const int64_t stride = int64_t(gridDim.x) * kArThreads;
  const int64_t first = int64_t(blockIdx.x) * kArThreads + threadIdx.x;
  if (!ok) {
    // a peer never arrived: the status word says which one; the output gets a defined value, this rank's
    // own partial, instead of whatever the buffer held
    for (int64_t i = first; i < p.n16; i += stride) p.out[i] = p.data[p.rank][i];
  } else if (!p.two_shot) {
    for (int64_t i = first; i < p.n16; i += stride) p.out[i] = sum_over_ranks(p, i);
  } else {
    // Large partials on many ranks: reading every peer's whole partial is (world - 1) x the bytes.  Instead this
    // rank sums only its own slice of the vectors -- and puts the result back into its own partial buffer, a part
    // no peer reads before the second announcement -- and then fetches the other slices, already summed, from
    // their owners: 2 (world - 1) / world x the bytes, one more hand-shake.
    const int64_t len = (p.n16 + p.world - 1) / p.world;
    const int64_t lo = int64_t(p.rank) * len, hi = lo + len < p.n16 ? lo + len : p.n16;
    uint4* own = const_cast<uint4*>(p.data[p.rank]);
    for (int64_t i = lo + first; i < hi; i += stride) {
      const uint4 o = sum_over_ranks(p, i);
      own[i] = o;
      p.out[i] = o;
    }
    // the last block to finish its part of the slice announces it
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      last_block = atomicAdd(p.state + 2, 1u) == gridDim.x - 1;
      if (last_block) p.state[2] = 0;
    }
    __syncthreads();
    if (last_block && threadIdx.x < p.world && threadIdx.x != p.rank) {
      __threadfence();                                   // the other blocks' stores, observed through the ticket
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[threadIdx.x] + kMaxRanks + p.rank), "r"(epoch) : "memory");
    }
    if (threadIdx.x == p.rank) *(volatile uint32_t*)(p.flags[p.rank] + kMaxRanks + p.rank) = epoch;   // nobody waits for itself
    wait_for_peers(p, epoch, 1, &ok);
    __syncthreads();
    if (ok) {
      // every vector outside this rank's slice from its owner; one load per thread and pass, all of them in flight
      for (int64_t i = first; i < p.n16; i += stride) {
        if (i >= lo && i < hi) continue;
        const int q = int(i / len);
        const uint4* src = p.data[0];                      // (selected with compile-time indices)
#pragma unroll
        for (int r = 1; r < kMaxRanks; ++r)
          if (r == q) src = p.data[r];
        uint4 v;
        asm volatile("ld.global.cv.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src + i));
        p.out[i] = v;
      }
    } else {
      for (int64_t i = first; i < p.n16; i += stride)
        if (i < lo || i >= hi) p.out[i] = p.data[p.rank][i];
    }
  }
  // the last block to finish closes the call: the next launch on this rank sees epoch as "completed"
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t t = atomicAdd(p.state + 1, 1u);
    if (t == gridDim.x - 1) {
      p.state[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(p.state) = epoch;
    }
  }
}

}  // namespace
}  // namespace ri

namespace ri {
namespace {
long long g_wait_ns = 10ll * 1000 * 1000 * 1000;       // ten seconds: rank skew from a first-call module load or a host stall
}
long long peer_wait_ns() { return g_wait_ns; }
}  // namespace ri

extern "C" void ri_peer_allreduce_set_wait_ms(int milliseconds) {
  ri::g_wait_ns = (long long)(milliseconds < 1 ? 1 : milliseconds) * 1000000ll;
}
extern "C" int64_t ri_peer_allreduce_flag_bytes(void) { return 2 * ri::kMaxRanks * 4; }
extern "C" int64_t ri_peer_allreduce_state_bytes(void) { return 16; }

extern "C" int ri_peer_allreduce_bf16(const void* const* rank_data, void* const* rank_flags, int rank, int world,
                                      int64_t numel, void* out, void* state, int32_t* status, void* stream,
                                      int enable_pdl) {
  using namespace ri;
  RI_CHECK_ARG(world >= 2 && world <= kMaxRanks && rank >= 0 && rank < world, "bad rank %d / world %d (2..%d ranks)",
               rank, world, kMaxRanks);
  RI_CHECK_ARG(numel > 0 && numel % 8 == 0, "element count must be a positive multiple of 8, got %lld", (long long)numel);
  RI_CHECK_ARG(rank_data && rank_flags && out && state, "null argument");
  PeerArParams p{};
  for (int r = 0; r < world; ++r) {
    RI_CHECK_ARG(rank_data[r] && rank_flags[r] && (reinterpret_cast<uintptr_t>(rank_data[r]) & 15) == 0,
                 "rank %d: buffers must be mapped and 16-byte aligned", r);
    p.data[r] = static_cast<const uint4*>(rank_data[r]);
    p.flags[r] = static_cast<uint32_t*>(rank_flags[r]);
  }
  RI_CHECK_ARG((reinterpret_cast<uintptr_t>(out) & 15) == 0, "output must be 16-byte aligned");
  p.out = static_cast<uint4*>(out);
  p.state = static_cast<uint32_t*>(state);
  p.status = status;
  p.n16 = numel / 8;
  p.rank = rank;
  p.world = world;
  p.wait_ns = g_wait_ns;
  // one pass reads (world - 1) x the partial over NVLink; from 4 MB of that on, two passes over a slice each are less
  p.two_shot = (int64_t(world - 1) * numel * 2 > (int64_t(4) << 20) && world > 2) ? 1 : 0;
  DeviceInfo di;
  int s = device_info(&di);
  if (s) return s;
  const int64_t want = (p.n16 + kArThreads - 1) / kArThreads;
  // every block must be resident at once (blocks wait for announcements that the last block of a pass makes)
  static int blocks_per_sm = 0;
  if (blocks_per_sm == 0) {
    int b = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, peer_allreduce_kernel, kArThreads, 0) != cudaSuccess || b < 1) {
      (void)cudaGetLastError();
      b = 1;
    }
    blocks_per_sm = b > 2 ? 2 : b;
  }
  const int64_t cap = int64_t(blocks_per_sm) * di.sm_count;
  const int grid = int(want < 1 ? 1 : (want > cap ? cap : want));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kArThreads);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr{};
  if (enable_pdl) {                  // its launch latency then hides under the tail of the kernel that wrote the partial
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  return cuda_status(cudaLaunchKernelEx(&cfg, peer_allreduce_kernel, p), "peer all-reduce launch");
}
