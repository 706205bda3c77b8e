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
  uint32_t* state;                  // local: [0] calls completed so far, [1] block ticket
  int32_t* status;
  int64_t n16;                      // 16-byte units (8 BF16 values) to reduce
  long long wait_ns;                // how long a block waits for the peers before it gives up
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

__global__ void __launch_bounds__(kArThreads) peer_allreduce_kernel(const PeerArParams p) {
  __shared__ int ok;
  // launched with programmatic stream serialisation: the partial is the previous kernel's output
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(p.state) + 1;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const int r = threadIdx.x;
    // The partial was written by the previous kernel of this stream.  Block 0 announces it to every rank
    // (this one included) ...
    if (blockIdx.x == 0) {
      __threadfence_system();
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[r] + p.rank), "r"(epoch) : "memory");
    }
    // ... and every block waits until every rank has announced this call, for at most p.wait_ns.
    const uint32_t* mine = p.flags[p.rank] + r;
    const long long t0 = global_ns();
    for (uint32_t spin = 0;; ++spin) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (int32_t(seen - epoch) >= 0) break;
      if ((spin & 255u) == 255u && global_ns() - t0 > p.wait_ns) {
        ok = 0;
        if (p.status) atomicExch(p.status, 0x40000000 | (r << 8) | p.rank);    // which peer never arrived
        break;
      }
    }
  }
  __syncthreads();
  if (ok) {
    for (int64_t i = int64_t(blockIdx.x) * kArThreads + threadIdx.x; i < p.n16; i += int64_t(gridDim.x) * kArThreads) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < p.world; ++r) {
        uint4 v;
        asm volatile("ld.global.cv.v4.u32 {%0, %1, %2, %3}, [%4];"       // never from a stale line of this GPU's caches
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p.data[r] + i));
        add8(acc, v);
      }
      uint4 o;
      uint32_t* ow = &o.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        ow[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
      p.out[i] = o;
    }
  } else {
    // a peer never arrived: the status word says which one; the output gets a defined value, this rank's
    // own partial, instead of whatever the buffer held
    for (int64_t i = int64_t(blockIdx.x) * kArThreads + threadIdx.x; i < p.n16; i += int64_t(gridDim.x) * kArThreads)
      p.out[i] = p.data[p.rank][i];
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
extern "C" int64_t ri_peer_allreduce_flag_bytes(void) { return ri::kMaxRanks * 4; }
extern "C" int64_t ri_peer_allreduce_state_bytes(void) { return 8; }

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
  DeviceInfo di;
  int s = device_info(&di);
  if (s) return s;
  const int64_t want = (p.n16 + kArThreads - 1) / kArThreads;
  const int grid = int(want < 1 ? 1 : (want > di.sm_count ? di.sm_count : want));
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
