// One-shot all-reduce of the row-parallel partial outputs over peer memory (NVLink): every rank
// has written its fp16 partial [M, N] into its own region of a buffer that all ranks of the node
// have mapped; each rank then reads every rank's partial with plain loads, adds them in rank
// order in fp32 (the same order on every rank: results are identical everywhere and from run to
// run) and writes the fp16 sum to local memory.  It replaces, for the small messages of decode
// and short prefill, the NCCL all-reduce behind vLLM's RowParallelLinear
// (model_executor/layers/linear.py:1556-1559, distributed/device_communicators/
// custom_all_reduce.py:232-245).  No multicast objects, no TMA: ld/st only.
//
// Synchronisation: per block and per peer one 32-bit flag in the peer's region, written with
// st.release.sys and polled with relaxed system-scope loads followed by one acquire fence.  Flags carry the call number (kept in local
// device memory and advanced by the last block of every call, so CUDA-graph replays need no host
// value), compared with >=, so a peer that is already one call ahead does not confuse a slow
// block.  Every poll loop has an iteration limit; when it runs out the kernel records a status
// code, skips its reads and returns.
#include "common.cuh"

namespace awq {
namespace {

static __device__ int g_ar_status = 0;
static uint32_t g_ar_spin_limit = 1u << 22;

constexpr int kArThreads = 512;

struct ArParams {
  const uint4* data[AWQ_B200_AR_MAX_RANKS];   // every rank's partial, as mapped here
  uint32_t* flags[AWQ_B200_AR_MAX_RANKS];     // every rank's flag area, as mapped here
  uint4* out;
  uint32_t* state;   // local: [0] calls completed, [1] blocks finished in this call
  int64_t n16;       // 16-byte units
  int rank, world;
  uint32_t spin_limit;
  int end_barrier;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_acquire_sys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}

// flag index of (phase, block, writer rank) inside one rank's flag area
__device__ __forceinline__ int flag_index(int phase, int block, int writer) {
  return (phase * AWQ_B200_AR_MAX_BLOCKS + block) * AWQ_B200_AR_MAX_RANKS + writer;
}

// Tell every peer "this block of mine has reached `phase` of call `epoch`", then wait until every
// peer's same block has said so.  Returns false when a wait ran out.
__device__ __forceinline__ bool peer_barrier(const ArParams& p, int phase, uint32_t epoch,
                                             int* s_abort) {
  const int t = threadIdx.x, b = blockIdx.x;
  if (t < p.world && t != p.rank) {
    // release at system scope: everything this thread has observed (the partial written by the
    // kernel before this one, the loads of this block before the barrier above) is ordered first
    st_release_sys(p.flags[t] + flag_index(phase, b, p.rank), epoch);
    const uint32_t* mine = p.flags[p.rank] + flag_index(phase, b, t);
    bool ok = false;
    for (uint32_t i = 0; i < p.spin_limit; ++i) {
      // relaxed polls, one acquire fence once the flag is there
      if ((int32_t)(ld_relaxed_sys(mine) - epoch) >= 0) {
        fence_acquire_sys();
        ok = true;
        break;
      }
      if ((i & 63u) == 63u && *(volatile int*)s_abort) break;
    }
    if (!ok) {
      *(volatile int*)s_abort = 1;
      atomicCAS(&g_ar_status, 0, 70 + 10 * phase + t);   // 7x: start barrier, 8x: end barrier
    }
  }
  __syncthreads();
  return *(volatile int*)s_abort == 0;
}

__global__ void __launch_bounds__(kArThreads) allreduce_oneshot_kernel(ArParams p) {
  // with programmatic dependent launch: everything the producer of the partial wrote is visible
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  const uint32_t epoch = *(volatile uint32_t*)p.state + 1;
  if (peer_barrier(p, 0, epoch, &s_abort)) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.n16; i += stride) {
      uint4 v[AWQ_B200_AR_MAX_RANKS];
#pragma unroll
      for (int r = 0; r < AWQ_B200_AR_MAX_RANKS; ++r)
        if (r < p.world) v[r] = __ldcg(p.data[r] + i);
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
      for (int r = 0; r < AWQ_B200_AR_MAX_RANKS; ++r) {
        if (r < p.world) {
          const __half2* h = reinterpret_cast<const __half2*>(&v[r]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        }
      }
      uint4 o;
      __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
      p.out[i] = o;
    }
    // a caller that reuses the same region in its next call must not overwrite it while a peer
    // still reads it
    if (p.end_barrier) {
      __syncthreads();
      peer_barrier(p, 1, epoch, &s_abort);
    }
  }
  // the last block to finish advances the call counter (every block has read it by then)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t ticket = atomicAdd(p.state + 1, 1u);
    if (ticket == gridDim.x - 1) {
      p.state[1] = 0;
      __threadfence();
      *(volatile uint32_t*)p.state = epoch;
    }
  }
}

}  // namespace

void ar_set_spin_limit(uint32_t polls) { g_ar_spin_limit = polls ? polls : (1u << 22); }

int ar_device_status(int* out, int clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_ar_status, sizeof(int)) != cudaSuccess) return AWQ_B200_ERR_LAUNCH;
  if (clear && v != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_ar_status, &zero, sizeof(int)) != cudaSuccess)
      return AWQ_B200_ERR_LAUNCH;
  }
  *out = v;
  return AWQ_B200_OK;
}

int launch_allreduce(const void* const* regions, size_t data_offset, void* out, size_t bytes,
                     void* state, int rank, int world, int flags, cudaStream_t stream) {
  ArParams p{};
  for (int r = 0; r < world; ++r) {
    const char* base = static_cast<const char*>(regions[r]);
    p.flags[r] = reinterpret_cast<uint32_t*>(const_cast<char*>(base));
    p.data[r] = reinterpret_cast<const uint4*>(base + data_offset);
  }
  p.out = static_cast<uint4*>(out);
  p.state = static_cast<uint32_t*>(state);
  p.n16 = (int64_t)(bytes / 16);
  p.rank = rank;
  p.world = world;
  p.spin_limit = g_ar_spin_limit;
  p.end_barrier = flags & 1;
  int blocks = (int)((p.n16 + kArThreads - 1) / kArThreads);
  if (blocks > AWQ_B200_AR_MAX_BLOCKS) blocks = AWQ_B200_AR_MAX_BLOCKS;
  if (blocks < 1) blocks = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(kArThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  cfg.attrs = attr;
  cfg.numAttrs = (flags & 2) ? add_pdl_attribute(attr, 0) : 0;
  return cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel, p) == cudaSuccess
             ? AWQ_B200_OK : AWQ_B200_ERR_LAUNCH;
}

}  // namespace awq
