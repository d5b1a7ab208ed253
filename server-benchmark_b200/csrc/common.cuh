// Shared device/host helpers for the AWQ W4A16 kernels (sm_100a only).
#pragma once

#include <atomic>

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/awq_b200.h"

namespace awq {

// Programmatic dependent launch.  The decode kernels are launched with the stream-serialisation
// attribute: when the kernel before them in the stream has let its dependents go (every CTA
// executed pdl_launch_dependents or exited), their CTAs start on whatever SMs are free, set
// their barriers up and prefetch WEIGHTS, which no kernel writes; pdl_wait then blocks until
// the earlier kernel has completed and its writes are visible, and only after it are
// activations read and outputs written.  After a kernel that never lets go, or after a copy,
// the attribute changes nothing.  AWQ_B200_NO_PDL in the environment turns the attribute off.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
inline bool pdl_enabled() {
  static const bool on = getenv("AWQ_B200_NO_PDL") == nullptr;
  return on;
}
// How many clusters of `S` CTAs (x dimension) of `kernel` the GPU holds at once.  A cluster must
// find all its SMs free inside one GPC, so odd sizes pack badly: a grid with more clusters than
// this runs in waves.  `cache` holds one answer per size (0 = not asked yet); an answer the
// runtime cannot give counts as "enough".  The kernel's dynamic shared-memory limit must have
// been raised before the first call.
template <typename Kernel>
inline int resident_clusters(Kernel kernel, int S, int threads, size_t smem,
                             std::atomic<int>* cache) {
  if (S < 1 || S > 8) return 1 << 30;
  const int known = cache[S];
  if (known > 0) return known;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(S, 1024, 1);
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int got = 0;
  if (cudaOccupancyMaxActiveClusters(&got, kernel, &cfg) != cudaSuccess || got <= 0) {
    (void)cudaGetLastError();
    got = 1 << 30;
  }
  cache[S] = got;
  return got;
}

// Plain (non-cluster) launch with the attribute.  The kernel must execute pdl_wait before it
// touches anything an earlier kernel writes or reads.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args);
// Appends the attribute at attr[n]; returns the new attribute count.
inline int add_pdl_attribute(cudaLaunchAttribute* attr, int n) {
  if (!pdl_enabled()) return n;
  attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[n].val.programmaticStreamSerializationAllowed = 1;
  return n + 1;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  cudaLaunchAttribute attr[1];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = add_pdl_attribute(attr, 0);
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

constexpr int kPack = 8;  // int4 values per int32 word

// ---------------------------------------------------------------------------------------
// AWQ nibble order.  Nibble p (LSB first) of a word holds column [0,2,4,6,1,3,5,7][p], so
// for p in 0..3 nibble p is column 2p and nibble p+4 is column 2p+1: the two columns of an
// adjacent pair sit exactly 16 bits apart.  (w >> 4p) & 0x000F000F therefore yields columns
// (2p, 2p+1) in the low/high half of one register.
// ---------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & b) | c
  return r;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

__device__ __forceinline__ __half2 as_half2(uint32_t v) {
  return *reinterpret_cast<__half2*>(&v);
}
__device__ __forceinline__ uint32_t as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }

// One packed word -> 4 registers; register p holds the fp16 values 1024 + q of columns
// (2p, 2p+1).  1024 + q is exact in fp16 (0x6400 | q).
__device__ __forceinline__ void unpack_word_magic(uint32_t w, uint32_t (&r)[4]) {
  constexpr uint32_t kMask = 0x000F000Fu, kMagic = 0x64006400u;
  r[0] = lop3_and_or(w, kMask, kMagic);
  r[1] = lop3_and_or(w >> 4, kMask, kMagic);
  r[2] = lop3_and_or(w >> 8, kMask, kMagic);
  r[3] = lop3_and_or(w >> 12, kMask, kMagic);
}

// (q - z) * s in fp16 for the 8 columns of one word: the difference is exact, the product is
// rounded once.  zmagic[p] = 1024 + z of columns (2p, 2p+1); s2[p] the matching scales.
__device__ __forceinline__ uint4 dequant_word(uint32_t w, const uint32_t (&zmagic)[4],
                                              const __half2 (&s2)[4]) {
  uint32_t q[4];
  unpack_word_magic(w, q);
  uint4 o;
  o.x = as_u32(__hmul2(__hsub2(as_half2(q[0]), as_half2(zmagic[0])), s2[0]));
  o.y = as_u32(__hmul2(__hsub2(as_half2(q[1]), as_half2(zmagic[1])), s2[1]));
  o.z = as_u32(__hmul2(__hsub2(as_half2(q[2]), as_half2(zmagic[2])), s2[2]));
  o.w = as_u32(__hmul2(__hsub2(as_half2(q[3]), as_half2(zmagic[3])), s2[3]));
  return o;
}

// Integer nibble of column j (0..7) of a packed word.
__device__ __forceinline__ int nibble_of_col(uint32_t w, int j) {
  return (w >> (4 * ((j >> 1) + 4 * (j & 1)))) & 0xF;
}

// ---------------------------------------------------------------------------------------
// cp.async (16-byte, L2-only) with zero fill when `valid` is false.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

// mma.sync m16n8k16, fp16 inputs, fp32 accumulate: d = a * b + c.
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1, const float (&c)[4]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]),
        "f"(c[2]), "f"(c[3]));
}

// ---------------------------------------------------------------------------------------
// Host-side entry points of the individual kernels (defined in the .cu files).
// ---------------------------------------------------------------------------------------
int sm_count();  // SMs of the current device (cached)

int launch_dequantize(const uint32_t* qweight, const __half* scales, const uint32_t* qzeros,
                      __half* out, int K, int N, int group, cudaStream_t stream);

int launch_gemm_generic(const __half* x, const uint32_t* qweight, const __half* scales,
                        const uint32_t* qzeros, const __half* bias, __half* out, int M, int N,
                        int K, int group, cudaStream_t stream);

bool gemm_stream_supported(int M, int N, int K, int group);
int launch_gemm_stream(const __half* x, const uint32_t* qweight, const __half* scales,
                       const uint32_t* qzeros, const __half* bias, __half* out, int M, int N,
                       int K, int group, bool exact, cudaStream_t stream);

bool gemm_tc_supported(int M, int N, int K, int group);
size_t gemm_tc_workspace_bytes(int M, int N, int K, int group);
int launch_gemm_tc(const __half* x, const uint32_t* qweight, const __half* scales,
                   const uint32_t* qzeros, const __half* bias, __half* out, int M, int N, int K,
                   int group, void* workspace, size_t workspace_bytes, cudaStream_t stream);

int tc_device_status(int* out, int clear);
int launch_tc_grouped(int mode, const __half* a, int64_t a_rows, const uint32_t* w, int experts,
                      const __half* scales, const uint32_t* qzeros, const float* topk_weights,
                      const int32_t* sorted_ids, const int32_t* expert_ids,
                      const int32_t* num_post_pad, __half* out, int numel, int K, int N, int group,
                      int half_cols, int nblk, cudaStream_t stream);

bool gemm_stream_rp_supported(int M, int N, int K, int group);
int launch_gemm_stream_rp(const __half* x, const uint32_t* qweight_rp, const __half* scales,
                          const uint32_t* qzeros, const __half* bias, __half* out, int M, int N,
                          int K, int group, cudaStream_t stream);
int launch_repack_qweight(const uint32_t* qweight, uint32_t* out, int K, int N,
                          cudaStream_t stream);
bool gemm_ts_supported(int M, int N, int K, int group);
int launch_gemm_ts(const __half* x, const uint32_t* qweight, const __half* scales,
                   const uint32_t* qzeros, const __half* bias, __half* out, int M, int N, int K,
                   int group, bool exact, cudaStream_t stream);
int ts_device_status(int* out, int clear);

// gemm_wt.cu: dequantised weights in tensor memory as the A operand, activations as B
bool gemm_wt_supported(int M, int N, int K, int group);
int launch_gemm_wt(const __half* x, const uint32_t* qweight, const __half* scales,
                   const uint32_t* qzeros, const __half* bias, __half* out, int M, int N, int K,
                   int group, cudaStream_t stream);
int wt_device_status(int* out, int clear);

// gemm_q8.cu: K-major nibble copy of the weights, widened to bytes by tcgen05.cp on the way into
// tensor memory, int8 MMAs against fixed-point activations (M <= 32)
bool gemm_q8_supported(int M, int N, int K, int group);
size_t repack_kmajor_bytes(int K, int N);
int launch_repack_kmajor(const uint32_t* qweight, void* out, int K, int N, cudaStream_t stream);
size_t gemm_q8_workspace_bytes(int M, int N, int K, int group);
int launch_gemm_q8(const __half* x, const void* qweight_km, const __half* scales,
                   const uint32_t* qzeros, const __half* bias, __half* out, int M, int N, int K,
                   int group, void* workspace, size_t workspace_bytes, cudaStream_t stream);
void q8_set_spin_limit(uint32_t polls);
int launch_wait_selftest(uint32_t polls, cudaStream_t stream);
int q8_device_status(int* out, int clear);
// allreduce.cu: one-shot all-reduce of fp16 partial outputs over peer memory
int launch_allreduce(const void* const* regions, size_t data_offset, void* out, size_t bytes,
                     void* state, int rank, int world, int flags, cudaStream_t stream);
void ar_set_spin_limit(uint32_t polls);
int ar_device_status(int* out, int clear);

// wna16.cu: expert weights from the MoE WNA16 byte layout back to the AWQ checkpoint layout
int launch_wna16_to_awq(const uint8_t* w, const __half* scales, const uint8_t* zeros,
                        uint32_t* qweight, __half* scales_out, uint32_t* qzeros, int E, int N,
                        int K, int group, cudaStream_t stream);
bool moe_wt_supported(int H, int I, int group);
int launch_wt_grouped(int mode, const __half* a, int64_t a_rows, const uint32_t* w, int experts,
                      const __half* scales, const uint32_t* qzeros, const float* topk_weights,
                      const int32_t* sorted_ids, const int32_t* expert_ids,
                      const int32_t* num_post_pad, __half* out, int numel, int K, int N, int group,
                      int half_cols, int nblk, cudaStream_t stream);

int launch_topk_softmax(const void* gating, int gating_dtype, int T, int E, int topk,
                        int renormalize, float* topk_weights, int32_t* topk_ids,
                        int32_t* token_expert_indices, cudaStream_t stream);
int launch_moe_align(const int32_t* topk_ids, int numel, int E, int block,
                     const int32_t* expert_map, int32_t* sorted_ids, int64_t sorted_capacity,
                     int32_t* expert_ids, int32_t* num_post_pad, cudaStream_t stream);

struct MoeArgs {
  const __half* x;
  const uint32_t* w13_q;
  const __half* w13_s;
  const uint32_t* w13_z;
  const uint32_t* w2_q;
  const __half* w2_s;
  const uint32_t* w2_z;
  const float* topk_weights;
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post_pad;
  __half* out;
  int T, topk, E, H, I, group, block;
  int64_t sorted_capacity;
  int expert_parallel;
  int decode_layout;  // w13_q / w2_q are decode-layout copies (blocks of 8 or 16 rows only)
  int direct;         // no permutation: one 8-row block per pair, expert_ids = routed-id table
};
constexpr int kMoeDirectTicketBytes = 4096;  // AWQ_B200_MOE_DIRECT_MAX_PAIRS tokens x 64 slabs
bool moe_supported(int H, int I, int group, int block);
size_t moe_workspace_bytes(int T, int topk, int E, int H, int I);
int moe_block_size(int T, int topk, int E, int H, int I, int group);
bool moe_tc_supported(int H, int I, int group);
size_t moe_tc_workspace_bytes(int T, int topk, int E, int H, int I);
size_t moe_tc_layout_bytes(const MoeArgs& a);
size_t moe_layout_bytes(const MoeArgs& a);  // scratch a call with these arguments lays out
int launch_moe_experts_tc(const MoeArgs& a, void* workspace, size_t workspace_bytes,
                          cudaStream_t stream);
int launch_moe_sum(const __half* pair_out, __half* out, int T, int topk, int H,
                   cudaStream_t stream);
int launch_moe_experts(const MoeArgs& a, void* workspace, size_t workspace_bytes,
                       cudaStream_t stream);
int launch_moe_experts_static(const MoeArgs& a, cudaStream_t stream);
size_t moe_static_scratch_bytes();

}  // namespace awq
