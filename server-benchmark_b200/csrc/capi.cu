// extern "C" boundary of libawq_b200.so: argument validation and kernel selection.
// Declarations and their reference counterparts: include/awq_b200.h.
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_device() {
  static std::mutex mu;
  static int cc_major[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return AWQ_B200_ERR_DEVICE;
  if (dev < 0 || dev >= 64) return AWQ_B200_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(mu);
  if (cc_major[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
      return AWQ_B200_ERR_DEVICE;
    cc_major[dev] = v;
  }
  return cc_major[dev] == 10 ? AWQ_B200_OK : AWQ_B200_ERR_DEVICE;
}

int check_awq_shape(int N, int K, int group) {
  if (N <= 0 || K <= 0 || group <= 0) return AWQ_B200_ERR_SHAPE;
  if (N % awq::kPack != 0) return AWQ_B200_ERR_SHAPE;
  if (group % 8 != 0) return AWQ_B200_ERR_GROUP;
  if (K % group != 0) return AWQ_B200_ERR_SHAPE;
  return AWQ_B200_OK;
}

// Kernel choice for AWQ_B200_KERNEL_AUTO (measured crossovers on B200, Qwen2.5-72B shapes):
//   M <= 8                      mma.sync streaming kernel (one 8-token tile: 4 TB/s)
//   M <= 16                     tcgen05 with the unpacked weights in TMEM (gemm_ts)
//   M <= 128, or M <= 256 and   dequantised weights in TMEM as the A operand (gemm_wt)
//   fewer tiles than SMs
//   larger M                    tcgen05 with the weights dequantised into shared memory
int pick_gemm_kernel(int M, int N, int K, int group) {
  const int sms = awq::sm_count();
  const int slabs = (N + 255) / 256;
  if (M <= 8 && awq::gemm_stream_supported(M, N, K, group)) return AWQ_B200_KERNEL_STREAM;
  if (M <= 16) {
    if (awq::gemm_ts_supported(M, N, K, group)) return AWQ_B200_KERNEL_TS;
    if (awq::gemm_stream_supported(M, N, K, group)) return AWQ_B200_KERNEL_STREAM;
  }
  if (awq::gemm_wt_supported(M, N, K, group) &&
      (M <= 128 || (M <= 256 && slabs * ((M + 127) / 128) < sms)))
    return AWQ_B200_KERNEL_WT;
  if (M <= 32 && awq::gemm_stream_supported(M, N, K, group)) return AWQ_B200_KERNEL_STREAM;
  if (awq::gemm_tc_supported(M, N, K, group)) return AWQ_B200_KERNEL_TCGEN05;
  return AWQ_B200_KERNEL_GENERIC;
}

}  // namespace

extern "C" {

const char* awq_b200_strerror(int code) {
  switch (code) {
    case AWQ_B200_OK: return "ok";
    case AWQ_B200_ERR_NULL: return "a required pointer is NULL";
    case AWQ_B200_ERR_SHAPE: return "bad shape: size not positive or divisibility rule violated";
    case AWQ_B200_ERR_ALIGN: return "pointer not 16-byte aligned";
    case AWQ_B200_ERR_GROUP: return "unsupported quantisation group size";
    case AWQ_B200_ERR_WORKSPACE: return "workspace missing or too small";
    case AWQ_B200_ERR_LAUNCH: return "CUDA launch failed";
    case AWQ_B200_ERR_DEVICE: return "current device is not an sm_100 GPU";
    case AWQ_B200_ERR_DRIVER: return "CUDA driver entry point unavailable";
    case AWQ_B200_ERR_LIMIT: return "size exceeds a built-in capacity";
    case AWQ_B200_ERR_SYMBOL: return "the built-in scratch array could not be bound on this GPU";
    default: return "unknown error code";
  }
}

const char* awq_b200_version(void) { return "0.1"; }

int awq_b200_dequantize(const void* qweight, const void* scales, const void* qzeros, void* out,
                        int K, int N, int group, void* stream) {
  if (!qweight || !scales || !qzeros || !out) return AWQ_B200_ERR_NULL;
  if (int rc = check_awq_shape(N, K, group)) return rc;
  if (!aligned16(scales) || !aligned16(out) || !aligned16(qweight) || !aligned16(qzeros))
    return AWQ_B200_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  return awq::launch_dequantize(static_cast<const uint32_t*>(qweight),
                                static_cast<const __half*>(scales),
                                static_cast<const uint32_t*>(qzeros), static_cast<__half*>(out), K,
                                N, group, static_cast<cudaStream_t>(stream));
}

int awq_b200_repack_qweight(const void* qweight, void* out, int K, int N, void* stream) {
  if (!qweight || !out) return AWQ_B200_ERR_NULL;
  if (K <= 0 || N <= 0 || N % awq::kPack != 0 || K % 4 != 0) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(qweight) || !aligned16(out)) return AWQ_B200_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  return awq::launch_repack_qweight(static_cast<const uint32_t*>(qweight),
                                    static_cast<uint32_t*>(out), K, N,
                                    static_cast<cudaStream_t>(stream));
}

size_t awq_b200_repack_kmajor_bytes(int K, int N) {
  if (K <= 0 || N <= 0 || N % awq::kPack != 0 || K % 128 != 0) return 0;
  return awq::repack_kmajor_bytes(K, N);
}

int awq_b200_repack_kmajor(const void* qweight, void* out, int K, int N, void* stream) {
  if (!qweight || !out) return AWQ_B200_ERR_NULL;
  if (K <= 0 || N <= 0 || N % awq::kPack != 0 || K % 128 != 0) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(qweight) || (reinterpret_cast<uintptr_t>(out) & 31u) != 0)
    return AWQ_B200_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  return awq::launch_repack_kmajor(static_cast<const uint32_t*>(qweight), out, K, N,
                                   static_cast<cudaStream_t>(stream));
}

int awq_b200_wna16_to_awq(const void* w, const void* scales, const void* zeros, void* qweight,
                          void* scales_out, void* qzeros, int E, int N, int K, int group,
                          void* stream) {
  if (!w || !scales || !zeros || !qweight || !scales_out || !qzeros) return AWQ_B200_ERR_NULL;
  if (E <= 0 || N <= 0 || K <= 0 || group <= 0) return AWQ_B200_ERR_SHAPE;
  if (N % awq::kPack != 0 || K % 2 != 0 || K % group != 0) return AWQ_B200_ERR_SHAPE;
  if (int rc = check_device()) return rc;
  return awq::launch_wna16_to_awq(static_cast<const uint8_t*>(w),
                                  static_cast<const __half*>(scales),
                                  static_cast<const uint8_t*>(zeros),
                                  static_cast<uint32_t*>(qweight),
                                  static_cast<__half*>(scales_out),
                                  static_cast<uint32_t*>(qzeros), E, N, K, group,
                                  static_cast<cudaStream_t>(stream));
}

size_t awq_b200_gemm_workspace_bytes(int M, int N, int K, int group, int kernel) {
  if (M <= 0 || check_awq_shape(N, K, group) != AWQ_B200_OK) return 0;
  if (kernel == AWQ_B200_KERNEL_Q8) return awq::gemm_q8_workspace_bytes(M, N, K, group);
  if (kernel == AWQ_B200_KERNEL_AUTO) kernel = pick_gemm_kernel(M, N, K, group);
  if (kernel == AWQ_B200_KERNEL_TCGEN05) return awq::gemm_tc_workspace_bytes(M, N, K, group);
  return 0;
}

int awq_b200_gemm(const void* x, const void* qweight, const void* scales, const void* qzeros,
                  const void* bias, void* out, int M, int N, int K, int group, int kernel,
                  void* workspace, size_t workspace_bytes, void* stream) {
  if (M == 0) return AWQ_B200_OK;
  if (M < 0) return AWQ_B200_ERR_SHAPE;
  if (!x || !qweight || !scales || !qzeros || !out) return AWQ_B200_ERR_NULL;
  if (int rc = check_awq_shape(N, K, group)) return rc;
  if (K % 8 != 0) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(qweight) || !aligned16(scales) || !aligned16(qzeros) ||
      !aligned16(out) || (bias && !aligned16(bias)))
    return AWQ_B200_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  if (kernel == AWQ_B200_KERNEL_AUTO) kernel = pick_gemm_kernel(M, N, K, group);

  const __half* xh = static_cast<const __half*>(x);
  const uint32_t* qw = static_cast<const uint32_t*>(qweight);
  const __half* sc = static_cast<const __half*>(scales);
  const uint32_t* qz = static_cast<const uint32_t*>(qzeros);
  const __half* bh = static_cast<const __half*>(bias);
  __half* oh = static_cast<__half*>(out);
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  switch (kernel) {
    case AWQ_B200_KERNEL_GENERIC:
      return awq::launch_gemm_generic(xh, qw, sc, qz, bh, oh, M, N, K, group, st);
    case AWQ_B200_KERNEL_STREAM:
    case AWQ_B200_KERNEL_STREAM_EXACT:
      if (!awq::gemm_stream_supported(M, N, K, group)) return AWQ_B200_ERR_SHAPE;
      return awq::launch_gemm_stream(xh, qw, sc, qz, bh, oh, M, N, K, group,
                                     kernel == AWQ_B200_KERNEL_STREAM_EXACT, st);
    case AWQ_B200_KERNEL_TS:
    case AWQ_B200_KERNEL_TS_EXACT:
      if (!awq::gemm_ts_supported(M, N, K, group)) return AWQ_B200_ERR_SHAPE;
      return awq::launch_gemm_ts(xh, qw, sc, qz, bh, oh, M, N, K, group,
                                 kernel == AWQ_B200_KERNEL_TS_EXACT, st);
    case AWQ_B200_KERNEL_STREAM_RP:
      if (!awq::gemm_stream_rp_supported(M, N, K, group)) return AWQ_B200_ERR_SHAPE;
      return awq::launch_gemm_stream_rp(xh, qw, sc, qz, bh, oh, M, N, K, group, st);
    case AWQ_B200_KERNEL_WT:
      if (!awq::gemm_wt_supported(M, N, K, group)) return AWQ_B200_ERR_SHAPE;
      return awq::launch_gemm_wt(xh, qw, sc, qz, bh, oh, M, N, K, group, st);
    case AWQ_B200_KERNEL_Q8: {
      if (!awq::gemm_q8_supported(M, N, K, group)) return AWQ_B200_ERR_SHAPE;
      if ((reinterpret_cast<uintptr_t>(qweight) & 31u) != 0) return AWQ_B200_ERR_ALIGN;
      const size_t need = awq::gemm_q8_workspace_bytes(M, N, K, group);
      if (!workspace || workspace_bytes < need) return AWQ_B200_ERR_WORKSPACE;
      if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return AWQ_B200_ERR_ALIGN;
      return awq::launch_gemm_q8(xh, qweight, sc, qz, bh, oh, M, N, K, group, workspace,
                                 workspace_bytes, st);
    }
    case AWQ_B200_KERNEL_TCGEN05: {
      if (!awq::gemm_tc_supported(M, N, K, group)) return AWQ_B200_ERR_SHAPE;
      const size_t need = awq::gemm_tc_workspace_bytes(M, N, K, group);
      if (need > 0) {
        if (!workspace || workspace_bytes < need) return AWQ_B200_ERR_WORKSPACE;
        if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return AWQ_B200_ERR_ALIGN;
      }
      return awq::launch_gemm_tc(xh, qw, sc, qz, bh, oh, M, N, K, group, workspace,
                                 workspace_bytes, st);
    }
    default:
      return AWQ_B200_ERR_SHAPE;
  }
}

static int device_status(int* status, int clear) {
  if (!status) return AWQ_B200_ERR_NULL;
  if (int rc = check_device()) return rc;
  int v[5] = {0, 0, 0, 0, 0};
  if (int rc = awq::tc_device_status(&v[0], clear)) return rc;
  if (int rc = awq::ts_device_status(&v[1], clear)) return rc;
  if (int rc = awq::wt_device_status(&v[2], clear)) return rc;
  if (int rc = awq::q8_device_status(&v[3], clear)) return rc;
  if (int rc = awq::ar_device_status(&v[4], clear)) return rc;
  *status = 0;
  for (int i = 0; i < 5; ++i)
    if (v[i] != 0 && *status == 0) *status = v[i];
  return AWQ_B200_OK;
}

int awq_b200_device_status(int* status) { return device_status(status, 0); }

int awq_b200_device_status_clear(int* status) { return device_status(status, 1); }

void awq_b200_set_wait_limit(unsigned int polls) {
  awq::q8_set_spin_limit(polls);
  awq::ar_set_spin_limit(polls);
}

int awq_b200_peer_region_create(size_t bytes, void** region, void* handle) {
  if (!region || !handle) return AWQ_B200_ERR_NULL;
  if (bytes < AWQ_B200_AR_FLAG_BYTES) return AWQ_B200_ERR_SHAPE;
  if (int rc = check_device()) return rc;
  static_assert(sizeof(cudaIpcMemHandle_t) == AWQ_B200_IPC_HANDLE_BYTES, "handle size");
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return AWQ_B200_ERR_WORKSPACE;
  }
  cudaIpcMemHandle_t h;
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
      cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    (void)cudaGetLastError();
    cudaFree(p);
    return AWQ_B200_ERR_LAUNCH;
  }
  memcpy(handle, &h, sizeof(h));
  *region = p;
  return AWQ_B200_OK;
}

int awq_b200_peer_region_open(const void* handle, void** region) {
  if (!handle || !region) return AWQ_B200_ERR_NULL;
  if (int rc = check_device()) return rc;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  // mapped into the CURRENT device's context, peer access to the owning device enabled with it
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    (void)cudaGetLastError();
    return AWQ_B200_ERR_DEVICE;
  }
  *region = p;
  return AWQ_B200_OK;
}

int awq_b200_peer_region_close(void* region) {
  if (!region) return AWQ_B200_ERR_NULL;
  return cudaIpcCloseMemHandle(region) == cudaSuccess ? AWQ_B200_OK : AWQ_B200_ERR_LAUNCH;
}

int awq_b200_peer_region_destroy(void* region) {
  if (!region) return AWQ_B200_ERR_NULL;
  return cudaFree(region) == cudaSuccess ? AWQ_B200_OK : AWQ_B200_ERR_LAUNCH;
}

int awq_b200_allreduce(const void* const* regions, int rank, int world, size_t data_offset,
                       void* out, size_t bytes, void* state, int flags, void* stream) {
  if (!regions || !out || !state) return AWQ_B200_ERR_NULL;
  if (world < 1 || world > AWQ_B200_AR_MAX_RANKS || rank < 0 || rank >= world)
    return AWQ_B200_ERR_SHAPE;
  if (bytes == 0) return AWQ_B200_OK;
  if (bytes % 16 != 0 || data_offset % 16 != 0 || data_offset < AWQ_B200_AR_FLAG_BYTES)
    return AWQ_B200_ERR_SHAPE;
  for (int r = 0; r < world; ++r) {
    if (!regions[r]) return AWQ_B200_ERR_NULL;
    if (!aligned16(regions[r])) return AWQ_B200_ERR_ALIGN;
  }
  if (!aligned16(out)) return AWQ_B200_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  // every region must be device memory this process has mapped (a stale or foreign pointer is
  // refused here instead of faulting in the kernel)
  for (int r = 0; r < world; ++r) {
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, regions[r]) != cudaSuccess ||
        attr.type != cudaMemoryTypeDevice) {
      (void)cudaGetLastError();
      return AWQ_B200_ERR_DEVICE;
    }
  }
  return awq::launch_allreduce(regions, data_offset, out, bytes, state, rank, world, flags,
                               static_cast<cudaStream_t>(stream));
}

int awq_b200_selftest_wait(unsigned int polls, void* stream) {
  if (int rc = check_device()) return rc;
  return awq::launch_wait_selftest(polls, static_cast<cudaStream_t>(stream));
}

int awq_b200_topk_softmax(const void* gating, int gating_dtype, int T, int E, int topk,
                          int renormalize, float* topk_weights, int32_t* topk_ids,
                          int32_t* token_expert_indices, void* stream) {
  if (T == 0) return AWQ_B200_OK;
  if (!gating || !topk_weights || !topk_ids) return AWQ_B200_ERR_NULL;
  if (T < 0 || E <= 0 || topk <= 0 || topk > E) return AWQ_B200_ERR_SHAPE;
  if (gating_dtype != 0 && gating_dtype != 1) return AWQ_B200_ERR_SHAPE;
  if (E > 1024 || topk > 32) return AWQ_B200_ERR_LIMIT;
  if (int rc = check_device()) return rc;
  return awq::launch_topk_softmax(gating, gating_dtype, T, E, topk, renormalize, topk_weights,
                                  topk_ids, token_expert_indices,
                                  static_cast<cudaStream_t>(stream));
}

int64_t awq_b200_moe_sorted_capacity(int64_t numel, int E, int block) {
  if (numel < 0 || E <= 0 || block <= 0) return 0;
  int64_t cap = numel + (int64_t)E * (block - 1);
  if (numel < E) cap = numel * block < cap ? numel * block : cap;
  return cap;
}

int awq_b200_moe_align_block_size(const int32_t* topk_ids, int T, int topk, int E, int block,
                                  const int32_t* expert_map, int32_t* sorted_ids,
                                  int64_t sorted_capacity, int32_t* expert_ids,
                                  int32_t* num_post_pad, void* stream) {
  if (!sorted_ids || !expert_ids || !num_post_pad) return AWQ_B200_ERR_NULL;
  if (T < 0 || topk <= 0 || E <= 0 || block <= 0) return AWQ_B200_ERR_SHAPE;
  if (T > 0 && !topk_ids) return AWQ_B200_ERR_NULL;
  const int64_t numel = (int64_t)T * topk;
  if (E > 1024 || numel > (1 << 24)) return AWQ_B200_ERR_LIMIT;
  if (sorted_capacity < awq_b200_moe_sorted_capacity(numel, E, block))
    return AWQ_B200_ERR_WORKSPACE;
  if (int rc = check_device()) return rc;
  return awq::launch_moe_align(topk_ids, (int)numel, E, block, expert_map, sorted_ids,
                               sorted_capacity, expert_ids, num_post_pad,
                               static_cast<cudaStream_t>(stream));
}

int awq_b200_moe_block_size(int T, int topk, int E, int H, int I, int group) {
  return awq::moe_block_size(T, topk, E, H, I, group);
}

size_t awq_b200_moe_workspace_bytes(int T, int topk, int E, int H, int I) {
  return awq::moe_workspace_bytes(T, topk, E, H, I);
}

// Validation shared by the two expert entry points.  Everything here is arithmetic on the
// arguments: it runs (and refuses) before any CUDA call.  `limit` > 0: the scratch is a built-in
// array of that size and a larger need is AWQ_B200_ERR_LIMIT; else the caller's buffer is checked.
static int moe_validate(const void* x, const void* w13_q, const void* w13_s, const void* w13_z,
                        const void* w2_q, const void* w2_s, const void* w2_z,
                        const float* topk_weights, const int32_t* sorted_ids,
                        const int32_t* expert_ids, const int32_t* num_post_pad, void* out, int T,
                        int topk, int E, int H, int I, int group, int block, int expert_parallel,
                        int64_t sorted_capacity, const void* workspace, size_t workspace_bytes,
                        size_t limit, awq::MoeArgs* args) {
  const bool direct = (expert_parallel & 4) != 0;
  if (!x || !w13_q || !w13_s || !w13_z || !w2_q || !w2_s || !w2_z || !topk_weights ||
      !expert_ids || !out)
    return AWQ_B200_ERR_NULL;
  if (!direct && (!sorted_ids || !num_post_pad)) return AWQ_B200_ERR_NULL;
  if (T < 0 || topk <= 0 || E <= 0 || H <= 0 || I <= 0 || block <= 0) return AWQ_B200_ERR_SHAPE;
  if (direct) {
    // no permutation: one 8-row block per pair, expert_ids is the routed-id table itself
    if (block != 8 || (expert_parallel & 1) || (int64_t)T * topk > AWQ_B200_MOE_DIRECT_MAX_PAIRS)
      return AWQ_B200_ERR_SHAPE;
    if (sorted_capacity != (int64_t)T * topk * 8) return AWQ_B200_ERR_WORKSPACE;
    sorted_ids = nullptr;
    num_post_pad = nullptr;
  }
  if (group != 128 && group != 64 && group != 32) return AWQ_B200_ERR_GROUP;
  if (!awq::moe_supported(H, I, group, block)) return AWQ_B200_ERR_SHAPE;
  if ((int64_t)T * topk > (1 << 24)) return AWQ_B200_ERR_LIMIT;
  if ((sorted_capacity + block - 1) / block > 65535) return AWQ_B200_ERR_LIMIT;
  if (!direct && sorted_capacity < awq_b200_moe_sorted_capacity((int64_t)T * topk, E, block))
    return AWQ_B200_ERR_WORKSPACE;
  *args = awq::MoeArgs{static_cast<const __half*>(x),
                       static_cast<const uint32_t*>(w13_q),
                       static_cast<const __half*>(w13_s),
                       static_cast<const uint32_t*>(w13_z),
                       static_cast<const uint32_t*>(w2_q),
                       static_cast<const __half*>(w2_s),
                       static_cast<const uint32_t*>(w2_z),
                       topk_weights,
                       sorted_ids,
                       expert_ids,
                       num_post_pad,
                       static_cast<__half*>(out),
                       T, topk, E, H, I, group, block,
                       sorted_capacity,
                       expert_parallel & 1,
                       (expert_parallel >> 1) & 1,
                       direct ? 1 : 0};
  // the scratch need follows sorted_capacity, which the caller chose (it is at least the
  // minimum for the stacked expert count, larger if the permutation was built for more experts)
  const size_t need = awq::moe_layout_bytes(*args);
  if (limit > 0) {
    if (need > limit) return AWQ_B200_ERR_LIMIT;
  } else {
    if (!workspace || workspace_bytes < need) return AWQ_B200_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return AWQ_B200_ERR_ALIGN;
  }
  if (!aligned16(x) || !aligned16(w13_q) || !aligned16(w13_s) || !aligned16(w13_z) ||
      !aligned16(w2_q) || !aligned16(w2_s) || !aligned16(w2_z) || !aligned16(out))
    return AWQ_B200_ERR_ALIGN;
  return AWQ_B200_OK;
}

int awq_b200_moe_experts(const void* x, const void* w13_q, const void* w13_s, const void* w13_z,
                         const void* w2_q, const void* w2_s, const void* w2_z,
                         const float* topk_weights, const int32_t* sorted_ids,
                         const int32_t* expert_ids, const int32_t* num_post_pad, void* out,
                         int T, int topk, int E, int H, int I, int group, int block,
                         int expert_parallel, int64_t sorted_capacity, void* workspace,
                         size_t workspace_bytes, void* stream) {
  if (T == 0) return AWQ_B200_OK;
  awq::MoeArgs a;
  if (int rc = moe_validate(x, w13_q, w13_s, w13_z, w2_q, w2_s, w2_z, topk_weights, sorted_ids,
                            expert_ids, num_post_pad, out, T, topk, E, H, I, group, block,
                            expert_parallel, sorted_capacity, workspace, workspace_bytes, 0, &a))
    return rc;
  if (int rc = check_device()) return rc;
  return awq::launch_moe_experts(a, workspace, workspace_bytes,
                                 static_cast<cudaStream_t>(stream));
}

size_t awq_b200_moe_static_scratch_bytes(void) { return awq::moe_static_scratch_bytes(); }

int awq_b200_moe_experts_static(const void* x, const void* w13_q, const void* w13_s,
                                const void* w13_z, const void* w2_q, const void* w2_s,
                                const void* w2_z, const float* topk_weights,
                                const int32_t* sorted_ids, const int32_t* expert_ids,
                                const int32_t* num_post_pad, void* out, int T, int topk, int E,
                                int H, int I, int group, int block, int expert_parallel,
                                int64_t sorted_capacity, void* stream) {
  if (T == 0) return AWQ_B200_OK;
  awq::MoeArgs a;
  // the built-in scratch has a fixed size: larger problems are refused, not truncated
  if (int rc = moe_validate(x, w13_q, w13_s, w13_z, w2_q, w2_s, w2_z, topk_weights, sorted_ids,
                            expert_ids, num_post_pad, out, T, topk, E, H, I, group, block,
                            expert_parallel, sorted_capacity, nullptr, 0,
                            awq::moe_static_scratch_bytes(), &a))
    return rc;
  if (int rc = check_device()) return rc;
  return awq::launch_moe_experts_static(a, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
