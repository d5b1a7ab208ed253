// Grouped AWQ expert GEMMs on tcgen05 for prefill-sized token counts (many rows per expert).
//
// The (token, slot) pairs are already sorted by expert with every expert's run padded to 128 rows
// (moe_align_kernel, block = 128), so row block b of the permuted list belongs to exactly one
// expert, expert_ids[b].  One CTA computes one [128 rows x 256 columns] tile of one row block
// with the pipeline of gemm_tc.cu (TMA -> dequantisation warps -> tcgen05.mma into TMEM):
//
//   moe_gather_kernel   x_perm[pos] = x[token(pos)]           (padding rows = 0)
//   gemm_tc_kernel<.., 1>  gate_up: columns [128 j, 128 j + 128) of the gate half and of the up half
//                       form one 256-column tile; epilogue silu(gate) * up -> act[pos] fp16
//   gemm_tc_kernel<.., 2>  down: act rows x w2[e]; epilogue times routed weight ->
//                       pair_out[flat pair id] fp16
// followed by moe_sum_kernel (moe.cu).
//
// The packed weights of a tile arrive as two TMA boxes of [64 rows x 16 words] ("left" and
// "right" half of the tile's columns; for gate_up these are the gate and the up segment).
// Every wait is bounded (tc_ptx.cuh).
#include "common.cuh"

namespace awq {

namespace {

constexpr int kMBM = 128;

// x_perm[pos, :] = x[token(pos), :] for the rows of the used blocks; padding rows are zero.
// One warp per row, eight rows per CTA; a lane keeps four 16-byte loads in flight.
constexpr int kGatherRows = 8;
__global__ void __launch_bounds__(32 * kGatherRows)
moe_gather_kernel(const __half* __restrict__ x, const int32_t* __restrict__ sorted_ids,
                  const int32_t* __restrict__ num_post_pad, __half* __restrict__ x_perm,
                  int64_t capacity, int numel, int topk, int H) {
  const int lane = threadIdx.x & 31;
  const int64_t pos = (int64_t)blockIdx.x * kGatherRows + (threadIdx.x >> 5);
  // both loads in flight together
  const int post = num_post_pad[0];
  const int fid = pos < capacity ? sorted_ids[pos] : numel;
  if (pos >= post) return;
  uint4* dst = reinterpret_cast<uint4*>(x_perm + (size_t)pos * H);
  const int units = H / 8;
  if (fid < numel) {
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(fid / topk) * H);
    int i = lane;
    for (; i + 96 < units; i += 128) {
      const uint4 a = __ldg(src + i), b = __ldg(src + i + 32), c = __ldg(src + i + 64),
                  d = __ldg(src + i + 96);
      dst[i] = a;
      dst[i + 32] = b;
      dst[i + 64] = c;
      dst[i + 96] = d;
    }
    for (; i < units; i += 32) dst[i] = __ldg(src + i);
  } else {
    for (int i = lane; i < units; i += 32) dst[i] = make_uint4(0, 0, 0, 0);
  }
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

bool moe_tc_supported(int H, int I, int group) {
  // tiles: gate/up segments of 128 columns (I % 128), 256 hidden columns (H % 256);
  // stages of 64 rows inside one quantisation group; 16-byte TMA row pitches
  return H % 256 == 0 && I % 128 == 0 && (group == 128 || group == 64);
}

size_t moe_tc_workspace_bytes(int T, int topk, int E, int H, int I) {
  const int64_t cap = awq_b200_moe_sorted_capacity((int64_t)T * topk, E, kMBM);
  const int64_t rows = (cap + kMBM - 1) / kMBM * kMBM;
  return align_up((size_t)rows * H * 2, 256) + align_up((size_t)rows * I * 2, 256) +
         align_up((size_t)T * topk * H * 2, 256);
}

int launch_moe_sum(const __half* pair_out, __half* out, int T, int topk, int H, cudaStream_t stream);

size_t moe_tc_layout_bytes(const MoeArgs& a) {
  const int64_t rows = (a.sorted_capacity + kMBM - 1) / kMBM * kMBM;
  return align_up((size_t)rows * a.H * 2, 256) + align_up((size_t)rows * a.I * 2, 256) +
         align_up((size_t)a.T * a.topk * a.H * 2, 256);
}

int launch_moe_experts_tc(const MoeArgs& a, void* workspace, size_t workspace_bytes,
                          cudaStream_t stream) {
  if (a.block != kMBM || !moe_tc_supported(a.H, a.I, a.group)) return AWQ_B200_ERR_SHAPE;
  const size_t need = moe_tc_layout_bytes(a);
  if (workspace == nullptr || workspace_bytes < need) return AWQ_B200_ERR_WORKSPACE;
  const int numel = a.T * a.topk;
  const int64_t rows = (a.sorted_capacity + kMBM - 1) / kMBM * kMBM;
  const int nblk = (int)(rows / kMBM);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  __half* x_perm = reinterpret_cast<__half*>(ws);
  __half* act = reinterpret_cast<__half*>(ws + align_up((size_t)rows * a.H * 2, 256));
  __half* pair_out = reinterpret_cast<__half*>(ws + align_up((size_t)rows * a.H * 2, 256) +
                                               align_up((size_t)rows * a.I * 2, 256));

  if (a.expert_parallel) {
    if (cudaMemsetAsync(pair_out, 0, (size_t)numel * a.H * 2, stream) != cudaSuccess)
      return AWQ_B200_ERR_LAUNCH;
  }
  moe_gather_kernel<<<(unsigned)((rows + kGatherRows - 1) / kGatherRows), 32 * kGatherRows, 0,
                      stream>>>(a.x, a.sorted_ids, a.num_post_pad, x_perm, a.sorted_capacity, numel,
                                a.topk, a.H);
  if (cudaGetLastError() != cudaSuccess) return AWQ_B200_ERR_LAUNCH;
  // group 128: dequantised weights in TMEM as the A operand (gemm_wt.cu), padding tokens cost no
  // weight work there; group 64: weights dequantised into a shared-memory B tile (gemm_tc.cu)
  const bool wt = moe_wt_supported(a.H, a.I, a.group);
  auto grouped = wt ? launch_wt_grouped : launch_tc_grouped;
  if (int rc = grouped(1, x_perm, rows, a.w13_q, a.E, a.w13_s, a.w13_z, nullptr, a.sorted_ids,
                       a.expert_ids, a.num_post_pad, act, numel, a.H, 2 * a.I, a.group, a.I, nblk,
                       stream))
    return rc;
  if (int rc = grouped(2, act, rows, a.w2_q, a.E, a.w2_s, a.w2_z, a.topk_weights, a.sorted_ids,
                       a.expert_ids, a.num_post_pad, pair_out, numel, a.I, a.H, a.group, 0, nblk,
                       stream))
    return rc;
  return launch_moe_sum(pair_out, a.out, a.T, a.topk, a.H, stream);
}

}  // namespace awq
