// AWQ fused-MoE layer: router, token -> expert permutation, grouped expert GEMMs.
//
//   topk_softmax_kernel   one warp per token: softmax over E logits, k rounds of warp arg-max
//                         (ties -> lower expert id), optional renormalisation.
//   moe_align_kernel      stable counting sort of the T*k (token, slot) pairs by expert with
//                         every expert's run padded to the GEMM row block; one CTA per 256 pairs,
//                         each CTA rebuilds the (cheap) histograms itself so a single launch
//                         suffices; ranks come from warp match masks, in ascending flat index,
//                         hence a deterministic order.
//   moe_gemm1_kernel      per (row block, 128 gate + 128 up columns): x rows gathered through the
//                         permutation, expert weights streamed (stream_core.cuh), epilogue
//                         silu(gate) * up -> fp16 activation in permuted row order.
//   moe_gemm2_kernel      per (row block, 256 hidden columns): activation rows x down weights,
//                         epilogue times routed weight -> fp16 row of the (token, slot) pair.
//   moe_sum_kernel        out[t] = sum over the k slots of token t, fp32 accumulation.
// The GEMMs split K across a thread-block cluster and reduce through distributed shared
// memory, exactly like the dense small-M kernel.
#include <cooperative_groups.h>

#include <mutex>

#include "stream_core.cuh"

namespace cg = cooperative_groups;

// Scratch for awq_b200_moe_experts_static: 16 MiB of device memory per GPU, reserved when the
// library is loaded on that GPU and kept until the process ends.
constexpr size_t kMoeStaticScratchBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_moe_static_scratch[kMoeStaticScratchBytes];

namespace awq {

namespace {

using namespace stream;

// ------------------------------------------------------------------------------- router

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

constexpr int kTopkWarps = 4;

// NV = entries per lane (E <= 32 NV): the selection loops run over NV, not over the 32 that the
// largest supported expert count needs.
template <typename T, int NV>
__global__ void __launch_bounds__(kTopkWarps * 32)
topk_softmax_kernel(const T* __restrict__ gating, int tokens, int E, int topk, int renorm,
                    float* __restrict__ out_w, int32_t* __restrict__ out_ids,
                    int32_t* __restrict__ out_tok) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.x * kTopkWarps + warp;
  pdl_launch_dependents();
  pdl_wait();
  if (token >= tokens) return;
  const T* row = gating + (size_t)token * E;
  const float kNegInf = -__int_as_float(0x7f800000);
  float v[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? to_f32<T>(row[e]) : kNegInf;
  }
  float mx = kNegInf;
#pragma unroll
  for (int i = 0; i < NV; ++i) mx = fmaxf(mx, v[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) sum += (lane + 32 * i < E) ? __expf(v[i] - mx) : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;

  float my_w = 0.f;
  int my_id = 0;
  uint32_t taken = 0;  // bit i: entry lane + 32 i already selected
  for (int j = 0; j < topk; ++j) {
    float bv = kNegInf;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int e = lane + 32 * i;
      // ascending e: a strict comparison keeps the lower id on ties
      if (e < E && !((taken >> i) & 1u) && (bi == 0x7fffffff || v[i] > bv)) {
        bv = v[i];
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == j) {
      my_w = __expf(bv - mx) * inv;
      my_id = bi;
    }
    if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
  }
  if (renorm) {
    float s = lane < topk ? my_w : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    my_w = my_w / s;
  }
  if (lane < topk) {
    out_w[(size_t)token * topk + lane] = my_w;
    out_ids[(size_t)token * topk + lane] = my_id;
    if (out_tok != nullptr) out_tok[(size_t)token * topk + lane] = lane * tokens + token;
  }
}

// ------------------------------------------------------------------------------- permutation

constexpr int kAlignThreads = 256;                 // 8 warps
constexpr int kAlignChunk = kAlignThreads;         // ids ranked by one CTA
constexpr int kAlignMaxCtas = 296;                 // bounds the redundant histogram passes

// One CTA ranks a contiguous range of flat ids, 256 at a time.  Every CTA first builds, in shared memory,
// the histogram of ALL ids (-> padded expert offsets) and the histogram of the ids that precede
// its range (-> where its own entries start inside each expert's run); that redundant pass over
// the id list costs a few microseconds and saves a second launch or a grid-wide barrier.  Inside
// the chunk the order is kept by ranking with warp match masks plus per-warp counts, so the
// result is the stable counting sort the oracle defines, independent of scheduling.
__global__ void __launch_bounds__(kAlignThreads)
moe_align_kernel(const int32_t* __restrict__ ids, int numel, int E, int block,
                 const int32_t* __restrict__ expert_map, int32_t* __restrict__ sorted_ids,
                 int64_t capacity, int32_t* __restrict__ expert_ids,
                 int32_t* __restrict__ num_post_pad) {
  extern __shared__ int sm[];
  pdl_launch_dependents();
  int* total = sm;                 // [E]   histogram of all ids
  int* prior = sm + E;             // [E]   histogram of ids before this chunk
  int* offs = sm + 2 * E;          // [E+1] padded exclusive prefix
  int* wcnt = sm + 3 * E + 1;      // [8][E] per-warp histogram of this chunk
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // contiguous range of chunks owned by this CTA
  const int nchunks = (numel + kAlignChunk - 1) / kAlignChunk;
  const int per_cta = (nchunks + gridDim.x - 1) / gridDim.x;
  const int first = blockIdx.x * per_cta * kAlignChunk;
  const int last = min(numel, first + per_cta * kAlignChunk);
  for (int i = tid; i < 3 * E + 1 + 8 * E; i += kAlignThreads) sm[i] = 0;
  __syncthreads();
  pdl_wait();
  auto valid = [&](int id) {
    return id >= 0 && id < E && (expert_map == nullptr || expert_map[id] >= 0);
  };
#pragma unroll 4
  for (int i = tid; i < numel; i += kAlignThreads) {
    const int id = ids[i];
    if (valid(id)) {
      atomicAdd(&total[id], 1);
      if (i < first) atomicAdd(&prior[id], 1);
    }
  }
  __syncthreads();
  // exclusive prefix of the padded counts: thread t owns experts [t * per, (t + 1) * per),
  // warp shuffles scan the per-thread sums, the first warp scans the eight warp sums
  {
    const int per = (E + kAlignThreads - 1) / kAlignThreads;
    const int e0 = tid * per, e1 = min(E, e0 + per);
    int mine_sum = 0;
    for (int e = e0; e < e1; ++e) mine_sum += ((total[e] + block - 1) / block) * block;
    int incl = mine_sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += v;
    }
    __shared__ int s_warp_sum[kAlignThreads / 32];
    if (lane == 31) s_warp_sum[warp] = incl;
    __syncthreads();
    int base = 0;
    for (int w = 0; w < warp; ++w) base += s_warp_sum[w];
    int run = base + incl - mine_sum;
    for (int e = e0; e < e1; ++e) {
      offs[e] = run;
      run += ((total[e] + block - 1) / block) * block;
    }
    if (tid == kAlignThreads - 1) offs[E] = base + incl;
  }
  __syncthreads();
  const int post = offs[E];
  for (int chunk0 = first; chunk0 < last; chunk0 += kAlignChunk) {
    // this thread's id and its rank among equal ids of its warp
    const int idx = chunk0 + tid;
    const int my = idx < last ? ids[idx] : -1;
    const bool mine = idx < last && valid(my);
    const unsigned peers = __match_any_sync(0xffffffffu, mine ? my : -1 - lane);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (mine && rank_in_warp == 0) wcnt[warp * E + my] = __popc(peers);
    __syncthreads();
    if (mine) {
      int before = prior[my];
      for (int w = 0; w < warp; ++w) before += wcnt[w * E + my];
      sorted_ids[offs[my] + before + rank_in_warp] = idx;
    }
    __syncthreads();
    if (chunk0 + kAlignChunk < last) {  // fold this chunk into the running counts
      for (int e = tid; e < E; e += kAlignThreads) {
        int c = 0;
        for (int w = 0; w < kAlignThreads / 32; ++w) {
          c += wcnt[w * E + e];
          wcnt[w * E + e] = 0;
        }
        prior[e] += c;
      }
      __syncthreads();
    }
  }
  // padding entries, block -> expert table and the tail are written by the first CTA
  if (blockIdx.x == 0) {
    for (int e = warp; e < E; e += kAlignThreads / 32) {
      const int cnt = total[e];
      if (cnt == 0) continue;
      const int base = offs[e], padded = offs[e + 1] - base;
      for (int j = cnt + lane; j < padded; j += 32) sorted_ids[base + j] = numel;
      const int local = expert_map == nullptr ? e : expert_map[e];
      for (int bk = lane; bk < padded / block; bk += 32) expert_ids[base / block + bk] = local;
    }
    if (tid == 0) num_post_pad[0] = post;
    for (int64_t j = post + tid; j < capacity; j += kAlignThreads) sorted_ids[j] = numel;
    const int64_t nblk = (capacity + block - 1) / block;
    for (int64_t bk = post / block + tid; bk < nblk; bk += kAlignThreads) expert_ids[bk] = -1;
  }
}

// ------------------------------------------------------------------------------- grouped GEMMs

constexpr bool kMoeExact = false;  // conversion used by the expert GEMMs (see stream_core.cuh)

// Direct mode (no permutation; sorted_ids == nullptr): row block `blk` holds the single pair
// `blk` in its row 0, and expert_ids is the flat [T * topk] table of routed expert ids itself.
// For a handful of pairs (decode of one or two tokens) this drops the permutation kernel from
// the chain; a pair that shares its expert with another one then reads that expert's weights
// again, which costs less than the launch it saves.
__device__ __forceinline__ int row_pair(const int32_t* sorted_ids, int pos0, int row, int blk,
                                        int numel) {
  return sorted_ids ? sorted_ids[pos0 + row] : (row == 0 ? blk : numel);
}

struct Gemm1Params {
  const __half* x;           // [T, H]
  const uint32_t* w13_q;     // [E, H, 2I/8]
  const __half* w13_s;       // [E, H/G, 2I]
  const uint32_t* w13_z;     // [E, H/G, 2I/8]
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post_pad;
  __half* act;               // [capacity, I] in permuted row order
  int numel, topk, H, I, group;
  uint32_t* tickets;         // direct mode: counters the down GEMM uses, cleared here; else nullptr
  int n_tickets;
};

// MT = token tiles of 8 per row block: 1 (8-row blocks, decode-size batches: almost every expert
// that is hit sees one or two tokens) or 2 (16-row blocks).
// GROUP: the quantisation group size when it is 128 (inner loops fully unrolled), else 0 (taken
// from the parameters at run time).  RP: the packed expert weights are the decode-layout copy
// (launch_repack_qweight over the stacked rows; see stream_core.cuh).
template <int MT, int GROUP, bool RP>
__global__ void __launch_bounds__(kThreads, MT == 1 ? 5 : 4) moe_gemm1_kernel(const Gemm1Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int S = (int)cluster.num_blocks();
  const int blk = blockIdx.z;
  const int pos0 = blk * (8 * MT);
  pdl_launch_dependents();
  pdl_wait();  // the routing tables come from the kernels before this one
  if (p.tickets != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
    // every kernel that used the counters before has completed (pdl_wait); the down GEMM of this
    // call starts counting only after this kernel has
    for (int i = threadIdx.x; i < p.n_tickets; i += kThreads) p.tickets[i] = 0u;
  }
  // uniform over the cluster: nobody reaches a cluster barrier if the block is unused
  // both loads in flight together (expert_ids covers every block of the grid)
  const int post = p.num_post_pad ? p.num_post_pad[0] : 0x7fffffff;
  const int e = p.expert_ids[blk];
  if (pos0 >= post || e < 0) return;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2;
  const int words = 2 * p.I / kPack;  // weight row pitch
  const int iw = p.I / kPack;         // words of the gate half
  const int seg0 = blockIdx.y * 16;   // first word of this slab inside the gate (and up) half
  const int groups = p.H / p.group;
  const uint32_t* wq = p.w13_q + (size_t)e * p.H * words;
  const uint32_t* wz = p.w13_z + (size_t)e * groups * words;
  const __half* ws = p.w13_s + (size_t)e * groups * (2 * p.I);

  TileSrc<MT> src;
  {
    if (RP) {
      // this thread copies the 16-byte unit of word column tid % 32: 0-15 gate, 16-31 up
      const int c = tid & 31;
      const int in_seg = seg0 + (c & 15);
      src.wvalid = in_seg < iw;
      const int wc = (c < 16 ? 0 : iw) + (src.wvalid ? in_seg : 0);
      src.wsrc = wq + (size_t)wc * 4;
      src.wrow_words = (size_t)words * 4;
    } else {
      const int c = tid & 7;
      const int in_seg = seg0 + (c & 3) * 4;       // word inside the half
      src.wvalid = in_seg < iw;
      const int wc = (c < 4 ? 0 : iw) + (src.wvalid ? in_seg : 0);
      src.wsrc = wq + wc;
      src.wrow_words = (size_t)words;
    }
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      const int row = (tid >> 4) + 8 * j;
      const int fid = row_pair(p.sorted_ids, pos0, row, blk, p.numel);
      src.xvalid[j] = fid < p.numel;
      const int token = src.xvalid[j] ? fid / p.topk : 0;
      src.xsrc[j] = p.x + (size_t)token * p.H + (tid & 15) * 8;
    }
    int in_seg_c = seg0 + 8 * (warp & 1) + g;
    if (in_seg_c >= iw) in_seg_c = iw - 1;
    const int wcol = (warp < 2 ? 0 : iw) + in_seg_c;
    src.zsrc = wz + wcol;
    src.ssrc = reinterpret_cast<const uint4*>(ws) + wcol;
    src.zpitch = (size_t)words;
    src.spitch = (size_t)words;
  }
  const int KT = p.H / kBK;
  const int st_begin = (int)(((long long)rank * KT) / S);
  const int st_end = (int)(((long long)(rank + 1) * KT) / S);

  float tot[MT][4][4];
  mainloop<MT, kMoeExact, GROUP, RP>(src, smem_u32(smem), tid, 0, st_begin, st_end - st_begin, p.group,
                              groups, tot);

  float* red = reinterpret_cast<float*>(smem);
  store_tile<MT>(red, tid, tot);
  cluster.sync();
  {
    constexpr int kUnits = 16;  // 8-column units of the 128 activation columns
    const int ubeg = (rank * kUnits) / S, uend = ((rank + 1) * kUnits) / S;
    const int nun = uend - ubeg;
    for (int idx = tid; idx < nun * MT * 8; idx += kThreads) {
      const int u = ubeg + idx % nun, m = idx / nun;
      const int col = blockIdx.y * 128 + u * 8;
      if (col >= p.I) continue;
      float gt[8], up[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) gt[j] = up[j] = 0.f;
      for (int q = 0; q < S; ++q) {
        const float* peer = cluster.map_shared_rank(red, q) + m * kRedPitch + u * 8;
        const float4 a = *reinterpret_cast<const float4*>(peer);
        const float4 b = *reinterpret_cast<const float4*>(peer + 4);
        const float4 c = *reinterpret_cast<const float4*>(peer + 128);
        const float4 d = *reinterpret_cast<const float4*>(peer + 132);
        gt[0] += a.x; gt[1] += a.y; gt[2] += a.z; gt[3] += a.w;
        gt[4] += b.x; gt[5] += b.y; gt[6] += b.z; gt[7] += b.w;
        up[0] += c.x; up[1] += c.y; up[2] += c.z; up[3] += c.w;
        up[4] += d.x; up[5] += d.y; up[6] += d.z; up[7] += d.w;
      }
      __align__(16) __half o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __float2half_rn(gt[j] / (1.f + __expf(-gt[j])) * up[j]);
      *reinterpret_cast<uint4*>(p.act + (size_t)(pos0 + m) * p.I + col) =
          *reinterpret_cast<uint4*>(o);
    }
  }
  cluster.sync();
}

struct Gemm2Params {
  const __half* act;         // [capacity, I]
  const uint32_t* w2_q;      // [E, I, H/8]
  const __half* w2_s;        // [E, I/G, H]
  const uint32_t* w2_z;      // [E, I/G, H/8]
  const float* topk_weights; // [T * topk]
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post_pad;
  __half* pair_out;          // [T * topk, H]
  int numel, H, I, group;
  uint32_t* tickets;         // direct mode: one counter per (token, column slab); else nullptr
  __half* out;               // direct mode: [T, H], written by the cluster that finishes a token's
  int topk;                  //              last pair for a slab
};

template <int MT, int GROUP, bool RP>
__global__ void __launch_bounds__(kThreads, MT == 1 ? 5 : 4) moe_gemm2_kernel(const Gemm2Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ int s_fid[8 * MT];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int S = (int)cluster.num_blocks();
  const int blk = blockIdx.z;
  const int pos0 = blk * (8 * MT);
  pdl_launch_dependents();
  pdl_wait();
  // both loads in flight together (expert_ids covers every block of the grid)
  const int post = p.num_post_pad ? p.num_post_pad[0] : 0x7fffffff;
  const int e = p.expert_ids[blk];
  if (pos0 >= post || e < 0) return;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2;
  const int words = p.H / kPack;
  const int word0 = blockIdx.y * (kBN / kPack);
  const int groups = p.I / p.group;
  const uint32_t* wq = p.w2_q + (size_t)e * p.I * words;
  const uint32_t* wz = p.w2_z + (size_t)e * groups * words;
  const __half* ws = p.w2_s + (size_t)e * groups * p.H;
  if (tid < 8 * MT) s_fid[tid] = row_pair(p.sorted_ids, pos0, tid, blk, p.numel);

  TileSrc<MT> src;
  {
    if (RP) {
      const int wc = word0 + (tid & 31);
      src.wvalid = wc < words;
      src.wsrc = wq + (size_t)(src.wvalid ? wc : 0) * 4;
      src.wrow_words = (size_t)words * 4;
    } else {
      const int wc = word0 + (tid & 7) * 4;
      src.wvalid = wc < words;
      src.wsrc = wq + (src.wvalid ? wc : 0);
      src.wrow_words = (size_t)words;
    }
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      const int row = (tid >> 4) + 8 * j;
      src.xvalid[j] = row_pair(p.sorted_ids, pos0, row, blk, p.numel) < p.numel;
      src.xsrc[j] = p.act + (size_t)(pos0 + row) * p.I + (tid & 15) * 8;
    }
    const int wcol = word0 + 8 * warp + g;
    const int wcol_ld = wcol < words ? wcol : words - 1;
    src.zsrc = wz + wcol_ld;
    src.ssrc = reinterpret_cast<const uint4*>(ws) + wcol_ld;
    src.zpitch = (size_t)words;
    src.spitch = (size_t)words;
  }
  const int KT = p.I / kBK;
  const int st_begin = (int)(((long long)rank * KT) / S);
  const int st_end = (int)(((long long)(rank + 1) * KT) / S);

  float tot[MT][4][4];
  mainloop<MT, kMoeExact, GROUP, RP>(src, smem_u32(smem), tid, 0, st_begin, st_end - st_begin, p.group,
                              groups, tot);

  float* red = reinterpret_cast<float*>(smem);
  store_tile<MT>(red, tid, tot);
  cluster.sync();
  {
    constexpr int kUnits = kBN / 8;
    const int ubeg = (rank * kUnits) / S, uend = ((rank + 1) * kUnits) / S;
    const int nun = uend - ubeg;
    for (int idx = tid; idx < nun * MT * 8; idx += kThreads) {
      const int u = ubeg + idx % nun, m = idx / nun;
      const int n = blockIdx.y * kBN + u * 8;
      const int fid = s_fid[m];
      if (fid >= p.numel || n >= p.H) continue;
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
      for (int q = 0; q < S; ++q) {
        const float* peer = cluster.map_shared_rank(red, q) + m * kRedPitch + u * 8;
        const float4 a = *reinterpret_cast<const float4*>(peer);
        const float4 b = *reinterpret_cast<const float4*>(peer + 4);
        v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
        v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
      }
      const float rw = __ldg(p.topk_weights + fid);
      __align__(16) __half o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __float2half_rn(v[j] * rw);
      *reinterpret_cast<uint4*>(p.pair_out + (size_t)fid * p.H + n) = *reinterpret_cast<uint4*>(o);
    }
  }
  cluster.sync();
  // Direct mode: the sum over a token's slots is done here instead of in moe_sum_kernel.  The
  // cluster that finishes a token's last pair for this column slab adds the topk rows in slot
  // order (the same fp32 sum of the stored fp16 values, so the result does not depend on which
  // cluster comes last).
  if (p.tickets != nullptr && rank == 0) {
    __shared__ int s_last;
    const int token = blk / p.topk;
    if (tid == 0) {
      __threadfence();
      const unsigned t = atomicAdd(p.tickets + token * gridDim.y + blockIdx.y, 1u);
      s_last = t == (unsigned)p.topk - 1u;
      if (s_last) __threadfence();
    }
    __syncthreads();
    if (s_last) {
      for (int u = tid; u < kBN / 8; u += kThreads) {
        const int n = blockIdx.y * kBN + u * 8;
        if (n >= p.H) continue;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.f;
        for (int sl = 0; sl < p.topk; ++sl) {
          const uint4 r = __ldcg(reinterpret_cast<const uint4*>(
              p.pair_out + ((size_t)token * p.topk + sl) * p.H + n));
          const __half* h = reinterpret_cast<const __half*>(&r);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] += __half2float(h[j]);
        }
        __align__(16) __half o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = __float2half_rn(v[j]);
        *reinterpret_cast<uint4*>(p.out + (size_t)token * p.H + n) = *reinterpret_cast<uint4*>(o);
      }
    }
  }
}

// out[t, h] = sum_slot pair_out[t * topk + slot, h]; one thread per 8 columns.
__global__ void __launch_bounds__(256)
moe_sum_kernel(const __half* __restrict__ pair_out, __half* __restrict__ out, int T, int topk,
               int H) {
  const int units = H / 8;
  const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (idx >= (long long)T * units) return;
  const int t = (int)(idx / units), u = (int)(idx % units);
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = 0.f;
  for (int s = 0; s < topk; ++s) {
    const uint4 r =
        __ldg(reinterpret_cast<const uint4*>(pair_out + ((size_t)t * topk + s) * H) + u);
    const __half* h = reinterpret_cast<const __half*>(&r);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] += __half2float(h[j]);
  }
  __align__(16) __half o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = __float2half_rn(v[j]);
  *(reinterpret_cast<uint4*>(out + (size_t)t * H) + u) = *reinterpret_cast<uint4*>(o);
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int pick_cluster(int tiles, int KT) {
  // five CTAs are resident per SM; filling those slots measured 6 % (T = 1) and 13 % (T = 4)
  // faster than two per SM, ten per SM slower again
  int S = tiles > 0 ? (5 * sm_count()) / tiles : 8;
  S = S < 1 ? 1 : (S > 8 ? 8 : S);
  return S > KT ? KT : S;
}

template <typename P>
int launch_clustered(void (*kernel)(const P), const P& p, dim3 grid, int S, int smem,
                     cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = add_pdl_attribute(attr, 1);
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) {
    cudaGetLastError();
    return AWQ_B200_ERR_LAUNCH;
  }
  return AWQ_B200_OK;
}

}  // namespace

template <typename T, int NV>
void launch_topk_nv(const void* gating, int T_, int E, int topk, int renormalize,
                    float* topk_weights, int32_t* topk_ids, int32_t* token_expert_indices,
                    cudaStream_t stream) {
  const int grid = (T_ + kTopkWarps - 1) / kTopkWarps;
  launch_pdl(topk_softmax_kernel<T, NV>, dim3(grid), dim3(kTopkWarps * 32), 0, stream,
             static_cast<const T*>(gating), T_, E, topk, renormalize, topk_weights, topk_ids,
             token_expert_indices);
}

template <typename T>
void launch_topk_t(const void* gating, int T_, int E, int topk, int renormalize,
                   float* topk_weights, int32_t* topk_ids, int32_t* token_expert_indices,
                   cudaStream_t stream) {
  if (E <= 128)
    launch_topk_nv<T, 4>(gating, T_, E, topk, renormalize, topk_weights, topk_ids,
                         token_expert_indices, stream);
  else if (E <= 256)
    launch_topk_nv<T, 8>(gating, T_, E, topk, renormalize, topk_weights, topk_ids,
                         token_expert_indices, stream);
  else
    launch_topk_nv<T, 32>(gating, T_, E, topk, renormalize, topk_weights, topk_ids,
                          token_expert_indices, stream);
}

int launch_topk_softmax(const void* gating, int gating_dtype, int T, int E, int topk,
                        int renormalize, float* topk_weights, int32_t* topk_ids,
                        int32_t* token_expert_indices, cudaStream_t stream) {
  if (gating_dtype == 0)
    launch_topk_t<float>(gating, T, E, topk, renormalize, topk_weights, topk_ids,
                         token_expert_indices, stream);
  else
    launch_topk_t<__half>(gating, T, E, topk, renormalize, topk_weights, topk_ids,
                          token_expert_indices, stream);
  return cudaGetLastError() == cudaSuccess ? AWQ_B200_OK : AWQ_B200_ERR_LAUNCH;
}

int launch_moe_align(const int32_t* topk_ids, int numel, int E, int block,
                     const int32_t* expert_map, int32_t* sorted_ids, int64_t sorted_capacity,
                     int32_t* expert_ids, int32_t* num_post_pad, cudaStream_t stream) {
  const int nchunks = (numel + kAlignChunk - 1) / kAlignChunk;
  const int grid = nchunks < 1 ? 1 : (nchunks < kAlignMaxCtas ? nchunks : kAlignMaxCtas);
  const size_t smem = (size_t)(3 * E + 1 + 8 * E) * sizeof(int);  // <= 45 KB for E <= 1024
  if (launch_pdl(moe_align_kernel, dim3(grid), dim3(kAlignThreads), smem, stream, topk_ids, numel,
                 E, block, expert_map, sorted_ids, sorted_capacity, expert_ids,
                 num_post_pad) != cudaSuccess) {
    cudaGetLastError();
    return AWQ_B200_ERR_LAUNCH;
  }
  return AWQ_B200_OK;
}

int launch_moe_sum(const __half* pair_out, __half* out, int T, int topk, int H,
                   cudaStream_t stream) {
  const long long work = (long long)T * (H / 8);
  if (launch_pdl(moe_sum_kernel, dim3((unsigned)((work + 255) / 256)), dim3(256), 0, stream,
                 pair_out, out, T, topk, H) != cudaSuccess) {
    cudaGetLastError();
    return AWQ_B200_ERR_LAUNCH;
  }
  return AWQ_B200_OK;
}

// Row block of the permutation: 128 (tcgen05 grouped GEMMs) once an expert sees 36 rows or more
// on average and the shapes fit that kernel's tiles (measured at 128 experts, top-8: the grouped
// kernels take 271 us from T = 256 to 768, the streaming kernels 169 / 215 / 254 / 336 us at
// T = 256 / 384 / 512 / 768); 8 up to eight rows per expert on
// average (one 8-token tile streams a third faster than two, which outweighs the experts that
// need a second block up to there: measured crossover between T = 128 and 192 at 128 experts,
// top-8); else 16.
int moe_block_size(int T, int topk, int E, int H, int I, int group) {
  const long long pairs = (long long)T * topk;
  if (pairs >= 36LL * E && moe_tc_supported(H, I, group)) return 128;
  return pairs <= 8LL * E ? 8 : 16;
}

bool moe_supported(int H, int I, int group, int block) {
  if (block == 128) return moe_tc_supported(H, I, group);
  // gate/up halves start on 16-byte boundaries (I % 32), stages are 128 rows of K
  return (block == 8 || block == 16) && H % kBK == 0 && I % kBK == 0 && I % 32 == 0 && H % 32 == 0 &&
         (group == 128 || group == 64 || group == 32);
}

size_t moe_workspace_bytes(int T, int topk, int E, int H, int I) {
  if (T <= 0 || topk <= 0 || E <= 0 || H <= 0 || I <= 0) return 0;
  const int block = 16;  // the larger of the two streaming block sizes bounds the row count
  const int64_t cap = awq_b200_moe_sorted_capacity((int64_t)T * topk, E, block);
  const int64_t rows = (cap + block - 1) / block * block;
  const size_t small = align_up((size_t)rows * I * sizeof(__half), 256) +
                       align_up((size_t)T * topk * H * sizeof(__half), 256) + kMoeDirectTicketBytes;
  if (moe_block_size(T, topk, E, H, I, 128) == 128) {
    const size_t big = moe_tc_workspace_bytes(T, topk, E, H, I);
    return big > small ? big : small;
  }
  return small;
}

// Bytes of scratch the launchers below lay out for a call: the row count comes from the caller's
// sorted_capacity (which may exceed the minimum, e.g. a permutation built for the global expert
// count under expert parallelism), so the size check uses exactly what the layout uses.
size_t moe_layout_bytes(const MoeArgs& a) {
  if (a.block == 128) return moe_tc_layout_bytes(a);
  const int64_t rows = (a.sorted_capacity + a.block - 1) / a.block * a.block;
  return align_up((size_t)rows * a.I * sizeof(__half), 256) +
         align_up((size_t)a.T * a.topk * a.H * sizeof(__half), 256) +
         (a.direct ? (size_t)kMoeDirectTicketBytes : 0);
}

template <int MT, int GROUP, bool RP>
int launch_moe_gemms(const MoeArgs& a, __half* act, __half* pair_out, uint32_t* tickets, int numel,
                     int nblk, cudaStream_t stream) {
  constexpr int smem = Cfg<MT>::kSmemBytes;
  static std::atomic<bool> attr_done[64];  // zero-initialised; setting the attribute twice is harmless
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return AWQ_B200_ERR_DEVICE;
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(moe_gemm1_kernel<MT, GROUP, RP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             smem) != cudaSuccess ||
        cudaFuncSetAttribute(moe_gemm2_kernel<MT, GROUP, RP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             smem) != cudaSuccess)
      return AWQ_B200_ERR_LAUNCH;
    attr_done[dev] = true;
  }
  {
    Gemm1Params p{a.x, a.w13_q, a.w13_s, a.w13_z, a.sorted_ids, a.expert_ids, a.num_post_pad,
                  act, numel, a.topk, a.H, a.I, a.group, tickets,
                  tickets ? a.T * ((a.H + kBN - 1) / kBN) : 0};
    const int slabs = (a.I + 127) / 128;
    const int S = pick_cluster(slabs * nblk, a.H / kBK);
    if (int rc = launch_clustered(moe_gemm1_kernel<MT, GROUP, RP>, p, dim3(S, slabs, nblk), S, smem, stream))
      return rc;
  }
  {
    Gemm2Params p{act, a.w2_q, a.w2_s, a.w2_z, a.topk_weights, a.sorted_ids, a.expert_ids,
                  a.num_post_pad, pair_out, numel, a.H, a.I, a.group, tickets, a.out, a.topk};
    const int slabs = (a.H + kBN - 1) / kBN;
    const int S = pick_cluster(slabs * nblk, a.I / kBK);
    if (int rc = launch_clustered(moe_gemm2_kernel<MT, GROUP, RP>, p, dim3(S, slabs, nblk), S, smem, stream))
      return rc;
  }
  return AWQ_B200_OK;
}

int launch_moe_experts(const MoeArgs& a, void* workspace, size_t workspace_bytes,
                       cudaStream_t stream) {
  // the decode-layout copy is read by the streaming kernels only (group 128, K % 128)
  if (a.decode_layout && (a.block == 128 || a.group != 128)) return AWQ_B200_ERR_SHAPE;
  if (a.block == 128) return launch_moe_experts_tc(a, workspace, workspace_bytes, stream);
  const size_t need = moe_layout_bytes(a);
  if (workspace == nullptr || workspace_bytes < need) return AWQ_B200_ERR_WORKSPACE;
  const int numel = a.T * a.topk;
  const int64_t rows = (a.sorted_capacity + a.block - 1) / a.block * a.block;
  const int nblk = (int)(rows / a.block);
  __half* act = static_cast<__half*>(workspace);
  __half* pair_out = reinterpret_cast<__half*>(static_cast<uint8_t*>(workspace) +
                                               align_up((size_t)rows * a.I * sizeof(__half), 256));
  // direct mode: the down GEMM sums a token's slots itself when the counters fit
  uint32_t* tickets = nullptr;
  if (a.direct && (size_t)a.T * ((a.H + kBN - 1) / kBN) * sizeof(uint32_t) <= kMoeDirectTicketBytes)
    tickets = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(pair_out) +
                                          align_up((size_t)numel * a.H * sizeof(__half), 256));

  if (a.expert_parallel) {
    // pairs routed to experts of other ranks are never written: they must read as zero
    if (cudaMemsetAsync(pair_out, 0, (size_t)numel * a.H * sizeof(__half), stream) != cudaSuccess)
      return AWQ_B200_ERR_LAUNCH;
  }
  int rc;
  if (a.decode_layout)
    rc = a.block == 8 ? launch_moe_gemms<1, 128, true>(a, act, pair_out, tickets, numel, nblk, stream)
                      : launch_moe_gemms<2, 128, true>(a, act, pair_out, tickets, numel, nblk, stream);
  else if (a.group == 128)
    rc = a.block == 8 ? launch_moe_gemms<1, 128, false>(a, act, pair_out, tickets, numel, nblk, stream)
                      : launch_moe_gemms<2, 128, false>(a, act, pair_out, tickets, numel, nblk, stream);
  else
    rc = a.block == 8 ? launch_moe_gemms<1, 0, false>(a, act, pair_out, tickets, numel, nblk, stream)
                      : launch_moe_gemms<2, 0, false>(a, act, pair_out, tickets, numel, nblk, stream);
  if (rc) return rc;
  if (tickets == nullptr) {
    const long long work = (long long)a.T * (a.H / 8);
    if (launch_pdl(moe_sum_kernel, dim3((unsigned)((work + 255) / 256)), dim3(256), 0, stream,
                   (const __half*)pair_out, a.out, a.T, a.topk, a.H) != cudaSuccess) {
      cudaGetLastError();
      return AWQ_B200_ERR_LAUNCH;
    }
  }
  return AWQ_B200_OK;
}

// ---- expert GEMMs with the scratch held inside the library ------------------------------------
//
// Same work as launch_moe_experts, but the activation / per-pair buffers live in
// g_moe_static_scratch, a fixed array in device memory that every GPU loading the library
// reserves until the process exits.  Nothing is allocated at call time.
//
// g_moe_static_scratch is a device symbol: in host code its name is only a handle, not an
// address a kernel could use, so the device address is looked up once per device with
// cudaGetSymbolAddress (that device being current) and cached.  The lookup happens in the first
// call on each device.
int launch_moe_experts_static(const MoeArgs& a, cudaStream_t stream) {
  if (moe_layout_bytes(a) > kMoeStaticScratchBytes) return AWQ_B200_ERR_LIMIT;
  static std::mutex mu;
  static void* scratch_addr[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return AWQ_B200_ERR_DEVICE;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (scratch_addr[dev] == nullptr) {
      // first use of this translation unit's device globals on this GPU: with lazy module
      // loading this is also where the 16 MiB get bound
      void* ptr = nullptr;
      if (cudaGetSymbolAddress(&ptr, g_moe_static_scratch) != cudaSuccess || ptr == nullptr) {
        cudaGetLastError();
        return AWQ_B200_ERR_SYMBOL;
      }
      scratch_addr[dev] = ptr;
    }
    scratch = scratch_addr[dev];
  }
  // The array still holds whatever the previous call left there.  Every row the kernels read is
  // written earlier in the same call; the one region that must start at zero (per-pair outputs
  // under expert parallelism) is cleared inside launch_moe_experts.
  return launch_moe_experts(a, scratch, kMoeStaticScratchBytes, stream);
}

size_t moe_static_scratch_bytes() { return kMoeStaticScratchBytes; }

}  // namespace awq
