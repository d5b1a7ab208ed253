// Grouped AWQ expert GEMMs on tcgen05 for prefill-sized token counts (many rows per expert).
//
// The (token, slot) pairs are already sorted by expert with every expert's run padded to 128 rows
// (moe_align_kernel, block = 128), so row block b of the permuted list belongs to exactly one
// expert, expert_ids[b].  One CTA computes one [128 rows x 256 columns] tile of one row block
// with the pipeline of gemm_tc.cu (TMA -> dequantisation warps -> tcgen05.mma into TMEM):
//
//   moe_gather_kernel   x_perm[pos] = x[token(pos)]           (padding rows = 0)
//   moe_tc_kernel<1>    gate_up: columns [128 j, 128 j + 128) of the gate half and of the up half
//                       form one 256-column tile; epilogue silu(gate) * up -> act[pos] fp16
//   moe_tc_kernel<2>    down: act rows x w2[e]; epilogue times routed weight ->
//                       pair_out[flat pair id] fp16
// followed by moe_sum_kernel (moe.cu).
//
// The packed weights of a tile arrive as two TMA boxes of [64 rows x 16 words] ("left" and
// "right" half of the tile's columns; for gate_up these are the gate and the up segment).
// Every wait is bounded (tc_ptx.cuh).
#include "tc_ptx.cuh"

namespace awq {

namespace {

using namespace tc;

constexpr int kMBM = 128, kMBN = 256, kMBK = 64;
constexpr int kMDqThreads = 256;
constexpr int kMThreads = kMDqThreads + 64;
constexpr int kMStages = 3;
constexpr int kMABytes = kMBM * kMBK * 2;         // 16384
constexpr int kMBBytes = kMBK * kMBN * 2;         // 32768
constexpr int kMRawHalf = kMBK * 16 * 4;          // 4096: one [64 x 16 words] box
constexpr int kMStageBytes = kMABytes + kMBBytes + 2 * kMRawHalf;
constexpr int kMSmemBytes = kMStages * kMStageBytes + 256 + 1024;

struct MoeTcParams {
  const __half* scales;       // stacked [E, K/G, N]
  const uint32_t* qzeros;     // stacked [E, K/G, N/8]
  const float* topk_weights;  // [T * topk]            (mode 2)
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post_pad;
  __half* out;                // mode 1: act [rows, I]; mode 2: pair_out [T * topk, H]
  int numel, K, N, group;     // N = weight columns per expert (2I or H)
  int half_cols;              // mode 1: I (offset of the up half); mode 2: unused
};

// MODE 1: gate_up + silu*mul, MODE 2: down + routed weight.
template <int MODE>
__global__ void __launch_bounds__(kMThreads, 1)
moe_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
              const MoeTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ volatile int s_abort;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_fid[kMBM];

  const int blk = blockIdx.x;
  const int pos0 = blk * kMBM;
  if (pos0 >= p.num_post_pad[0]) return;  // uniform over the CTA, before any barrier
  const int e = p.expert_ids[blk];
  if (e < 0) return;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + kMStages * kMStageBytes;
  auto a_addr = [&](int s) { return smem_base + s * kMStageBytes; };
  auto b_addr = [&](int s) { return smem_base + s * kMStageBytes + kMABytes; };
  auto raw_addr = [&](int s) { return smem_base + s * kMStageBytes + kMABytes + kMBBytes; };
  auto full_raw = [&](int s) { return bar_base + 8 * s; };
  auto full_b = [&](int s) { return bar_base + 8 * (kMStages + s); };
  auto empty = [&](int s) { return bar_base + 8 * (2 * kMStages + s); };
  const uint32_t tmem_full = bar_base + 8 * (3 * kMStages);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int KT = p.K / kMBK;
  const int words = p.N / kPack;            // words per weight row of one expert
  const int groups = p.K / p.group;
  // first packed word of the left / right 128-column half of this tile
  const int w_left = MODE == 1 ? blockIdx.y * 16 : blockIdx.y * 32;
  const int w_right = MODE == 1 ? p.half_cols / kPack + blockIdx.y * 16 : blockIdx.y * 32 + 16;

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < kMStages; ++s) {
      mbar_init(full_raw(s), 1);
      mbar_init(full_b(s), kMDqThreads);
      mbar_init(empty(s), 1);
    }
    mbar_init(tmem_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  if (tid < kMBM) s_fid[tid] = p.sorted_ids[pos0 + tid];
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "r"((uint32_t)kMBN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = s_tmem_base;
  bool ok = true;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int it = 0; it < KT; ++it) {
        const int s = it % kMStages;
        const uint32_t round = (uint32_t)(it / kMStages);
        if (!mbar_wait(empty(s), (round & 1u) ^ 1u, &s_abort, 21)) break;
        const int k0 = it * kMBK;
        mbar_arrive_expect_tx(full_raw(s), kMABytes + 2 * kMRawHalf);
        tma_load_2d(a_addr(s), &map_a, k0, pos0, full_raw(s));
        tma_load_2d(raw_addr(s), &map_w, w_left, e * p.K + k0, full_raw(s));
        tma_load_2d(raw_addr(s) + kMRawHalf, &map_w, w_right, e * p.K + k0, full_raw(s));
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 16) | ((uint32_t)(kMBN >> 3) << 17) |
                                 ((uint32_t)(kMBM >> 4) << 24);
      for (int it = 0; it < KT && ok; ++it) {
        const int s = it % kMStages;
        const uint32_t round = (uint32_t)(it / kMStages);
        ok = mbar_wait(full_raw(s), round & 1u, &s_abort, 22) &&
             mbar_wait(full_b(s), round & 1u, &s_abort, 23);
        if (!ok) break;
        tc_fence_after();
        const uint64_t da = make_desc(a_addr(s), 16, 1024);
        const uint64_t db = make_desc(b_addr(s), 8192, 1024);
#pragma unroll
        for (int k16 = 0; k16 < kMBK / 16; ++k16)
          umma_f16_ss(tmem_d, da + (uint64_t)((k16 * 32) >> 4), db + (uint64_t)((k16 * 2048) >> 4),
                      idesc, (it > 0 || k16 > 0) ? 1u : 0u);
        umma_commit(empty(s));
      }
      if (ok) umma_commit(tmem_full);
    }
  } else {
    // ------------------------------------------------------------------ dequant warps 0-7
    // threads 0-127 convert the left half of the tile's columns, 128-255 the right half;
    // inside a half: word column c = t % 16, rows (t / 16) + 8 j
    const int half = tid >> 7, th = tid & 127;
    const int c = th & 15, krow0 = th >> 4;
    const int wcol = min((half ? w_right : w_left) + c, words - 1);
    const uint32_t b_off = (uint32_t)(half * 2 + (c >> 3)) * (kMBK * 128) + krow0 * 128 +
                           (((uint32_t)(c & 7) ^ (uint32_t)(krow0 & 7)) << 4);
    const uint32_t raw_off = (uint32_t)half * kMRawHalf + (uint32_t)(krow0 * 16 + c) * 4;
    const uint32_t* zbase = p.qzeros + (size_t)e * groups * words + wcol;
    const uint4* sbase = reinterpret_cast<const uint4*>(p.scales + (size_t)e * groups * p.N) + wcol;
    int cur_group = -1;
    __half2 zE0, zO0, zE1, zO1, sE0, sO0, sE1, sO1;
    for (int it = 0; it < KT && ok; ++it) {
      const int s = it % kMStages;
      const uint32_t round = (uint32_t)(it / kMStages);
      const int grp = (it * kMBK) / p.group;
      if (grp != cur_group) {
        cur_group = grp;
        const uint32_t zw = __ldg(zbase + (size_t)grp * words);
        const uint4 sv = __ldg(sbase + (size_t)grp * words);
        const uint32_t zw8 = zw >> 8;
        zE0 = as_half2(lop3_and_or(zw, 0x000F000Fu, 0x64006400u));
        zO0 = as_half2(lop3_and_or(zw, 0x00F000F0u, 0x64006400u));
        zE1 = as_half2(lop3_and_or(zw8, 0x000F000Fu, 0x64006400u));
        zO1 = as_half2(lop3_and_or(zw8, 0x00F000F0u, 0x64006400u));
        const __half2 r16 = __float2half2_rn(0.0625f);
        sE0 = as_half2(sv.x);
        sO0 = __hmul2(as_half2(sv.y), r16);
        sE1 = as_half2(sv.z);
        sO1 = __hmul2(as_half2(sv.w), r16);
      }
      ok = mbar_wait(full_raw(s), round & 1u, &s_abort, 24);
      if (!ok) break;
      const uint32_t raw = raw_addr(s) + raw_off, bt = b_addr(s) + b_off;
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w[j]) : "r"(raw + j * (8 * 16 * 4)));
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t w8 = w[j] >> 8;
        uint4 o;
        o.x = as_u32(__hmul2(__hsub2(as_half2(lop3_and_or(w[j], 0x000F000Fu, 0x64006400u)), zE0), sE0));
        o.y = as_u32(__hmul2(__hsub2(as_half2(lop3_and_or(w[j], 0x00F000F0u, 0x64006400u)), zO0), sO0));
        o.z = as_u32(__hmul2(__hsub2(as_half2(lop3_and_or(w8, 0x000F000Fu, 0x64006400u)), zE1), sE1));
        o.w = as_u32(__hmul2(__hsub2(as_half2(lop3_and_or(w8, 0x00F000F0u, 0x64006400u)), zO1), sO1));
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(bt + j * (8 * 128)), "r"(o.x),
                     "r"(o.y), "r"(o.z), "r"(o.w)
                     : "memory");
      }
      fence_proxy_async();
      mbar_arrive(full_b(s));
    }

    // ---------------------------------------------------------------- epilogue
    // warp w reads TMEM lanes 32 (w % 4) ..; warps 4-7 take the upper 64 of the 128 column pairs
    const int q = warp & 3, hi = warp >> 2;
    const uint32_t tlane = tmem_d + ((uint32_t)(q * 32) << 16);
    ok = ok && mbar_wait(tmem_full, 0, &s_abort, 25);
    if (ok) {
      tc_fence_after();
      const int row = q * 32 + lane;
      const int fid = s_fid[row];
      if (MODE == 1) {
        // act[pos, 128 j + c] = silu(D[c]) * D[128 + c]
        __half* dst_row = p.out + (size_t)(pos0 + row) * p.half_cols + blockIdx.y * 128;
#pragma unroll 1
        for (int c0 = hi * 64; c0 < hi * 64 + 64; c0 += 32) {
          uint32_t g[32], u[32];
          tmem_ld32(tlane + (uint32_t)c0, g);
          tmem_ld32(tlane + (uint32_t)(128 + c0), u);
          __align__(16) __half2 h[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
            const float a0 = g0 / (1.f + __expf(-g0)) * __uint_as_float(u[2 * j]);
            const float a1 = g1 / (1.f + __expf(-g1)) * __uint_as_float(u[2 * j + 1]);
            h[j] = __floats2half2_rn(a0, a1);
          }
          if (blockIdx.y * 128 + c0 < p.half_cols) {
            uint4* dst = reinterpret_cast<uint4*>(dst_row + c0);
            const uint4* srcv = reinterpret_cast<const uint4*>(h);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = srcv[j];
          }
        }
      } else {
        const bool valid = fid < p.numel;
        const float rw = valid ? __ldg(p.topk_weights + fid) : 0.f;
        __half* dst_row = p.out + (size_t)(valid ? fid : 0) * p.N + blockIdx.y * kMBN;
#pragma unroll 1
        for (int c0 = hi * 128; c0 < hi * 128 + 128; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(tlane + (uint32_t)c0, r);
          if (valid && blockIdx.y * kMBN + c0 < p.N) {
            __align__(16) __half2 h[16];
#pragma unroll
            for (int j = 0; j < 16; ++j)
              h[j] = __floats2half2_rn(__uint_as_float(r[2 * j]) * rw,
                                       __uint_as_float(r[2 * j + 1]) * rw);
            uint4* dst = reinterpret_cast<uint4*>(dst_row + c0);
            const uint4* srcv = reinterpret_cast<const uint4*>(h);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = srcv[j];
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d),
                 "r"((uint32_t)kMBN)
                 : "memory");
  }
}

// x_perm[pos, :] = x[token(pos), :] for the rows of the used blocks; padding rows are zero.
__global__ void __launch_bounds__(256)
moe_gather_kernel(const __half* __restrict__ x, const int32_t* __restrict__ sorted_ids,
                  const int32_t* __restrict__ num_post_pad, __half* __restrict__ x_perm, int numel,
                  int topk, int H) {
  const int pos = blockIdx.x;
  if (pos >= num_post_pad[0]) return;
  const int fid = sorted_ids[pos];
  uint4* dst = reinterpret_cast<uint4*>(x_perm + (size_t)pos * H);
  if (fid < numel) {
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(fid / topk) * H);
    for (int i = threadIdx.x; i < H / 8; i += 256) dst[i] = __ldg(src + i);
  } else {
    for (int i = threadIdx.x; i < H / 8; i += 256) dst[i] = make_uint4(0, 0, 0, 0);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// rows x cols fp16 activations, box [64 k x 128 rows], 128-byte swizzle
int make_a_map(CUtensorMap* m, const __half* base, int64_t rows, int cols) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return AWQ_B200_ERR_DRIVER;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kMBK, (cuuint32_t)kMBM};
  const cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(base), dims, strides, box,
             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
             ? AWQ_B200_OK
             : AWQ_B200_ERR_DRIVER;
}

// stacked packed weights [E * K rows, N / 8 words], box [16 words x 64 rows]
int make_w_map(CUtensorMap* m, const uint32_t* base, int64_t rows, int words) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return AWQ_B200_ERR_DRIVER;
  const cuuint64_t dims[2] = {(cuuint64_t)words, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)words * 4};
  const cuuint32_t box[2] = {16, (cuuint32_t)kMBK};
  const cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<uint32_t*>(base), dims, strides, box,
             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
             ? AWQ_B200_OK
             : AWQ_B200_ERR_DRIVER;
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

int launch_moe_experts_tc(const MoeArgs& a, void* workspace, size_t workspace_bytes,
                          cudaStream_t stream) {
  if (a.block != kMBM || !moe_tc_supported(a.H, a.I, a.group)) return AWQ_B200_ERR_SHAPE;
  const size_t need = moe_tc_workspace_bytes(a.T, a.topk, a.E, a.H, a.I);
  if (workspace == nullptr || workspace_bytes < need) return AWQ_B200_ERR_WORKSPACE;
  const int numel = a.T * a.topk;
  const int64_t rows = (a.sorted_capacity + kMBM - 1) / kMBM * kMBM;
  const int nblk = (int)(rows / kMBM);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  __half* x_perm = reinterpret_cast<__half*>(ws);
  __half* act = reinterpret_cast<__half*>(ws + align_up((size_t)rows * a.H * 2, 256));
  __half* pair_out = reinterpret_cast<__half*>(ws + align_up((size_t)rows * a.H * 2, 256) +
                                               align_up((size_t)rows * a.I * 2, 256));

  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return AWQ_B200_ERR_DEVICE;
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(moe_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kMSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(moe_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kMSmemBytes) != cudaSuccess)
      return AWQ_B200_ERR_LAUNCH;
    attr_done[dev] = true;
  }
  CUtensorMap map_x, map_act, map_w13, map_w2;
  if (int rc = make_a_map(&map_x, x_perm, rows, a.H)) return rc;
  if (int rc = make_a_map(&map_act, act, rows, a.I)) return rc;
  if (int rc = make_w_map(&map_w13, a.w13_q, (int64_t)a.E * a.H, 2 * a.I / kPack)) return rc;
  if (int rc = make_w_map(&map_w2, a.w2_q, (int64_t)a.E * a.I, a.H / kPack)) return rc;

  if (a.expert_parallel) {
    if (cudaMemsetAsync(pair_out, 0, (size_t)numel * a.H * 2, stream) != cudaSuccess)
      return AWQ_B200_ERR_LAUNCH;
  }
  moe_gather_kernel<<<(unsigned)rows, 256, 0, stream>>>(a.x, a.sorted_ids, a.num_post_pad, x_perm,
                                                        numel, a.topk, a.H);
  if (cudaGetLastError() != cudaSuccess) return AWQ_B200_ERR_LAUNCH;
  {
    MoeTcParams p{a.w13_s, a.w13_z, nullptr, a.sorted_ids, a.expert_ids, a.num_post_pad, act,
                  numel, a.H, 2 * a.I, a.group, a.I};
    moe_tc_kernel<1><<<dim3(nblk, a.I / 128), kMThreads, kMSmemBytes, stream>>>(map_x, map_w13, p);
    if (cudaGetLastError() != cudaSuccess) return AWQ_B200_ERR_LAUNCH;
  }
  {
    MoeTcParams p{a.w2_s, a.w2_z, a.topk_weights, a.sorted_ids, a.expert_ids, a.num_post_pad,
                  pair_out, numel, a.I, a.H, a.group, 0};
    moe_tc_kernel<2><<<dim3(nblk, a.H / kMBN), kMThreads, kMSmemBytes, stream>>>(map_act, map_w2, p);
    if (cudaGetLastError() != cudaSuccess) return AWQ_B200_ERR_LAUNCH;
  }
  return launch_moe_sum(pair_out, a.out, a.T, a.topk, a.H, stream);
}

}  // namespace awq
