// Small-M AWQ GEMM (decode GEMV / small batches, M <= 32): weight streaming at HBM speed.
//
// y[M, N] = x[M, K] @ ((q - z) * s).  A CTA owns a slab of 256 output columns; the K range is
// split over the S CTAs of a thread-block cluster (S <= 8) and, inside a CTA, over WG
// independent warp groups (see stream_core.cuh for the tile mainloop each group runs).  The
// S * WG fp32 partial tiles are combined through distributed shared memory in a fixed order,
// so split-K needs no global scratch and no atomics, and the result is bit-reproducible.
#include <cooperative_groups.h>

#include "stream_core.cuh"

namespace cg = cooperative_groups;

namespace awq {

namespace {

using namespace stream;

struct StreamParams {
  const __half* x;
  const uint32_t* qweight;
  const __half* scales;
  const uint32_t* qzeros;
  const __half* bias;
  __half* out;
  int M, N, K, group;
};

constexpr int kBlocksMT1 = 5;    // resident CTAs per SM the 8-token kernel is sized for
constexpr int kMinStages = 6;    // stages a warp group must have for a K split to pay
constexpr int kMaxCluster = 8;   // portable cluster size
constexpr int kPdlMinStages = 12;
constexpr int min_blocks(int MT, int WG) {
  return WG == 1 ? (MT == 1 ? kBlocksMT1 : (MT == 2 ? 4 : 2)) : (MT == 1 && WG <= 3 ? 2 : 1);
}

template <int MT, bool EXACT, int GROUP, int WG, bool RP>
__global__ void __launch_bounds__(kGroupThreads * WG, min_blocks(MT, WG))
gemm_stream_kernel(const StreamParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int kRing = Cfg<MT>::kSmemBytes;  // bytes of one warp group's ring / partial tile
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int S = (int)cluster.num_blocks();
  pdl_launch_dependents();

  const int wg = threadIdx.x / kGroupThreads;
  const int tid = threadIdx.x % kGroupThreads, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2;
  const int words = p.N / kPack;
  const int word0 = blockIdx.y * (kBN / kPack);
  const int KT = p.K / kBK;
  const int vrank = rank * WG + wg, VS = S * WG;  // this warp group's share of K
  const int st_begin = (int)(((long long)vrank * KT) / VS);
  const int st_end = (int)(((long long)(vrank + 1) * KT) / VS);

  TileSrc<MT> src;
  {
    if (RP) {
      // repacked layout [K/4][N/8][4]: this thread copies the unit of word column tid % 32
      const int wc = word0 + (tid & 31);
      src.wvalid = wc < words;
      src.wsrc = p.qweight + (size_t)(src.wvalid ? wc : 0) * 4;
      src.wrow_words = (size_t)words * 4;
    } else {
      const int wc = word0 + (tid & 7) * 4;
      src.wvalid = wc < words;
      src.wsrc = p.qweight + (src.wvalid ? wc : 0);
      src.wrow_words = (size_t)words;
    }
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      const int row = (tid >> 4) + 8 * j;
      src.xvalid[j] = row < p.M;
      src.xsrc[j] = p.x + (size_t)(src.xvalid[j] ? row : 0) * p.K + (tid & 15) * 8;
    }
    const int wcol = word0 + 8 * warp + g;
    const int wcol_ld = wcol < words ? wcol : words - 1;  // clamped past the N edge
    src.zsrc = p.qzeros + wcol_ld;
    src.ssrc = reinterpret_cast<const uint4*>(p.scales) + wcol_ld;
    src.zpitch = (size_t)words;
    src.spitch = (size_t)words;
  }

  float tot[MT][4][4];
  mainloop<MT, EXACT, GROUP, RP>(src, smem_u32(smem) + wg * kRing, tid, wg, st_begin,
                             st_end - st_begin, p.group, p.K / p.group, tot);

  // ---- reduction over warp groups and cluster ranks through (distributed) shared memory ----
  float* red = reinterpret_cast<float*>(smem);
  store_tile<MT>(red + wg * (kRing / 4), tid, tot);
  cluster.sync();
  {
    constexpr int kUnits = kBN / 8;  // 8-column units in the slab
    const int ubeg = (rank * kUnits) / S, uend = ((rank + 1) * kUnits) / S;
    const int nun = uend - ubeg;
    const int n_slab = blockIdx.y * kBN;
    for (int idx = threadIdx.x; idx < nun * MT * 8; idx += kGroupThreads * WG) {
      const int u = ubeg + idx % nun, m = idx / nun;
      const int n = n_slab + u * 8;
      if (m >= p.M || n >= p.N) continue;
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
      for (int q = 0; q < S; ++q) {
        const float* peer = cluster.map_shared_rank(red, q) + m * kRedPitch + u * 8;
#pragma unroll
        for (int w = 0; w < WG; ++w) {
          const float4 a = *reinterpret_cast<const float4*>(peer + w * (kRing / 4));
          const float4 b = *reinterpret_cast<const float4*>(peer + w * (kRing / 4) + 4);
          v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
          v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
        }
      }
      if (p.bias != nullptr) {
        const uint4 bv = __ldg(reinterpret_cast<const uint4*>(p.bias + n));
        const __half* bh = reinterpret_cast<const __half*>(&bv);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] += __half2float(bh[j]);
      }
      __align__(16) __half o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __float2half_rn(v[j]);
      *reinterpret_cast<uint4*>(p.out + (size_t)m * p.N + n) = *reinterpret_cast<uint4*>(o);
    }
  }
  cluster.sync();  // keep this CTA's shared memory alive until every peer has read it
}

template <int MT, bool EXACT, int GROUP, int WG, bool RP = false>
int launch_variant(const StreamParams& p, int S, cudaStream_t stream) {
  constexpr int smem = Cfg<MT>::kSmemBytes * WG;
  static std::atomic<bool> attr_done[64];  // zero-initialised; setting the attribute twice is harmless
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return AWQ_B200_ERR_DEVICE;
  auto kernel = gemm_stream_kernel<MT, EXACT, GROUP, WG, RP>;
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess)
      return AWQ_B200_ERR_LAUNCH;
    if (kMaxCluster > 8 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) !=
            cudaSuccess)
      return AWQ_B200_ERR_LAUNCH;
    attr_done[dev] = true;
  }
  const int slabs = (p.N + kBN - 1) / kBN;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(S, slabs, 1);
  cfg.blockDim = dim3(kGroupThreads * WG, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  // Early start pays when a warp group has a ring's worth of stages and more to prefetch;
  // with fewer (measured at 4 and 8) the layer ran up to 40 % slower than behind a plain launch.
  const int stages_per_group = (p.K / kBK) / (S * WG);
  cfg.numAttrs = stages_per_group >= kPdlMinStages ? add_pdl_attribute(attr, 1) : 1;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) {
    cudaGetLastError();
    return AWQ_B200_ERR_LAUNCH;
  }
  return AWQ_B200_OK;
}

// Split of K: S cluster ranks x WG warp groups, sized so that about 3-4 warp groups are
// resident per SM (that is what the shared-memory rings allow) without starving a group of
// stages.
template <int MT, bool EXACT, int GROUP, bool RP = false>
int launch_split(const StreamParams& p, cudaStream_t stream) {
  const int slabs = (p.N + kBN - 1) / kBN;
  const int KT = p.K / kBK;
  const int want = (MT == 1 ? kBlocksMT1 : 4) * sm_count();  // warp groups in flight
  int S = want / slabs;
  S = S < 1 ? 1 : (S > kMaxCluster ? kMaxCluster : S);
  while (S > 1 && KT / S < 3) --S;
  // more warp groups per CTA when the cluster limit (8) leaves SMs under-filled
  int wg = 1;
  if (MT == 1) {
    wg = want / (slabs * S);
    wg = wg < 1 ? 1 : (wg > 3 ? 3 : wg);
    while (wg > 1 && KT / (S * wg) < kMinStages) --wg;
  }
  if (wg == 3) return launch_variant<MT, EXACT, GROUP, 3, RP>(p, S, stream);
  if (wg == 2) return launch_variant<MT, EXACT, GROUP, 2, RP>(p, S, stream);
  return launch_variant<MT, EXACT, GROUP, 1, RP>(p, S, stream);
}

template <bool EXACT, int GROUP>
int launch_by_m(const StreamParams& p, cudaStream_t stream) {
  if (p.M <= 8) return launch_split<1, EXACT, GROUP>(p, stream);
  if (p.M <= 16) return launch_split<2, EXACT, GROUP>(p, stream);
  return launch_variant<4, EXACT, GROUP, 1>(
      p, [&] {
        const int slabs = (p.N + kBN - 1) / kBN, KT = p.K / kBK;
        int S = (2 * sm_count()) / slabs;
        S = S < 1 ? 1 : (S > 8 ? 8 : S);
        return S > KT ? KT : S;
      }(),
      stream);
}

}  // namespace

int sm_count() {
  static std::atomic<int> cached[64];  // zero-initialised
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
      v = 148;
    cached[dev] = v;
  }
  return cached[dev].load();
}

bool gemm_stream_supported(int M, int N, int K, int group) {
  // 16-byte cp.async needs 16-byte-aligned weight rows (N % 32) and x rows (K % 128 covers it);
  // a stage is 128 rows and a group must tile it in whole 16-row steps.
  return M >= 1 && M <= 32 && N % 32 == 0 && K % kBK == 0 &&
         (group == 128 || group == 64 || group == 32);
}

bool gemm_stream_rp_supported(int M, int N, int K, int group) {
  return M >= 1 && M <= 8 && N % 32 == 0 && K % kBK == 0 && group == 128;
}

// The same kernel on weights repacked by launch_repack_qweight (M <= 8, group 128).
int launch_gemm_stream_rp(const __half* x, const uint32_t* qweight_rp, const __half* scales,
                          const uint32_t* qzeros, const __half* bias, __half* out, int M, int N,
                          int K, int group, cudaStream_t stream) {
  if (!gemm_stream_rp_supported(M, N, K, group)) return AWQ_B200_ERR_SHAPE;
  StreamParams p{x, qweight_rp, scales, qzeros, bias, out, M, N, K, group};
  return launch_split<1, false, 128, true>(p, stream);
}

int launch_gemm_stream(const __half* x, const uint32_t* qweight, const __half* scales,
                       const uint32_t* qzeros, const __half* bias, __half* out, int M, int N,
                       int K, int group, bool exact, cudaStream_t stream) {
  if (!gemm_stream_supported(M, N, K, group)) return AWQ_B200_ERR_SHAPE;
  StreamParams p{x, qweight, scales, qzeros, bias, out, M, N, K, group};
  if (group == 128)
    return exact ? launch_by_m<true, 128>(p, stream) : launch_by_m<false, 128>(p, stream);
  return exact ? launch_by_m<true, 0>(p, stream) : launch_by_m<false, 0>(p, stream);
}

}  // namespace awq
