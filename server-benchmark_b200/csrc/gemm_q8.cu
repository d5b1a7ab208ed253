// Decode-size AWQ GEMM (M <= 32) in which no thread ever unpacks a weight.
//
//   D[n, m] = sum_k W[k, n] * x[m, k]          (the transposed product: weights are the A operand)
//
// The int4 weights are kept in a load-time copy whose nibbles run along K (awq_b200_repack_kmajor):
// tile (slab, group) = 256 weight columns x 128 k = 16 KB, slabs outermost, so the stream a CTA
// reads is one contiguous range of memory.  Per tile:
//
//   TMA (CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 128-byte swizzle) lays the packed nibbles of a
//     tile into shared memory, 16 nibbles per 16-byte chunk (the upper 8 bytes of a chunk stay
//     unused).  Tile-contiguous boxes of this kind were measured to stream at 6.9 - 7.0 TB/s
//     with four to six boxes in flight per SM, as fast as plain bulk copies;
//   tcgen05.cp ... .b8x16.b4x16_p64 copies shared memory -> tensor memory and widens every nibble
//     q to the byte 4 q on the way: the A operand (128 lanes = weight columns, 128 k, one byte
//     each).  No thread executes an instruction on a weight;
//   tcgen05.mma.kind::i8 multiplies it with the activations, which a small kernel ahead of this
//     one has rewritten as 24-bit fixed point per token, split into three signed byte digits
//     (B operand: 3 x tokens rows, int32 accumulators in tensor memory, exact);
//   the fold warps read the three digit sums of a group, recombine them, subtract
//     zero * sum_k X (the per-group sums come from the activation kernel) and accumulate
//     scale * (...) in fp32 registers: six instructions per (column, token, group).
//
// Accuracy: x is represented as X * amax_token / 2^22 with |X| <= 2^22, so an element is off by
// at most 2^-23 of its row's largest magnitude (fp16 itself carries 2^-11 relative), products and
// group sums are exact integers, and the combination across groups is fp32 as in the other kernels.
//
// Work split (stream-K): the tiles of all slabs, flattened slab-major, are cut into one equal
// contiguous range per CTA, one CTA per SM.  A slab whose groups straddle CTAs is finished by
// the CTA that holds its first group, which processes it last; every other CTA processes its
// share of such a slab first, writes an fp32 partial tile to scratch and raises a flag.  The
// finisher's wait for those flags is bounded like every other wait here.
//
// Roles: producer warp (TMA for the weights, bulk copies for the activation digits), four issuing
// warps (converged, one elected lane each; tile parity x half slab: 4 copies + 4 MMAs per half
// slab), two sets of four fold warps on alternate tiles.  TMEM: 32 columns of A per issuing warp,
// accumulator ring behind them.
//
// The digit tiles use the canonical K-major layout without swizzle: 8 rows x 16 bytes form a
// contiguous 128-byte core matrix, core matrices of one row group follow each other along K.
#include "common.cuh"
#include "tc_ptx.cuh"

namespace awq {

namespace {

using namespace tc;

constexpr int kQ8BN = 256, kQ8BK = 128;
constexpr int kQ8ABytes = kQ8BN * 128;        // shared memory of a tile: 256 rows x 128 B, half of it unused
constexpr int kQ8ATx = kQ8BN * kQ8BK / 2;     // 16384: the tile in memory, and what the TMA reports
constexpr int kQ8ColD = 4 * 32;               // TMEM columns of the four issuing warps' A operands
constexpr int kQ8FoldWarps = 8;
constexpr int kQ8IssueWarps = 4;              // (tile parity, half slab)
constexpr int kQ8IssueWarp = kQ8FoldWarps;
constexpr int kQ8ProducerWarp = kQ8IssueWarp + kQ8IssueWarps;
constexpr int kQ8Threads = 32 * (kQ8ProducerWarp + 1);  // 416
constexpr int kQ8MaxGroups = 256;             // K <= 32768
constexpr int kQ8MaxGrid = 256;

template <int MT>
struct Q8Cfg {
  static constexpr int NB = (3 * MT + 15) / 16 * 16;     // rows of the B tile (MMA N)
  static constexpr int BBytes = NB * 128;
  static constexpr int StageBytes = kQ8ABytes + BBytes;
  // accumulator ring: one slot per half slab (128 columns x NB digit sums), a multiple of four so
  // that a slot always belongs to the same issuing warp / fold set
  static constexpr int NDB =
      ((512 - kQ8ColD) / NB) / 4 * 4 > 12 ? 12 : ((512 - kQ8ColD) / NB) / 4 * 4;
  static constexpr int SxBytes = kQ8MaxGroups * MT * 4;
  static constexpr int RedBytes = 2 * MT * 128 * 4;
  static constexpr int FixedBytes = SxBytes + RedBytes;
  // An even number of stages: tile i and tile i + Ring then have the same parity, so a stage is
  // always consumed by the same pair of issuing warps and each of them sees every phase of its
  // `full` barrier in order.  (With an odd ring a warp that never waited for a stage's first
  // load could ask for the parity of the second one while the first was still in flight -
  // loads complete out of order on a cold TLB - and be told it had completed.)
  static constexpr int Ring = (232448 - 2048 - FixedBytes) / StageBytes / 2 * 2;
  static constexpr int SmemBytes = Ring * StageBytes + FixedBytes + 1024 + 768;
  static_assert(Ring >= 4 && Ring % 2 == 0, "ring too shallow or odd");
  static_assert(NDB >= 4 && kQ8ColD + NDB * NB <= 512, "TMEM columns");
};

struct Q8Params {
  const uint8_t* xq;     // [G][NB x 128] digit tiles
  const __half* scales;
  const uint32_t* qzeros;
  const __half* bias;
  __half* out;
  const float* sx;       // [G][MT]
  const float* xscale;   // [MT]
  float* partial;        // [grid][2][MT][128]
  int* flags;            // [grid]: the launch number of the last partial tile a CTA handed over
  const int* epoch;      // this launch's number, written by the activation kernel
  int M, N, K, G;
  int tiles;             // slabs * G
  uint32_t spin_limit;   // polls of a peer's flag before giving up
};

// K-major shared-memory matrix descriptor without swizzle: lbo = byte distance of core matrices
// adjacent in K, sbo = of 8-row groups.
__device__ __forceinline__ uint64_t make_desc_k(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void cp_128x256b_u4(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.128x256b.b8x16.b4x16_p64 [%0], %1;" ::"r"(taddr), "l"(desc)
               : "memory");
}
__device__ __forceinline__ void umma_i8_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[N]);
template <>
__device__ __forceinline__ void tmem_ld_n<8>(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                 "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld_n<16>(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld_n<32>(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, "
      "[%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void named_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_arrive(int id, int count) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(int* p, int v) {
  asm volatile("st.release.gpu.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ------------------------------------------------------------------------------------------
// Activations -> fixed point.  Token t: amax = max |x|, X = rint(x * 2^22 / amax), written as three
// signed byte digits X = 65536 d2 + 256 d1 + d0 into the B tile of the group (row digit * MT + t,
// canonical K-major layout: byte k of row n at (n / 8) * 1024 + (k / 16) * 128 + (n % 8) * 16 +
// k % 16), with sum_k X per (group, token) and the factor amax / 2^24 that turns the folded sums
// (which carry the 4 q of the widened nibbles) back into real values.  Also numbers the launch
// for the GEMM that follows.  Grid (ceil(G / 8), M), 256 threads: warp w of block b owns group 8 b + w.
// ------------------------------------------------------------------------------------------
// Launch counter.  A CTA that hands a partial tile over stores the current launch number in its
// flag, and the finishing CTA waits for exactly that number: whatever an earlier launch left in
// the scratch buffer (or an uninitialised buffer holds) can never be mistaken for this launch's.
__device__ int g_q8_epoch = 0;

template <int MT>
__global__ void __launch_bounds__(256)
q8_prep_kernel(const __half* __restrict__ x, int M, int K, int G, uint8_t* __restrict__ xq,
               float* __restrict__ sx, float* __restrict__ xscale, int* __restrict__ epoch) {
  constexpr int NB = Q8Cfg<MT>::NB;
  __shared__ float s_max[8];
  pdl_launch_dependents();
  pdl_wait();  // x may be the output of the kernel ahead; the scratch is read by the GEMM ahead
  const int t = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint4* row = reinterpret_cast<const uint4*>(x + (size_t)t * K);
  float amax = 0.f;
  for (int i = tid; i < K / 8; i += 256) {
    const uint4 v = __ldg(row + i);
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(h[j]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) s_max[warp] = amax;
  __syncthreads();
  amax = s_max[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, s_max[w]);
  // a non-finite row keeps inv finite: its digits are meaningless, its outputs non-finite
  const float inv = (amax > 0.f && amax < 3.0e38f) ? 4194304.f / amax : 0.f;
  if (blockIdx.x == 0 && tid == 0) {
    xscale[t] = amax * (1.f / 16777216.f);
    if (t == 0) {
      int e = atomicAdd(&g_q8_epoch, 1) + 1;
      if (e == 0) e = atomicAdd(&g_q8_epoch, 1) + 1;  // 0 is what a fresh buffer may hold
      *epoch = e;
    }
  }
  const int g = blockIdx.x * 8 + warp;
  if (g >= G) return;
  const uint2 v = __ldg(reinterpret_cast<const uint2*>(x + (size_t)t * K + (size_t)g * 128) + lane);
  const __half2* h = reinterpret_cast<const __half2*>(&v);
  const float2 f01 = __half22float2(h[0]), f23 = __half22float2(h[1]);
  const int X[4] = {__float2int_rn(f01.x * inv), __float2int_rn(f01.y * inv),
                    __float2int_rn(f23.x * inv), __float2int_rn(f23.y * inv)};
  uint32_t d[3] = {0, 0, 0};
  int sum = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int a0 = ((X[j] + 128) & 255) - 128;
    const int r1 = (X[j] - a0) >> 8;
    const int a1 = ((r1 + 128) & 255) - 128;
    const int a2 = (r1 - a1) >> 8;
    d[0] |= (uint32_t)(a0 & 255) << (8 * j);
    d[1] |= (uint32_t)(a1 & 255) << (8 * j);
    d[2] |= (uint32_t)(a2 & 255) << (8 * j);
    sum += X[j];
  }
  uint8_t* tile = xq + (size_t)g * NB * 128 + (lane >> 2) * 128 + (lane & 3) * 4;
#pragma unroll
  for (int dg = 0; dg < 3; ++dg) {
    const int n = dg * MT + t;
    *reinterpret_cast<uint32_t*>(tile + (n >> 3) * 1024 + (n & 7) * 16) = d[dg];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) sx[g * MT + t] = (float)sum;
}

// ------------------------------------------------------------------------------------------
template <int MT>
__global__ void __launch_bounds__(kQ8Threads, 1)
gemm_q8_kernel(const __grid_constant__ CUtensorMap map_w, const Q8Params p) {
  using Cfg = Q8Cfg<MT>;
  constexpr int NB = Cfg::NB, Ring = Cfg::Ring, NDB = Cfg::NDB;
  extern __shared__ uint8_t smem_raw[];
  __shared__ volatile int s_abort;
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile int s_gather[2];  // [0]: all partial tiles of a slab have been handed over

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  constexpr int kSxOff = Ring * Cfg::StageBytes;
  float* sxs = reinterpret_cast<float*>(smem + kSxOff);                       // [G][MT]
  float* red = reinterpret_cast<float*>(smem + kSxOff + Cfg::SxBytes);        // [2][MT][128]
  float* xs_s = red + 2 * MT * 128;                                           // [MT]
  const uint32_t bar_base = smem_base + kSxOff + Cfg::SxBytes + Cfg::RedBytes + 256;
  auto full = [&](int s) { return bar_base + 8 * s; };
  auto empty = [&](int s) { return bar_base + 8 * (Ring + s); };
  auto d_full = [&](int b) { return bar_base + 8 * (2 * Ring + b); };
  auto d_empty = [&](int b) { return bar_base + 8 * (2 * Ring + NDB + b); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, S = gridDim.x;
  const int G = p.G;
  const int u0 = (int)(((long long)p.tiles * c) / S);
  const int u1 = (int)(((long long)p.tiles * (c + 1)) / S);
  const int nt = u1 - u0;
  // Loads of tile i of this CTA, issued by the producer warp: lane 0 the packed weights (TMA),
  // lane 1 the activation digits of the tile's group (bulk copy).
  auto load_a = [&](int i) {
    if (lane == 0) {
      const int s = i % Ring;
      mbar_arrive_expect_tx(full(s), kQ8ATx + Cfg::BBytes);
      tma_load_2d(smem_base + s * Cfg::StageBytes, &map_w, 0, (u0 + i) * kQ8BN, full(s));
    }
  };
  auto load_b = [&](int i, int g) {
    if (lane == 1) {
      const int s = i % Ring;
      bulk_load(smem_base + s * Cfg::StageBytes + kQ8ABytes, p.xq + (size_t)g * Cfg::BBytes,
                Cfg::BBytes, full(s));
    }
  };
  pdl_launch_dependents();
  if (warp == kQ8ProducerWarp) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      s_abort = 0;
      for (int s = 0; s < Ring; ++s) {
        mbar_init(full(s), 1);
        mbar_init(empty(s), 2);  // the commits of the two issuing warps that read the stage
      }
      for (int b = 0; b < NDB; ++b) {
        mbar_init(d_full(b), 1);
        mbar_init(d_empty(b), kQ8FoldWarps / 2);
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      fence_proxy_async();
    }
    __syncwarp();
    // weights first: no kernel writes them
    for (int i = 0; i < nt && i < Ring; ++i) load_a(i);
    pdl_wait();
    for (int i = 0; i < nt && i < Ring; ++i) load_b(i, (u0 + i) % G);
  }
  __syncwarp();
  if (warp == kQ8ProducerWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;

  if (warp == kQ8ProducerWarp) {
    // ------------------------------------------------------------------ producer
    bool ok = true;
    int gb = (u0 + Ring) % G;  // group of tile i
    for (int i = Ring; i < nt && ok; ++i) {
      ok = mbar_wait(empty(i % Ring), (uint32_t)((i / Ring - 1) & 1), &s_abort, 31);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        load_a(i);
        load_b(i, gb);
      }
      if (++gb == G) gb = 0;
      __syncwarp();
    }
    // The commits of the last tiles arrive on `empty` asynchronously and nobody else waits for
    // them: see them land before the CTA may exit, or they would hit the shared memory (the
    // barriers) of whichever CTA runs on this SM next.
    for (int i = nt > Ring ? nt - Ring : 0; i < nt && ok; ++i) {
      ok = mbar_wait(empty(i % Ring), (uint32_t)((i / Ring) & 1), &s_abort, 31);
      ok = __all_sync(0xffffffffu, ok);
    }
  } else if (warp >= kQ8IssueWarp) {
    // ------------------------------------------------------------------ copies + MMAs
    // Four issuing warps: (tiles of even / odd index) x (half slab).  What bounds this stage is
    // the ~50 cycles a warp spends per tcgen05 instruction it issues, not the tensor pipe, so
    // the instructions of a tile are spread over warps.  Each warp owns 32 TMEM columns for its A
    // operand.
    // D int32, A unsigned bytes (TMEM), B signed bytes (shared memory, K-major), M = 128 weight
    // columns, N = NB digit rows, K = 32 per instruction.
    constexpr uint32_t idesc =
        (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) | (8u << 24);
    const int iw = warp - kQ8IssueWarp, par = iw >> 1, sub = iw & 1;
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
    const uint32_t ring_u = __shfl_sync(0xffffffffu, smem_base, 0);
    const uint32_t acol = tmem_u + iw * 32;
    bool ok = true;
    for (int i = par; i < nt && ok; i += 2) {
      const int s = i % Ring;
      const int j = 2 * i + sub, h = j % NDB;
      const uint32_t stage = ring_u + s * Cfg::StageBytes;
      const uint32_t a_sm = stage + sub * (kQ8ABytes / 2);
      ok = mbar_wait(full(s), (uint32_t)((i / Ring) & 1), &s_abort, 32);
      if (ok && j >= NDB) {
        ok = mbar_wait(d_empty(h), (uint32_t)((j / NDB - 1) & 1), &s_abort, 33);
      }
      if (ok && i >= par + 2) {
        // The copies below overwrite the A columns that the MMAs of this warp's previous tile
        // read.  The pipe orders a copy before a later MMA, not an MMA before a later copy, so
        // those MMAs must be seen complete first: their commit went to d_full of that tile's
        // slot (the fold warps wait on the same phase; it cannot advance again before this warp
        // issues the slot's next commit).
        const int jp = j - 4;
        ok = mbar_wait(d_full(jp % NDB), (uint32_t)((jp / NDB) & 1), &s_abort, 33);
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t dcol = tmem_u + kQ8ColD + h * NB;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)  // 32 k each: two 16-byte chunks of the 128-byte rows
          cp_128x256b_u4(acol + ks * 8, make_desc(a_sm, 16, 1024) + (uint64_t)(ks * 2));
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_i8_ts(dcol, acol + ks * 8, make_desc_k(stage + kQ8ABytes + ks * 256, 128, 1024),
                     idesc, ks ? 1u : 0u);
        umma_commit(d_full(h));  // this half slab's digit sums are complete
        umma_commit(empty(s));   // this warp's half of the stage has been read
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ fold
    const int set = warp >> 2, q = warp & 3;
    const int ftid = tid & 127;                    // thread index inside the set
    const uint32_t lane_q = (uint32_t)(q * 32) << 16;
    const int nl = 32 * q + lane;                  // column inside a 128-column half slab
    float tot[2][MT];
#pragma unroll
    for (int sub = 0; sub < 2; ++sub)
#pragma unroll
      for (int m = 0; m < MT; ++m) tot[sub][m] = 0.f;

    // Scale and zero of this thread's two columns, fetched kSzAhead of this set's tiles ahead:
    // every one is used once, so each load is a DRAM miss that queues behind the weight stream
    // (2 - 3 microseconds under load, several tile times).  The loads are volatile so that
    // they are issued here and not wherever the scheduler likes.
    constexpr int kSzAhead = 3;
    const int words = p.N / kPack;
    __half sc_q[kSzAhead][2];
    uint32_t zw_q[kSzAhead][2];
#pragma unroll
    for (int a = 0; a < kSzAhead; ++a)
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        sc_q[a][sub] = __float2half(0.f);
        zw_q[a][sub] = 0;
      }
    int l_slab = (u0 + set) / G, l_g = (u0 + set) - l_slab * G;  // next tile to fetch for
    auto fetch_sz = [&](__half (&sc)[2], uint32_t (&zw)[2]) {
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        const int n = min(l_slab * kQ8BN + sub * 128 + nl, p.N - 1);
        uint16_t sv;
        asm volatile("ld.global.nc.u16 %0, [%1];"
                     : "=h"(sv)
                     : "l"(p.scales + (size_t)l_g * p.N + n));
        sc[sub] = __ushort_as_half(sv);
        asm volatile("ld.global.nc.u32 %0, [%1];"
                     : "=r"(zw[sub])
                     : "l"(p.qzeros + (size_t)l_g * words + (n >> 3)));
      }
      l_g += 2;  // this set's next tile
      while (l_g >= G) {
        l_g -= G;
        ++l_slab;
      }
    };
#pragma unroll
    for (int a = 0; a < kSzAhead; ++a)
      if (set + 2 * a < nt) fetch_sz(sc_q[a], zw_q[a]);

    // the activation kernel's per-group sums and per-token factors
    pdl_wait();
    // (L2 loads: another CTA of the previous launch may have left older values of these
    // addresses in this SM's read-only cache)
    for (int i = tid; i < G * MT; i += 32 * kQ8FoldWarps) sxs[i] = __ldcg(p.sx + i);
    if (tid < MT) xs_s[tid] = __ldcg(p.xscale + tid);
    const int epoch = __ldcg(p.epoch);
    named_sync(1, 32 * kQ8FoldWarps);

    bool ok = true;
    int seg = 0, g_first = u0 % G;
    int slab = u0 / G, g = u0 - slab * G;
    for (int i = 0; i < nt; ++i, ++g) {
      if (g == G) {
        g = 0;
        ++slab;
      }
      if ((i & 1) == set && ok) {
        const float s0 = __half2float(sc_q[0][0]), s1 = __half2float(sc_q[0][1]);
        // the widened nibbles are 4 q, so the zero point enters as 4 z (columns past N of a last
        // slab use the last column's values; nothing of them is stored)
        const int n0 = min(slab * kQ8BN + nl, p.N - 1), n1 = min(slab * kQ8BN + 128 + nl, p.N - 1);
        const float z0 = 4.f * (float)nibble_of_col(zw_q[0][0], n0 & 7);
        const float z1 = 4.f * (float)nibble_of_col(zw_q[0][1], n1 & 7);
#pragma unroll
        for (int a = 0; a + 1 < kSzAhead; ++a)
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
            sc_q[a][sub] = sc_q[a + 1][sub];
            zw_q[a][sub] = zw_q[a + 1][sub];
          }
        if (i + 2 * kSzAhead < nt) fetch_sz(sc_q[kSzAhead - 1], zw_q[kSzAhead - 1]);
        const float* sxg = sxs + g * MT;
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
          const int j = 2 * i + sub, h = j % NDB;
          if (ok) {
            ok = mbar_wait(d_full(h), (uint32_t)((j / NDB) & 1), &s_abort, 34);
          }
          // every lane polled on its own: bring the warp back together (the TMEM loads below are
          // warp-wide instructions) and make the outcome uniform
          ok = __all_sync(0xffffffffu, ok);
          if (ok) {
            tc_fence_after();
            const uint32_t dcol = tmem + lane_q + kQ8ColD + h * NB;
            uint32_t a0[MT], a1[MT], a2[MT];
            tmem_ld_n<MT>(dcol, a0);
            tmem_ld_n<MT>(dcol + MT, a1);
            tmem_ld_n<MT>(dcol + 2 * MT, a2);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            // the sums are in registers: the slot can take the next half slab
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(d_empty(h));
            const float sc = sub ? s1 : s0, zz = sub ? z1 : z0;
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              const float lo = (float)((int)a1[m] * 256 + (int)a0[m]);
              const float v = fmaf(65536.f, (float)(int)a2[m], lo);
              tot[sub][m] = fmaf(sc, fmaf(-zz, sxg[m], v), tot[sub][m]);
            }
          }
        }
      }
      if (g != G - 1 && i != nt - 1) continue;
      // ---- end of this CTA's share of a slab: the two sets' sums meet in set 0.  Every fold
      //      thread passes here whatever happened to its waits, so the named barriers always
      //      see their full count. ----
      if (set == 1) {
        if (seg > 0) named_sync(3, 32 * kQ8FoldWarps);  // set 0 has read the previous segment
#pragma unroll
        for (int sub = 0; sub < 2; ++sub)
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            red[(sub * MT + m) * 128 + nl] = tot[sub][m];
            tot[sub][m] = 0.f;
          }
        named_sync(2, 32 * kQ8FoldWarps);
      } else {
        named_sync(2, 32 * kQ8FoldWarps);
#pragma unroll
        for (int sub = 0; sub < 2; ++sub)
#pragma unroll
          for (int m = 0; m < MT; ++m) tot[sub][m] += red[(sub * MT + m) * 128 + nl];
        if (i != nt - 1) named_arrive(3, 32 * kQ8FoldWarps);
        if (g_first != 0) {
          // not the CTA that holds the slab's first group: hand the partial sums over
          float* dst = p.partial + (size_t)c * (2 * MT * 128);
#pragma unroll
          for (int sub = 0; sub < 2; ++sub)
#pragma unroll
            for (int m = 0; m < MT; ++m) dst[(sub * MT + m) * 128 + nl] = tot[sub][m];
          // the barrier orders the 128 threads' stores before thread 0, whose release store (it
          // is cumulative) then publishes them together with the flag
          named_sync(4, 128);
          if (ftid == 0 && !s_abort) {
            __threadfence();
            st_release(p.flags + c, epoch);
          }
        } else {
          bool complete = true;
          if (g != G - 1) {
            // The slab continues in the following CTAs, which processed their share first.  One
            // thread sees all their flags raised, then every thread adds the partial tiles in
            // CTA order, the loads of the next one in flight while the current one is added.
            const int u_last = slab * G + G - 1;
            int c_end = c + 1;
            while (c_end < S && (int)(((long long)p.tiles * c_end) / S) <= u_last) ++c_end;
            if (ftid == 0) {
              bool got = true;
              uint32_t n = 0;
              for (int cc = c + 1; cc < c_end && got; ++cc)
                while (ld_acquire(p.flags + cc) != epoch) {
                  if (++n >= p.spin_limit || s_abort) {
                    s_abort = 1;
                    atomicCAS(&g_tc_status, 0, 35);
                    got = false;
                    break;
                  }
                }
              s_gather[0] = got ? 1 : 0;
            }
            named_sync(4, 128);
            complete = s_gather[0] != 0;  // the same value in all 128 threads
            if (complete) {
              float nxt[2][MT];
              auto fetch = [&](int cc) {
                const float* src = p.partial + (size_t)cc * (2 * MT * 128);
#pragma unroll
                for (int sub = 0; sub < 2; ++sub)
#pragma unroll
                  for (int m = 0; m < MT; ++m) nxt[sub][m] = __ldcg(src + (sub * MT + m) * 128 + nl);
              };
              fetch(c + 1);
              for (int cc = c + 1; cc < c_end; ++cc) {
                float cur[2][MT];
#pragma unroll
                for (int sub = 0; sub < 2; ++sub)
#pragma unroll
                  for (int m = 0; m < MT; ++m) cur[sub][m] = nxt[sub][m];
                if (cc + 1 < c_end) fetch(cc + 1);
#pragma unroll
                for (int sub = 0; sub < 2; ++sub)
#pragma unroll
                  for (int m = 0; m < MT; ++m) tot[sub][m] += cur[sub][m];
              }
            }
          }
          if (complete && !s_abort) {
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
              const int n = slab * kQ8BN + sub * 128 + nl;
              if (n < p.N) {
                const float bv = p.bias != nullptr ? __half2float(__ldg(p.bias + n)) : 0.f;
#pragma unroll
                for (int m = 0; m < MT; ++m)
                  if (m < p.M)
                    p.out[(size_t)m * p.N + n] = __float2half_rn(fmaf(tot[sub][m], xs_s[m], bv));
              }
            }
          }
        }
#pragma unroll
        for (int sub = 0; sub < 2; ++sub)
#pragma unroll
          for (int m = 0; m < MT; ++m) tot[sub][m] = 0.f;
      }
      ++seg;
      g_first = 0;
    }
  }

  // ---- teardown ----
  __syncwarp();
  if (s_abort) {
    // a wait gave up: copies and MMAs may still be in flight towards this CTA's shared and
    // tensor memory.  Let them land (a millisecond) before both are given back.
    const long long t_end = clock64() + 2000000;
    while (clock64() < t_end) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kQ8ProducerWarp) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u)
                 : "memory");
  }
}

// Load-time repack: AWQ words [K][N/8] -> K-major nibbles, tile (slab, group) = 256 rows of 64 B
// (row r = column 256 slab + r, byte b = k 2b | k 2b+1 << 4 of the group).  One thread writes one
// 32-bit word (8 consecutive k of one column).  Columns past N are zero.
__global__ void __launch_bounds__(256)
repack_kmajor_kernel(const uint32_t* __restrict__ qweight, uint32_t* __restrict__ out, int K, int N,
                     long long total_words) {
  const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
  if (idx >= total_words) return;
  const int G = K / kQ8BK;
  const int w = (int)(idx & 15);            // word of the row: k 8 w .. 8 w + 7
  const long long rowi = idx >> 4;
  const int r = (int)(rowi & 255);
  const long long tile = rowi >> 8;
  const int g = (int)(tile % G);
  const int slab = (int)(tile / G);
  const int n = slab * kQ8BN + r;
  uint32_t o = 0;
  if (n < N) {
    const int words = N / kPack;
    const uint32_t* src = qweight + (size_t)(g * kQ8BK + 8 * w) * words + (n >> 3);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      o |= (uint32_t)nibble_of_col(__ldg(src + (size_t)j * words), n & 7) << (4 * j);
  }
  out[idx] = o;
}

struct Q8Scratch {
  uint8_t* xq;
  float* sx;
  float* xscale;
  int* epoch;
  int* flags;
  float* partial;
  size_t bytes;
};

template <int MT>
Q8Scratch q8_scratch(void* base, int G, int grid) {
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  Q8Scratch s;
  size_t off = 0;
  uint8_t* b = static_cast<uint8_t*>(base);
  s.xq = b + off;
  off = up(off + (size_t)G * Q8Cfg<MT>::BBytes);
  s.sx = reinterpret_cast<float*>(b + off);
  off = up(off + (size_t)G * MT * 4);
  s.xscale = reinterpret_cast<float*>(b + off);
  off = up(off + MT * 4);
  s.epoch = reinterpret_cast<int*>(b + off);
  off = up(off + 4);
  s.flags = reinterpret_cast<int*>(b + off);
  off = up(off + (size_t)kQ8MaxGrid * 4);
  s.partial = reinterpret_cast<float*>(b + off);
  off = up(off + (size_t)grid * 2 * MT * 128 * 4);
  s.bytes = off;
  return s;
}

uint32_t g_q8_spin_limit = kSpinLimit;

template <int MT>
int launch_q8(const __half* x, const void* qweight_km, const __half* scales, const uint32_t* qzeros,
              const __half* bias, __half* out, int M, int N, int K, void* workspace,
              size_t workspace_bytes, cudaStream_t stream) {
  using Cfg = Q8Cfg<MT>;
  static std::atomic<bool> attr_done[64];  // zero-initialised; setting the attribute twice is harmless
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return AWQ_B200_ERR_DEVICE;
  auto kernel = gemm_q8_kernel<MT>;
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::SmemBytes) != cudaSuccess)
      return AWQ_B200_ERR_LAUNCH;
    attr_done[dev] = true;
  }
  const int G = K / kQ8BK;
  const int slabs = (N + kQ8BN - 1) / kQ8BN;
  const int tiles = slabs * G;
  int grid = sm_count();
  if (grid > kQ8MaxGrid) grid = kQ8MaxGrid;
  if (grid > tiles) grid = tiles;
  const Q8Scratch ws = q8_scratch<MT>(workspace, G, grid);
  if (workspace == nullptr || workspace_bytes < ws.bytes) return AWQ_B200_ERR_WORKSPACE;

  CUtensorMap map_w;
  {
    // packed nibbles [tiles * 256 rows][128 nibbles], box = one tile
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return AWQ_B200_ERR_DRIVER;
    const cuuint64_t dims[2] = {128, (cuuint64_t)tiles * kQ8BN};
    const cuuint64_t strides[1] = {64};
    const cuuint32_t box[2] = {128, kQ8BN};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<void*>(qweight_km), dims,
            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return AWQ_B200_ERR_DRIVER;
  }
  if (launch_pdl(q8_prep_kernel<MT>, dim3((G + 7) / 8, M), dim3(256), 0, stream, x, M, K, G, ws.xq,
                 ws.sx, ws.xscale, ws.epoch) != cudaSuccess) {
    cudaGetLastError();
    return AWQ_B200_ERR_LAUNCH;
  }
  Q8Params p{ws.xq,
             scales,
             qzeros,
             bias,
             out,
             ws.sx,
             ws.xscale,
             ws.partial,
             ws.flags,
             ws.epoch,
             M,
             N,
             K,
             G,
             tiles,
             g_q8_spin_limit};
  if (launch_pdl(kernel, dim3(grid), dim3(kQ8Threads), Cfg::SmemBytes, stream, map_w, p) !=
      cudaSuccess) {
    cudaGetLastError();
    return AWQ_B200_ERR_LAUNCH;
  }
  return AWQ_B200_OK;
}

}  // namespace

bool gemm_q8_supported(int M, int N, int K, int group) {
  return M >= 1 && M <= 16 && N % kPack == 0 && K % kQ8BK == 0 && K / kQ8BK <= kQ8MaxGroups &&
         group == 128;
}

size_t repack_kmajor_bytes(int K, int N) {
  const size_t slabs = (size_t)(N + kQ8BN - 1) / kQ8BN;
  return slabs * (size_t)(K / kQ8BK) * kQ8ATx;
}

int launch_repack_kmajor(const uint32_t* qweight, void* out, int K, int N, cudaStream_t stream) {
  const long long total_words = (long long)(repack_kmajor_bytes(K, N) / 4);
  if (total_words == 0) return AWQ_B200_OK;
  repack_kmajor_kernel<<<(unsigned)((total_words + 255) / 256), 256, 0, stream>>>(
      qweight, static_cast<uint32_t*>(out), K, N, total_words);
  return cudaGetLastError() == cudaSuccess ? AWQ_B200_OK : AWQ_B200_ERR_LAUNCH;
}

size_t gemm_q8_workspace_bytes(int M, int N, int K, int group) {
  if (!gemm_q8_supported(M, N, K, group)) return 0;
  const int G = K / kQ8BK;
  if (M <= 8) return q8_scratch<8>(nullptr, G, kQ8MaxGrid).bytes;
  return q8_scratch<16>(nullptr, G, kQ8MaxGrid).bytes;
}

int launch_gemm_q8(const __half* x, const void* qweight_km, const __half* scales,
                   const uint32_t* qzeros, const __half* bias, __half* out, int M, int N, int K,
                   int group, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (!gemm_q8_supported(M, N, K, group)) return AWQ_B200_ERR_SHAPE;
  if (M <= 8)
    return launch_q8<8>(x, qweight_km, scales, qzeros, bias, out, M, N, K, workspace,
                        workspace_bytes, stream);
  return launch_q8<16>(x, qweight_km, scales, qzeros, bias, out, M, N, K, workspace,
                       workspace_bytes, stream);
}



// Exercise of the give-up path of the bounded waits: one warp waits on an mbarrier nobody arrives
// on (the same helper every kernel uses, with a short limit), then on a flag in global memory
// nobody sets (the wait of the stream-K finisher).  Both run out, the first one records code 90
// in the status word, the kernel returns normally.
__device__ int g_q8_never_set = 0;

__global__ void __launch_bounds__(32) wait_selftest_kernel(uint32_t polls) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ volatile int s_abort;
  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  const bool ok = mbar_wait_n(smem_u32(&bar), 0, &s_abort, 90, polls);
  if (threadIdx.x == 0 && !ok) {
    uint32_t n = 0;
    while (ld_acquire(&g_q8_never_set) == 0)
      if (++n >= polls) {
        atomicCAS(&g_tc_status, 0, 91);
        break;
      }
  }
}

int launch_wait_selftest(uint32_t polls, cudaStream_t stream) {
  wait_selftest_kernel<<<1, 32, 0, stream>>>(polls ? polls : 1);
  return cudaGetLastError() == cudaSuccess ? AWQ_B200_OK : AWQ_B200_ERR_LAUNCH;
}

void q8_set_spin_limit(uint32_t polls) { g_q8_spin_limit = polls ? polls : kSpinLimit; }

int q8_device_status(int* out, int clear) { return read_tc_status(out, clear); }

}  // namespace awq
