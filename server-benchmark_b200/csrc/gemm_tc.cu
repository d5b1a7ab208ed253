// Large-M AWQ GEMM on the 5th-generation tensor cores (tcgen05 / TMEM), weights dequantised in
// shared memory.
//
//   y[M, N] = x[M, K] @ ((q - z) * s)
//
// CTA tile: (128 * MT) tokens x BN columns (MT = 1 or 2, BN = 256 or 128), K walked in stages of
// 64 rows.  Per stage
//   D_mt (TMEM, fp32, 128 lanes x BN columns) += A_mt (smem) * B (smem)    tcgen05.mma kind::f16
//     A_mt = x tile [128 x 64] fp16, K-major, 128-byte swizzle, written by TMA.
//     B    = W tile [64 x BN] fp16, MN-major (columns contiguous, as the AWQ packing delivers
//            them), 128-byte swizzle: per block of 64 columns a [64 rows x 128 B] region, 16-byte
//            chunk c of row k stored at c ^ (k & 7).  Written by the dequantisation warps; with
//            MT = 2 one dequantised tile feeds two MMAs, halving the conversion work per flop.
//   The packed weights [64 x BN/8 words] arrive by TMA (no swizzle) next to A.
//
// Warp roles (608 threads):
//   warps 0-15 dequantise (two teams of 8 warps on alternate stages): one packed word -> 8 fp16
//              -> one 16-byte store; afterwards the epilogue: tcgen05.ld of their TMEM lane
//              quarter, fp16 conversion, global stores.
//   warp 16    TMA producer of the packed weights (one elected lane), own ring of 4-8 slots.
//   warp 17    TMEM allocation; one elected lane issues tcgen05.mma and tcgen05.commit.
//   warp 18    TMA producer of the x tiles (one elected lane).
// Barriers: raw_full / raw_empty per packed-weight slot; per x+B slot one `full` barrier (the
// conversion threads' arrivals plus the x tile's TMA byte count) and one `empty` barrier
// (tcgen05.commit), so the MMA thread waits once and commits once per stage -- tcgen05.mma issue is
// paced by execution, and whatever else that thread does is a bubble in the tensor pipe.  A
// packed-weight slot is released only after its words have been consumed by the conversion (an
// issued shared-memory load is not yet a performed one).  tmem_full hands the accumulators to
// the epilogue.
//
// Split-K (MT = 1 only): the Z CTAs of a thread-block cluster take consecutive K ranges of the
// same tile; their fp32 accumulators are spilled to shared memory and summed through
// distributed shared memory in rank order (deterministic, no global scratch).
//
// Every wait is bounded: after kSpinLimit polls a thread records a status code in
// g_tc_status, raises the CTA's abort flag, and all roles fall through to the teardown, where
// TMEM is freed.  Nothing here uses cluster multicast.
#include <cooperative_groups.h>
#include "tc_ptx.cuh"

namespace cg = cooperative_groups;

namespace awq {

namespace {

using namespace tc;

constexpr int kBM = 128;
constexpr int kBKtc = 64;
constexpr int kDqWarps = 16;
constexpr int kDqThreads = kDqWarps * 32;
// The conversion warps form two teams that take alternate stages, so that one team's barrier
// waits and dependency chains overlap with the other team's work.
constexpr int kTeams = 2;
constexpr int kTeamThreads = kDqThreads / kTeams;
constexpr int kTcThreads = kDqThreads + 96;  // + raw producer, MMA issuer, A producer warps

// Three rings with their own depths, because their producers have very different latencies:
//   raw  packed weights from HBM (8 KB / stage)  -> deep, to keep enough bytes in flight
//   A    x tiles, mostly L2 hits (16 KB per 128 rows / stage)
//   B    dequantised tile handed from the conversion warps to the MMA (double buffer)
template <int BN, int MT>
struct TcCfg {
  static constexpr int kABytes = MT * kBM * kBKtc * 2;        // 16384 per 128-row tile
  static constexpr int kBBytes = kBKtc * BN * 2;              // 32768 / 16384
  static constexpr int kRawBytes = kBKtc * (BN / kPack) * 4;  // 8192 / 4096
  // The hand-off latencies (conversion of a stage, MMA, commit -> barrier -> wake-up) add up to
  // about three stage times, so the B ring must hold 3-4 stages for the tensor core to stay busy.
  // x tile and dequantised tile of a stage share one full / one empty barrier, so the MMA
  // thread waits once and commits once per stage; the packed weights have their own deeper ring.
  static constexpr int kNA = BN == 128 ? 5 : (MT == 2 ? 3 : 4);
  static constexpr int kNB = kNA;
  static constexpr int kNR = BN == 128 ? 8 : (MT == 2 ? 4 : 4);
  static constexpr int kAOff = 0;
  static constexpr int kBOff = kNA * kABytes;
  static constexpr int kRawOff = kBOff + kNB * kBBytes;
  static constexpr int kPipeBytes = kRawOff + kNR * kRawBytes;
  static constexpr int kBarBytes = 512;
  static constexpr int kRedPitch = BN + 4;  // floats, split-K spill tile
  static constexpr int kRedBytes = kBM * kRedPitch * 4;
  static constexpr int kMainBytes = kPipeBytes > kRedBytes ? kPipeBytes : kRedBytes;
  static constexpr int kSmemBytes = kMainBytes + kBarBytes + 1024;  // + alignment slack
  static constexpr int kTmemCols = BN * MT;
};

struct TcParams {
  const __half* scales;
  const uint32_t* qzeros;
  const __half* bias;
  __half* out;
  int M, N, K, group;
  // grouped (MoE) modes only
  const float* topk_weights;   // [T * topk]
  const int32_t* sorted_ids;   // permuted (token, slot) list, padded to 128 per expert
  const int32_t* expert_ids;   // expert of every 128-row block
  const int32_t* num_post_pad;
  int numel;                   // T * topk
  int half_cols;               // gate_up: I (column offset of the up half)
};

// MODE 0: dense linear  y[M, N] = x @ W (+ bias).
// MODE 1: grouped gate_up of a fused-MoE layer: row block b of the permuted list belongs to expert
//         expert_ids[b]; the tile's 256 columns are 128 gate columns and the matching 128 up
//         columns; epilogue silu(gate) * up -> act[pos] (N = 2I per expert).
// MODE 2: grouped down projection: epilogue times routed weight -> pair_out[flat pair id].
template <int BN, int MT, int MODE>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               const TcParams p) {
  using C = TcCfg<BN, MT>;
  constexpr int NA = C::kNA, NB = C::kNB, NR = C::kNR;
  // the packed weights of a tile arrive as BN / 128 boxes of [64 rows x 16 words]
  constexpr int HALVES = BN / 128;
  constexpr int HALF_THREADS = kTeamThreads / HALVES;  // team threads converting one box
  constexpr int KSTEP = HALF_THREADS / 16;    // rows covered per pass
  constexpr int PASSES = kBKtc / KSTEP;
  static_assert(MODE == 0 || (BN == 256 && MT == 1), "grouped modes use 128 x 256 tiles");
  extern __shared__ uint8_t smem_raw[];
  __shared__ volatile int s_abort;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_fid[MODE == 2 ? kBM : 1];

  cg::cluster_group cluster = cg::this_cluster();
  const int zrank = (int)cluster.block_rank();
  const int Z = (int)cluster.num_blocks();

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + C::kMainBytes;
  auto a_addr = [&](int s) { return smem_base + C::kAOff + s * C::kABytes; };
  auto b_addr = [&](int s) { return smem_base + C::kBOff + s * C::kBBytes; };
  auto raw_addr = [&](int s) { return smem_base + C::kRawOff + s * C::kRawBytes; };
  auto raw_full = [&](int s) { return bar_base + 8 * s; };
  auto raw_empty = [&](int s) { return bar_base + 8 * (NR + s); };
  // full[s]: kTeamThreads arrivals (B tile written) + 1 arrival with the x tile's byte count
  auto full = [&](int s) { return bar_base + 8 * (2 * NR + s); };
  auto empty = [&](int s) { return bar_base + 8 * (2 * NR + NA + s); };
  const uint32_t tmem_full = bar_base + 8 * (2 * NR + 2 * NA);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int words = p.N / kPack;  // packed words per weight row (of one expert)
  int m0, n0, w_left, w_right, wrow0 = 0;
  const __half* scales = p.scales;
  const uint32_t* qzeros = p.qzeros;
  if (MODE == 0) {
    m0 = blockIdx.x * (kBM * MT);
    n0 = blockIdx.y * BN;
    w_left = n0 / kPack;
    w_right = w_left + 16;
  } else {
    m0 = blockIdx.x * kBM;  // position in the permuted list
    // uniform over the CTA and before anything is allocated: unused blocks leave at once
    if (m0 >= p.num_post_pad[0]) return;
    const int e = p.expert_ids[blockIdx.x];
    if (e < 0) return;
    if (MODE == 1) {
      n0 = blockIdx.y * 128;  // activation column of the tile
      w_left = blockIdx.y * 16;
      w_right = p.half_cols / kPack + blockIdx.y * 16;
    } else {
      n0 = blockIdx.y * BN;
      w_left = n0 / kPack;
      w_right = w_left + 16;
    }
    wrow0 = e * p.K;
    const size_t groups = (size_t)(p.K / p.group);
    scales += (size_t)e * groups * p.N;
    qzeros += (size_t)e * groups * words;
  }
  const int KT_all = p.K / kBKtc;
  const int kt_begin = (int)(((long long)zrank * KT_all) / Z);
  const int kt_end = (int)(((long long)(zrank + 1) * KT_all) / Z);
  const int KT = kt_end - kt_begin;

  if (MODE == 2 && tid < kBM) s_fid[tid] = p.sorted_ids[m0 + tid];
  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < NR; ++s) {
      mbar_init(raw_full(s), 1);
      mbar_init(raw_empty(s), kTeamThreads);
    }
    for (int s = 0; s < NA; ++s) {
      mbar_init(full(s), kTeamThreads + 1);
      mbar_init(empty(s), 1);
    }
    mbar_init(tmem_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  if (warp == kDqWarps + 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "r"((uint32_t)C::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = s_tmem_base;
  bool ok = true;

  if (warp == kDqWarps) {
    // ------------------------------------------------------------------ packed-weight producer
    if (lane == 0) {
      for (int it = 0; it < KT; ++it) {
        const int s = it % NR;
        const uint32_t round = (uint32_t)(it / NR);
        if (!mbar_wait(raw_empty(s), (round & 1u) ^ 1u, &s_abort, 1)) break;
        mbar_arrive_expect_tx(raw_full(s), C::kRawBytes);
        const int krow = wrow0 + (kt_begin + it) * kBKtc;
        tma_load_2d(raw_addr(s), &map_w, w_left, krow, raw_full(s));
        if (HALVES == 2) tma_load_2d(raw_addr(s) + 4096, &map_w, w_right, krow, raw_full(s));
      }
    }
  } else if (warp == kDqWarps + 2) {
    // ------------------------------------------------------------------ activation producer
    if (lane == 0) {
      for (int it = 0; it < KT; ++it) {
        const int s = it % NA;
        const uint32_t round = (uint32_t)(it / NA);
        if (!mbar_wait(empty(s), (round & 1u) ^ 1u, &s_abort, 6)) break;
        const int k0 = (kt_begin + it) * kBKtc;
        mbar_arrive_expect_tx(full(s), C::kABytes);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          tma_load_2d(a_addr(s) + mt * (kBM * kBKtc * 2), &map_x, k0, m0 + mt * kBM, full(s));
      }
    }
  } else if (warp == kDqWarps + 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs the loop and stays converged; one elected lane issues.  (A lane that
    // loops alone while the rest of its warp is parked pays several times more per tcgen05
    // instruction, see elect_one in tc_ptx.cuh.)
    {
      // instruction descriptor: D fp32, A/B fp16, A K-major, B MN-major, N = BN, M = 128
      constexpr uint32_t idesc = (1u << 4) | (1u << 16) | ((uint32_t)(BN >> 3) << 17) |
                                 ((uint32_t)(kBM >> 4) << 24);
      // tcgen05 operands live in uniform registers: derive them from warp-uniform values only
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_d, 0);
      // descriptors of every ring slot, built once
      uint64_t da[NA][MT], db[NA];
#pragma unroll
      for (int s = 0; s < NA; ++s) {
        // A: K-major SW128, 8-row core blocks 1024 B apart; B: MN-major SW128, 64-column
        // blocks 8192 B apart (LBO), 8-row k blocks 1024 B apart (SBO).
        db[s] = make_desc(__shfl_sync(0xffffffffu, b_addr(s), 0), 8192, 1024);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          da[s][mt] = make_desc(
              __shfl_sync(0xffffffffu, a_addr(s) + mt * (kBM * kBKtc * 2), 0), 16, 1024);
      }
      // The tensor pipe runs one MMA after the other, so whatever else this warp does between
      // two of them is a bubble.  The wait for the next stage is therefore done before the last
      // MMA of the current one is issued (it then overlaps with a running MMA).
      int s = 0;
      uint32_t phase = 0;
      ok = KT == 0 || mbar_wait(full(0), 0, &s_abort, 2);
      ok = __all_sync(0xffffffffu, ok);
      for (int it = 0; it < KT && ok; ++it) {
        tc_fence_after();
        int sn = s + 1;
        uint32_t phase_n = phase;
        if (sn == NA) { sn = 0; phase_n ^= 1u; }
        constexpr int kLast = MT * (kBKtc / 16) - 1;
        auto issue = [&](int first, int last) {  // MMAs [first, last] of the stage
#pragma unroll
          for (int ss = 0; ss < NA; ++ss) {
            if (ss != s) continue;  // compile-time slot index keeps the descriptors in registers
#pragma unroll
            for (int i = 0; i <= kLast; ++i) {
              if (i < first || i > last) continue;
              const int mt = i / (kBKtc / 16), k16 = i % (kBKtc / 16);
              // advance 16 k: +32 B inside A's 128-byte rows, +16 rows (2048 B) in B
              umma_f16_ss(tmem_u + mt * BN, da[ss][mt] + (uint64_t)((k16 * 32) >> 4),
                          db[ss] + (uint64_t)((k16 * 2048) >> 4), idesc,
                          (it > 0 || k16 > 0) ? 1u : 0u);
            }
          }
        };
        if (elect_one()) issue(0, kLast - 1);
        __syncwarp();
        if (it + 1 < KT) {
          ok = mbar_wait(full(sn), phase_n, &s_abort, 2);
          ok = __all_sync(0xffffffffu, ok);
        }
        if (elect_one()) {
          issue(kLast, kLast);
          umma_commit(empty(s));
        }
        __syncwarp();
        s = sn;
        phase = phase_n;
      }
      if (ok && elect_one()) umma_commit(tmem_full);
      __syncwarp();
    }
  } else if (warp < kDqWarps) {
    // ------------------------------------------------------------------ dequant warps
    const int team = tid / kTeamThreads, tt = tid % kTeamThreads;
    // inside a team: threads [0, HALF_THREADS) convert the left box, the rest the right box
    const int half = tt / HALF_THREADS, th = tt % HALF_THREADS;
    const int c16 = th & 15, krow0 = th >> 4;
    const int c = half * 16 + c16;      // packed word column inside the tile
    const int wcol = min((half ? w_right : w_left) + c16, words - 1);  // clamped past the N edge
    // KSTEP is a multiple of 8, so (k & 7) is the same for every row this thread converts
    const uint32_t b_off = (uint32_t)(c / 8) * (kBKtc * 128) + krow0 * 128 +
                           (((uint32_t)(c & 7) ^ (uint32_t)(krow0 & 7)) << 4);
    const uint32_t raw_off = (uint32_t)half * 4096 + (uint32_t)(krow0 * 16 + c16) * 4;
    constexpr int kPrefetchGroups = 3;
    int cur_group = -1;
    __half2 zE0, zO0, zE1, zO1, sE0, sO0, sE1, sO1;
    // scales / zeros are fetched one group ahead so that their L2 latency hides behind a group
    const int ngroups = p.K / p.group;
    const int g_first = min(((kt_begin + team) * kBKtc) / p.group, ngroups - 1);
    uint32_t zw_n = __ldg(qzeros + (size_t)g_first * words + wcol);
    uint4 sv_n = __ldg(reinterpret_cast<const uint4*>(scales + (size_t)g_first * p.N) + wcol);
    for (int it = team; it < KT && ok; it += kTeams) {
      const int sr = it % NR, sb = it % NA;
      const int grp = ((kt_begin + it) * kBKtc) / p.group;
      if (grp != cur_group) {
        cur_group = grp;
        const uint32_t zw = zw_n;
        const uint4 sv = sv_n;
        // prefetch for the next stage of this team that lies in a different group
        int itn = it + kTeams;
        while (itn < KT && ((kt_begin + itn) * kBKtc) / p.group == grp) itn += kTeams;
        const int gn = min(((kt_begin + itn) * kBKtc) / p.group, ngroups - 1);
        // Under the weight stream an L2 miss on these small rows was measured at more than one
        // team iteration (~2800 cycles): pull the rows of a few groups further on into L2 now,
        // so that the register prefetch above only ever waits for an L2 hit.
        if (krow0 == 0) {
          const int gp = min(gn + kPrefetchGroups, ngroups - 1);
          asm volatile("prefetch.global.L2 [%0];" ::"l"(qzeros + (size_t)gp * words + wcol));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(
              reinterpret_cast<const uint4*>(scales + (size_t)gp * p.N) + wcol));
        }
        zw_n = __ldg(qzeros + (size_t)gn * words + wcol);
        sv_n = __ldg(reinterpret_cast<const uint4*>(scales + (size_t)gn * p.N) + wcol);
        const uint32_t zw8 = zw >> 8;
        zE0 = as_half2(lop3_and_or(zw, 0x000F000Fu, 0x64006400u));   // 1024 + z, cols 0,1
        zO0 = as_half2(lop3_and_or(zw, 0x00F000F0u, 0x64006400u));   // 1024 + 16 z, cols 2,3
        zE1 = as_half2(lop3_and_or(zw8, 0x000F000Fu, 0x64006400u));  // cols 4,5
        zO1 = as_half2(lop3_and_or(zw8, 0x00F000F0u, 0x64006400u));  // cols 6,7
        const __half2 r16 = __float2half2_rn(0.0625f);
        sE0 = as_half2(sv.x);
        sO0 = __hmul2(as_half2(sv.y), r16);  // nibbles kept in place carry a factor 16
        sE1 = as_half2(sv.z);
        sO1 = __hmul2(as_half2(sv.w), r16);
      }
      ok = mbar_wait(raw_full(sr), (uint32_t)((it / NR) & 1), &s_abort, 4);
      if (!ok) break;
      const uint32_t raw = raw_addr(sr) + raw_off, bt = b_addr(sb) + b_off;
      uint32_t w[PASSES];
#pragma unroll
      for (int j = 0; j < PASSES; ++j)
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w[j]) : "r"(raw + j * (KSTEP * 16 * 4)));
      // the B slot was last read by the MMAs of stage it - NB
      ok = mbar_wait(empty(sb), (uint32_t)(((it / NA) & 1) ^ 1), &s_abort, 7);
      if (!ok) break;
#pragma unroll
      for (int j = 0; j < PASSES; ++j) {
        const uint32_t w8 = w[j] >> 8;
        uint4 o;
        o.x = as_u32(__hmul2(__hsub2(as_half2(lop3_and_or(w[j], 0x000F000Fu, 0x64006400u)), zE0), sE0));
        o.y = as_u32(__hmul2(__hsub2(as_half2(lop3_and_or(w[j], 0x00F000F0u, 0x64006400u)), zO0), sO0));
        o.z = as_u32(__hmul2(__hsub2(as_half2(lop3_and_or(w8, 0x000F000Fu, 0x64006400u)), zE1), sE1));
        o.w = as_u32(__hmul2(__hsub2(as_half2(lop3_and_or(w8, 0x00F000F0u, 0x64006400u)), zO1), sO1));
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(bt + j * (KSTEP * 128)),
                     "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w)
                     : "memory");
      }
      mbar_arrive(raw_empty(sr));  // every packed word of the slot has been consumed
      fence_proxy_async();  // generic-proxy stores -> visible to the tensor core's async proxy
      mbar_arrive(full(sb));
    }

    // ---------------------------------------------------------------- epilogue
    // warp w reads TMEM lanes 32 (w % 4) ..; with MT = 2 warps 4-7 own the second accumulator,
    // with MT = 1 they own the upper half of the columns.
    // sixteen warps: four per lane quarter, each taking a quarter of that quarter's columns
    constexpr int kSlices = kDqWarps / 4;  // warps per lane quarter
    const int q = warp & 3, hi = warp >> 2;
    const int acc = MT == 2 ? hi / (kSlices / 2) : 0;
    const int cols_per = MT == 2 ? BN / (kSlices / 2) : BN / kSlices;
    const int col_begin = (MT == 2 ? hi % (kSlices / 2) : hi) * cols_per;
    const int col_end = col_begin + cols_per;
    const uint32_t tlane = tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
    if (KT > 0) ok = ok && mbar_wait(tmem_full, 0, &s_abort, 5);
    if (ok && MODE == 1) {
      // act[pos, n0 + c] = silu(D[c]) * D[128 + c]; warp slice hi owns 32 of the 128 columns
      tc_fence_after();
      const int row = q * 32 + lane;
      const int c0 = hi * 32;
      uint32_t g[32], u[32];
      tmem_ld32(tlane + (uint32_t)c0, g);
      tmem_ld32(tlane + (uint32_t)(128 + c0), u);
      if (n0 + c0 < p.half_cols) {
        __align__(16) __half2 h[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
          h[j] = __floats2half2_rn(g0 / (1.f + __expf(-g0)) * __uint_as_float(u[2 * j]),
                                   g1 / (1.f + __expf(-g1)) * __uint_as_float(u[2 * j + 1]));
        }
        uint4* dst =
            reinterpret_cast<uint4*>(p.out + (size_t)(m0 + row) * p.half_cols + n0 + c0);
        const uint4* srcv = reinterpret_cast<const uint4*>(h);
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[j] = srcv[j];
      }
    } else if (ok && MODE == 2) {
      // pair_out[fid, n0 + c] = routed weight * D[c]; warp slice hi owns 64 of the 256 columns
      tc_fence_after();
      const int fid = s_fid[q * 32 + lane];
      const bool valid = fid < p.numel;
      const float rw = valid ? __ldg(p.topk_weights + fid) : 0.f;
#pragma unroll 1
      for (int c0 = hi * 64; c0 < hi * 64 + 64; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tlane + (uint32_t)c0, r);
        if (valid && n0 + c0 < p.N) {
          __align__(16) __half2 h[16];
#pragma unroll
          for (int j = 0; j < 16; ++j)
            h[j] = __floats2half2_rn(__uint_as_float(r[2 * j]) * rw,
                                     __uint_as_float(r[2 * j + 1]) * rw);
          uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)fid * p.N + n0 + c0);
          const uint4* srcv = reinterpret_cast<const uint4*>(h);
#pragma unroll
          for (int j = 0; j < 4; ++j) dst[j] = srcv[j];
        }
      }
    } else if (ok && Z == 1) {
      tc_fence_after();
      const int m = m0 + acc * kBM + q * 32 + lane;
#pragma unroll 1
      for (int c0 = col_begin; c0 < col_end; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tlane + (uint32_t)c0, r);
        const int n = n0 + c0;
        if (m < p.M && n < p.N) {
          __align__(16) __half2 h[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float v0 = __uint_as_float(r[2 * j]), v1 = __uint_as_float(r[2 * j + 1]);
            if (p.bias != nullptr) {
              const __half2 b = __ldg(reinterpret_cast<const __half2*>(p.bias + n) + j);
              v0 += __low2float(b);
              v1 += __high2float(b);
            }
            h[j] = __floats2half2_rn(v0, v1);
          }
          uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)m * p.N + n);
          const uint4* srcv = reinterpret_cast<const uint4*>(h);
#pragma unroll
          for (int j = 0; j < 4; ++j) dst[j] = srcv[j];
        }
      }
    } else if (ok && MT == 1) {
      // split-K: spill this CTA's fp32 partial tile to shared memory (the rings are idle now)
      tc_fence_after();
      float* red = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)));
      const int row = q * 32 + lane;
#pragma unroll 1
      for (int c0 = col_begin; c0 < col_end; c0 += 32) {
        uint32_t r[32];
        if (KT > 0) {
          tmem_ld32(tlane + (uint32_t)c0, r);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        float4* dst = reinterpret_cast<float4*>(red + row * C::kRedPitch + c0);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                               __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
      }
    }
  }

  if (MODE == 0 && MT == 1 && Z > 1) {
    // ---------------------------------------------------------------- cluster split-K reduce
    cluster.sync();
    if (!s_abort) {
      float* red = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)));
      constexpr int kUnits = BN / 8;
      const int rbeg = (zrank * kBM) / Z, rend = ((zrank + 1) * kBM) / Z;
      for (int idx = tid; idx < (rend - rbeg) * kUnits; idx += kTcThreads) {
        const int row = rbeg + idx / kUnits, u = idx % kUnits;
        const int m = m0 + row, n = n0 + u * 8;
        if (m >= p.M || n >= p.N) continue;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.f;
        for (int zq = 0; zq < Z; ++zq) {
          const float* peer = cluster.map_shared_rank(red, zq) + row * C::kRedPitch + u * 8;
          const float4 a = *reinterpret_cast<const float4*>(peer);
          const float4 b = *reinterpret_cast<const float4*>(peer + 4);
          v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
          v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
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
    cluster.sync();  // peers may still be reading this CTA's tile
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == kDqWarps + 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d),
                 "r"((uint32_t)C::kTmemCols)
                 : "memory");
  }
}

// ---- host side -------------------------------------------------------------------------------

// fp16 activations [rows, cols], box [64 k x 128 rows], 128-byte swizzle
int make_a_map(CUtensorMap* m, const __half* base, int64_t rows, int cols) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return AWQ_B200_ERR_DRIVER;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBKtc, (cuuint32_t)kBM};
  const cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(base), dims, strides, box,
             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
             ? AWQ_B200_OK
             : AWQ_B200_ERR_DRIVER;
}

// packed weights [rows, words] (experts stacked along the rows), box [16 words x 64 rows]
int make_w_map(CUtensorMap* m, const uint32_t* base, int64_t rows, int words) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return AWQ_B200_ERR_DRIVER;
  const cuuint64_t dims[2] = {(cuuint64_t)words, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)words * 4};
  const cuuint32_t box[2] = {16, (cuuint32_t)kBKtc};
  const cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<uint32_t*>(base), dims, strides, box,
             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
             ? AWQ_B200_OK
             : AWQ_B200_ERR_DRIVER;
}

template <int BN, int MT, int MODE>
int launch_kernel(const CUtensorMap& map_a, const CUtensorMap& map_w, const TcParams& p, dim3 grid,
                  int Z, cudaStream_t stream) {
  using C = TcCfg<BN, MT>;
  static std::atomic<bool> attr_done[64];  // zero-initialised; setting the attribute twice is harmless
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return AWQ_B200_ERR_DEVICE;
  auto kernel = gemm_tc_kernel<BN, MT, MODE>;
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::kSmemBytes) != cudaSuccess)
      return AWQ_B200_ERR_LAUNCH;
    attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kTcThreads, 1, 1);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = Z;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, map_a, map_w, p) != cudaSuccess) {
    cudaGetLastError();
    return AWQ_B200_ERR_LAUNCH;
  }
  return AWQ_B200_OK;
}

template <int BN, int MT>
int launch_tc(const __half* x, const uint32_t* qweight, const TcParams& p, int Z,
              cudaStream_t stream) {
  CUtensorMap map_x, map_w;
  if (int rc = make_a_map(&map_x, x, p.M, p.K)) return rc;
  if (int rc = make_w_map(&map_w, qweight, p.K, p.N / kPack)) return rc;
  const dim3 grid((p.M + kBM * MT - 1) / (kBM * MT), (p.N + BN - 1) / BN, Z);
  return launch_kernel<BN, MT, 0>(map_x, map_w, p, grid, Z, stream);
}

}  // namespace

bool gemm_tc_supported(int M, int N, int K, int group) {
  // TMA needs 16-byte row pitches (K % 8, N % 32); a stage is 64 rows of K and must not
  // straddle quantisation groups.
  return M >= 1 && N % 32 == 0 && K % kBKtc == 0 && (group == 128 || group == 64) &&
         (M + kBM - 1) / kBM <= 65535;
}

size_t gemm_tc_workspace_bytes(int, int, int, int) { return 0; }

int launch_gemm_tc(const __half* x, const uint32_t* qweight, const __half* scales,
                   const uint32_t* qzeros, const __half* bias, __half* out, int M, int N, int K,
                   int group, void*, size_t, cudaStream_t stream) {
  if (!gemm_tc_supported(M, N, K, group)) return AWQ_B200_ERR_SHAPE;
  TcParams p{scales, qzeros, bias, out, M, N, K, group, nullptr, nullptr, nullptr, nullptr, 0, 0};
  const int sms = sm_count();
  const int KT = K / kBKtc;
  auto tiles = [&](int bn, int mt) {
    return (long)((M + kBM * mt - 1) / (kBM * mt)) * ((N + bn - 1) / bn);
  };
  // Preference: the 256-row tile (one dequantised B tile feeds two MMAs) when it fills the GPU;
  // otherwise single-tile CTAs with K split across a cluster until about every SM has work.
  if (M > kBM && tiles(256, 2) * 10 >= (long)sms * 8) return launch_tc<256, 2>(x, qweight, p, 1, stream);
  auto split = [&](long t) {
    long z = t > 0 ? sms / t : 1;
    z = z < 1 ? 1 : (z > 8 ? 8 : z);
    while (z > 1 && KT / z < 4) --z;
    return (int)z;
  };
  const long t256 = tiles(256, 1);
  if (N >= 256 && t256 * 8 >= sms) return launch_tc<256, 1>(x, qweight, p, split(t256), stream);
  return launch_tc<128, 1>(x, qweight, p, split(tiles(128, 1)), stream);
}

// Grouped expert GEMM of a fused-MoE layer on the same pipeline (see the MODE comment of the
// kernel).  a: activations in permuted row order [a_rows, K]; w: packed expert weights stacked
// along the rows [E * K, N / 8].
int launch_tc_grouped(int mode, const __half* a, int64_t a_rows, const uint32_t* w, int experts,
                      const __half* scales, const uint32_t* qzeros, const float* topk_weights,
                      const int32_t* sorted_ids, const int32_t* expert_ids,
                      const int32_t* num_post_pad, __half* out, int numel, int K, int N, int group,
                      int half_cols, int nblk, cudaStream_t stream) {
  CUtensorMap map_a, map_w;
  if (int rc = make_a_map(&map_a, a, a_rows, K)) return rc;
  if (int rc = make_w_map(&map_w, w, (int64_t)experts * K, N / kPack)) return rc;
  TcParams p{scales, qzeros, nullptr, out, (int)a_rows, N, K, group, topk_weights, sorted_ids,
             expert_ids, num_post_pad, numel, half_cols};
  if (mode == 1)
    return launch_kernel<256, 1, 1>(map_a, map_w, p, dim3(nblk, half_cols / 128, 1), 1, stream);
  return launch_kernel<256, 1, 2>(map_a, map_w, p, dim3(nblk, N / 256, 1), 1, stream);
}

int tc_device_status(int* out, int clear) { return read_tc_status(out, clear); }

}  // namespace awq
