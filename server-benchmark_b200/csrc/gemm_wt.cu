// AWQ GEMM with the dequantised weights in tensor memory (any M; built for 32 < M <= 4096).
//
//   D[n, m] = sum_k W[k, n] * x[m, k]          (the transposed product)
//
// The weights are the A operand of tcgen05.mma.kind::f16 (M = 128 weight columns x K = 16) and
// live in TMEM: conversion warps read the packed words from shared memory, dequantise them in
// registers to (q - z) * s in fp16 and write the fragments with tcgen05.st.16x256b.  The
// activations are the B operand ([NT tokens x 64 k] K-major, 128-byte swizzle) exactly as TMA
// delivers them.  Compared with dequantising into a shared-memory B tile (gemm_tc.cu) the fp16
// weights never cross shared memory: per 128-row stage of a 256-column slab the CTA moves
// 48 + 16 KB (TMA writes, packed reads) + 2 * NT * 256 B (operand reads) instead of 352 KB,
// which is what bounds the other kernel.
//
// One CTA per SM (all 512 TMEM columns): slab of 256 output columns = two interleaved A tiles
// (tile u = columns 4u..4u+3 of every packed word), NT = 64 or 128 tokens, K range split over a
// thread-block cluster when the grid would not fill the GPU.  Roles, joined by mbarrier rings:
//
//   producer (1 thread)    TMA: packed weights [128 rows x 128 B] + x [NT x 128 k] of a stage
//                          into a 4-deep ring                                raw_full / raw_empty
//   conversion (16 warps)  warp (q, h, par): TMEM lane quarter q, 16-row steps 4h .. 4h + 3 of the
//                          stages of parity par -> A half par; the A ring holds two stages, so
//                          conversion runs up to two stages ahead of the MMAs
//                                                                            a_full / a_empty
//   issue (1 warp)         converged warp, elected lane: per step one MMA per tile into
//                          D[tile] (fp32, accumulated over the CTA's whole K range);
//                          one tcgen05.commit per stage and ring             d_full
//   epilogue               the conversion warps: tcgen05.ld -> fp32 partial tile in shared
//                          memory -> sum over the cluster ranks through DSMEM -> fp16 (+ bias)
//
// MODE 0 is the dense linear.  MODE 1 / 2 are the grouped expert GEMMs of a fused-MoE layer on
// the permuted token list (moe_align_kernel with block = NT): row block b belongs to expert
// expert_ids[b]; padding tokens only widen the B operand, so they cost no weight work.
//   MODE 1  gate_up: the slab's first 128 columns are gate columns, the other 128 the matching
//           up columns; epilogue act[pos, c] = silu(gate) * up.
//   MODE 2  down: epilogue pair_out[flat pair id, c] = routed weight * D.
//
// TMEM columns: D[2 tiles][NT] at 0 .. 255, A[2 stages][8 steps][2 tiles][8] at 256 .. 511.
// Lane l of quarter q holds output column  64 q + 8 (l % 8) + 2 (2 tile + l / 16) + (l % 16) / 8
// of the slab.  All mbarrier waits are bounded (tc_ptx.cuh).
#include <cooperative_groups.h>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace cg = cooperative_groups;

namespace awq {

namespace {

using namespace tc;

constexpr int kWtBN = 256, kWtBK = 128;
constexpr int kWtRing = 4;
constexpr int kWtWBytes = kWtBK * (kWtBN / kPack) * 4;  // 16384
constexpr int kWtRedPitch = kWtBN + 8;                  // floats
constexpr int kWtCvWarps = 16;
constexpr int kWtIssueWarp = kWtCvWarps, kWtProducerWarp = kWtCvWarps + 1;
constexpr int kWtThreads = 32 * (kWtCvWarps + 2);  // 576
constexpr int kWtTmemCols = 512;
constexpr int kWtColA = 256;  // + (stage parity * 8 + step) * 16 + tile * 8

template <int NT>
struct WtCfg {
  static constexpr int kXBytes = NT * kWtBK * 2;  // two [NT x 64] boxes
  static constexpr int kStageBytes = kWtWBytes + kXBytes;
  static constexpr int kRingBytes = kWtRing * kStageBytes;
  static constexpr int kRedBytes = NT * kWtRedPitch * 4;
  static constexpr int kSmemBytes = (kRingBytes > kRedBytes ? kRingBytes : kRedBytes) + 256 + 1024;
};

struct WtParams {
  const __half* scales;
  const uint32_t* qzeros;
  const __half* bias;
  __half* out;
  int M, N, K;
  // grouped modes
  const float* topk_weights;   // [numel] routed weights (MODE 2)
  const int32_t* sorted_ids;   // permuted flat (token, slot) ids, padding = numel
  const int32_t* expert_ids;   // expert of every NT-row block
  const int32_t* num_post_pad;
  int numel;                   // tokens * topk
  int half_cols;               // MODE 1: I (gate columns [0, I), up columns [I, 2 I))
};

__device__ __forceinline__ void wt_tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ __half2 dup_lo(uint32_t v) { return as_half2(prmt(v, v, 0x1010)); }
__device__ __forceinline__ __half2 dup_hi(uint32_t v) { return as_half2(prmt(v, v, 0x3232)); }

template <int NT, int MODE>
__global__ void __launch_bounds__(kWtThreads, 1)
gemm_wt_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const WtParams p) {
  using C = WtCfg<NT>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ volatile int s_abort;
  __shared__ uint32_t s_tmem_base;

  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int S = (int)cluster.num_blocks();

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  float* red = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)));
  const uint32_t bar_base =
      smem_base + (C::kRingBytes > C::kRedBytes ? C::kRingBytes : C::kRedBytes);
  auto raw_full = [&](int s) { return bar_base + 8 * s; };
  auto raw_empty = [&](int s) { return bar_base + 8 * (kWtRing + s); };
  auto a_full = [&](int par) { return bar_base + 8 * (2 * kWtRing + par); };
  auto a_empty = [&](int par) { return bar_base + 8 * (2 * kWtRing + 2 + par); };
  const uint32_t d_full = bar_base + 8 * (2 * kWtRing + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int words = p.N / kPack;
  const int m0 = blockIdx.z * NT;
  const int KT = p.K / kWtBK;
  // The slab's packed words come as two boxes of 16 words: [w_left, +16) and [w_right, +16).
  int w_left, w_right, wrow0 = 0, grp0 = 0;
  if (MODE == 0) {
    w_left = blockIdx.y * (kWtBN / kPack);
    w_right = w_left + 16;
  } else {
    if (m0 >= p.num_post_pad[0]) return;  // block past the permuted list (whole CTA, cluster of 1)
    const int e = p.expert_ids[blockIdx.z];
    if (e < 0) return;
    wrow0 = e * p.K;
    grp0 = e * KT;
    if (MODE == 1) {
      w_left = blockIdx.y * 16;
      w_right = p.half_cols / kPack + blockIdx.y * 16;
    } else {
      w_left = blockIdx.y * (kWtBN / kPack);
      w_right = w_left + 16;
    }
  }
  const int st_begin = (int)(((long long)rank * KT) / S);
  const int st_end = (int)(((long long)(rank + 1) * KT) / S);
  const int nst = st_end - st_begin;

  // producer thread: TMA loads of local stage j, packed weights and tokens
  auto load_w = [&](int j) {
    const int s = j % kWtRing;
    const uint32_t dst = smem_base + s * C::kStageBytes;
    const int k0 = (st_begin + j) * kWtBK;
    mbar_arrive_expect_tx(raw_full(s), C::kStageBytes);
    tma_load_2d(dst, &map_w, w_left, wrow0 + k0, raw_full(s));
    tma_load_2d(dst + kWtWBytes / 2, &map_w, w_right, wrow0 + k0, raw_full(s));
  };
  auto load_x = [&](int j) {
    const int s = j % kWtRing;
    const uint32_t dst = smem_base + s * C::kStageBytes + kWtWBytes;
    const int k0 = (st_begin + j) * kWtBK;
    tma_load_2d(dst, &map_x, k0, m0, raw_full(s));
    tma_load_2d(dst + NT * 128, &map_x, k0 + 64, m0, raw_full(s));
  };
  if (MODE == 0) pdl_launch_dependents();
  if (warp == kWtProducerWarp && lane == 0) {
    // this thread sets the barriers up and has the first stages in flight before anyone else
    // is through the prologue (the first TMA round trip is the longest latency of a short CTA)
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    s_abort = 0;
    for (int s = 0; s < kWtRing; ++s) {
      mbar_init(raw_full(s), 1);
      mbar_init(raw_empty(s), kWtCvWarps / 2 + 1);  // the stage's conversion warps + the issuer's commit
    }
    for (int par = 0; par < 2; ++par) {
      mbar_init(a_full(par), kWtCvWarps / 2);  // one arrival per conversion warp of that parity
      mbar_init(a_empty(par), 1);
    }
    mbar_init(d_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
    // weights first: they do not depend on the kernel before this one in the stream
    for (int j = 0; j < nst && j < kWtRing; ++j) load_w(j);
    pdl_wait();
    for (int j = 0; j < nst && j < kWtRing; ++j) load_x(j);
  }
  __syncwarp();
  if (warp == kWtProducerWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "r"((uint32_t)kWtTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;

  if (warp == kWtProducerWarp) {
    // ------------------------------------------------------------------ producer: TMA
    // (the first kWtRing stages were issued in the prologue)
    if (lane == 0) {
      bool ok = true;
      for (int j = kWtRing; j < nst && ok; ++j) {
        ok = mbar_wait(raw_empty(j % kWtRing), (uint32_t)((j / kWtRing - 1) & 1), &s_abort, 31);
        if (ok) {
          load_w(j);
          load_x(j);
        }
      }
    }
  } else if (warp == kWtIssueWarp) {
    // ------------------------------------------------------------------ MMA issue
    // D fp32, A/B fp16, both K-major, N = NT tokens, M = 128 weight columns.  The whole warp
    // runs the loop converged, one elected lane issues; operands are kept warp-uniform.
    constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | (8u << 24);
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
    const uint32_t ring_u = __shfl_sync(0xffffffffu, smem_base, 0);
    bool ok = true;
    int s = 0;
    uint32_t ring_phase = 0;
    // Every wait costs this warp ~100 cycles of latency even when the phase is complete, so
    // there are two per stage (x tile landed, A half converted), and both are probed for stage
    // j + 1 before the last MMAs of stage j are issued.
    if (nst > 0) {
      ok = mbar_wait(raw_full(0), 0, &s_abort, 32);
      if (ok) ok = mbar_wait(a_full(0), 0, &s_abort, 33);
      ok = __all_sync(0xffffffffu, ok);
    }
    for (int j = 0; j < nst && ok; ++j) {
      const uint32_t xt = ring_u + s * C::kStageBytes + kWtWBytes;
      const int par = j & 1;
      int sn = s + 1;
      uint32_t phase_n = ring_phase;
      if (sn == kWtRing) {
        sn = 0;
        phase_n ^= 1u;
      }
      auto issue = [&](int first, int last) {  // 16-row steps [first, last] of the stage
#pragma unroll
        for (int step = 0; step < 8; ++step) {
          if (step < first || step > last) continue;
          const uint64_t db = make_desc(xt + (step >> 2) * (NT * 128), 16, 1024) +
                              (uint64_t)(((step & 3) * 32) >> 4);
          const uint32_t acc = (j > 0 || step > 0) ? 1u : 0u;
          const uint32_t acol = tmem_u + kWtColA + (par * 8 + step) * 16;
          umma_f16_ts(tmem_u, acol, db, idesc, acc);
          umma_f16_ts(tmem_u + NT, acol + 8, db, idesc, acc);
        }
      };
      tc_fence_after();
      if (elect_one()) issue(0, 5);
      __syncwarp();
      // What stage j + 1 needs is probed while the MMAs just issued run.  The probe must not
      // block: the commit of stage j below is what lets the conversion of stage j + 2 start.
      bool ready = true;
      if (j + 1 < nst) {
        ready = mbar_test(raw_full(sn), phase_n);
        ready &= mbar_test(a_full(par ^ 1), (uint32_t)(((j + 1) >> 1) & 1));
        ready = __all_sync(0xffffffffu, ready);
      }
      if (elect_one()) {
        issue(6, 7);
        umma_commit(a_empty(par));
        umma_commit(raw_empty(s));  // x tile of the stage read
      }
      __syncwarp();
      if (!ready) {
        ok = mbar_wait(raw_full(sn), phase_n, &s_abort, 32);
        if (ok) ok = mbar_wait(a_full(par ^ 1), (uint32_t)(((j + 1) >> 1) & 1), &s_abort, 33);
        ok = __all_sync(0xffffffffu, ok);
      }
      s = sn;
      ring_phase = phase_n;
    }
    if (ok && elect_one()) umma_commit(d_full);
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ conversion warps
    const int g = lane >> 2, t = lane & 3;
    // Warp (q, h, par): TMEM lane quarter q, steps 4 h .. 4 h + 3 of the stages of parity par
    // (one set-up of the group's scales and zeros serves four steps; the chains of consecutive
    // stages run on different warps and overlap).  In the epilogue the same warp is (q, r).
    const int q = warp & 3, h = (warp >> 2) & 1, par = warp >> 3, r = warp >> 2;
    const uint32_t lane_q = (uint32_t)(q * 32) << 16;
    // raw tile as TMA leaves it: two boxes of [128 rows x 64 B] (64-byte swizzle): row k of box
    // q / 2 at k * 64, 16-byte chunk c at position c ^ ((k / 2) % 4).
    // This lane reads word 8 (q % 2) + g of that box, rows 16 step + 4 t + rr.
    const int chunk_id = 2 * (q & 1) + (g >> 2);
    uint32_t off[4];
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
      const int row = 4 * t + rr;
      off[rr] = (uint32_t)((q >> 1) * (kWtWBytes / 2) + row * 64 +
                           ((chunk_id ^ ((row >> 1) & 3)) << 4) + (g & 3) * 4);
    }
    const int conv_word = min(((q >> 1) ? w_right : w_left) + 8 * (q & 1) + g, words - 1);
    const uint32_t* zp = p.qzeros + (size_t)(grp0 + st_begin) * words + conv_word;
    const uint4* sp =
        reinterpret_cast<const uint4*>(p.scales + (size_t)(grp0 + st_begin) * p.N) + conv_word;
    const size_t spitch = (size_t)p.N / 8;
    // scale / zero rows of this warp's next stage (two stages on) are fetched while it converts
    // the current one; rows further on are pulled into L2
    uint32_t zw_n = 0;
    uint4 sv_n = make_uint4(0, 0, 0, 0);
    if (par < nst) {
      zw_n = __ldg(zp + (size_t)par * words);
      sv_n = __ldg(sp + (size_t)par * spitch);
    }

    bool ok = true;
    for (int j = par; j < nst && ok; j += 2) {
      const int s = j % kWtRing;
      const uint32_t wsm = smem_base + s * C::kStageBytes;
      // zero point and scale of this lane's eight columns for the group (= stage):
      // zu/su[i] belong to column 2 i, zv/sv[i] to column 2 i + 1, duplicated over (k, k + 1).
      // Odd i keep the nibble in place (1024 + 16 q): their zero is 1024 + 16 z, their scale s / 16.
      __half2 zu[4], zv[4], su[4], sv[4];
      {
        const uint32_t zw = zw_n;
        const uint4 sc = sv_n;
        if (j + 2 < nst) {
          zw_n = __ldg(zp + (size_t)(j + 2) * words);
          sv_n = __ldg(sp + (size_t)(j + 2) * spitch);
          if (t == 0 && h == 0) {
            const int jp = min(j + 6, nst - 1);
            asm volatile("prefetch.global.L2 [%0];" ::"l"(zp + (size_t)jp * words));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(sp + (size_t)jp * spitch));
          }
        }
        const uint32_t uz = prmt(zw, zw, 0x1010), vz = prmt(zw, zw, 0x3232);
        zu[0] = as_half2(lop3_and_or(uz, 0x000F000Fu, 0x64006400u));
        zv[0] = as_half2(lop3_and_or(vz, 0x000F000Fu, 0x64006400u));
        zu[1] = as_half2(lop3_and_or(uz, 0x00F000F0u, 0x64006400u));
        zv[1] = as_half2(lop3_and_or(vz, 0x00F000F0u, 0x64006400u));
        zu[2] = as_half2(lop3_and_or(uz >> 8, 0x000F000Fu, 0x64006400u));
        zv[2] = as_half2(lop3_and_or(vz >> 8, 0x000F000Fu, 0x64006400u));
        zu[3] = as_half2(lop3_and_or(uz >> 8, 0x00F000F0u, 0x64006400u));
        zv[3] = as_half2(lop3_and_or(vz >> 8, 0x00F000F0u, 0x64006400u));
        const __half2 r16 = __float2half2_rn(0.0625f);
        su[0] = dup_lo(sc.x);
        sv[0] = dup_hi(sc.x);
        su[1] = __hmul2(dup_lo(sc.y), r16);
        sv[1] = __hmul2(dup_hi(sc.y), r16);
        su[2] = dup_lo(sc.z);
        sv[2] = dup_hi(sc.z);
        su[3] = __hmul2(dup_lo(sc.w), r16);
        sv[3] = __hmul2(dup_hi(sc.w), r16);
      }
      ok = mbar_wait(raw_full(s), (uint32_t)((j / kWtRing) & 1), &s_abort, 34);
      if (!ok) break;
      // all four steps' packed words first: the loads must not queue up behind tcgen05.st
      uint32_t w[4][4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t rowA = wsm + (16 * (4 * h + e)) * 64;
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) w[e][rr] = lds32(rowA + off[rr]);
      }
      // the MMAs of stage j - 2 must have read this half of the A ring
      if (j >= 2) ok = mbar_wait(a_empty(par), (uint32_t)(((j >> 1) - 1) & 1), &s_abort, 35);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int sp2 = 0; sp2 < 2; ++sp2) {
        // fragments of two steps: frag[hq][4 * (2 e + tile) + k] -- the two tiles of a step and
        // two consecutive steps are adjacent column groups of the A ring, so one x4 store per
        // half-quarter writes all four
        uint32_t frag[2][16];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t* ww = w[2 * sp2 + e];
          const uint32_t u0 = prmt(ww[0], ww[1], 0x5410), v0 = prmt(ww[0], ww[1], 0x7632);
          const uint32_t u1 = prmt(ww[2], ww[3], 0x5410), v1 = prmt(ww[2], ww[3], 0x7632);
          const uint32_t u0h = u0 >> 8, v0h = v0 >> 8, u1h = u1 >> 8, v1h = v1 >> 8;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t mask = (i & 1) ? 0x00F000F0u : 0x000F000Fu;
            const uint32_t su0 = (i & 2) ? u0h : u0, sv0 = (i & 2) ? v0h : v0;
            const uint32_t su1 = (i & 2) ? u1h : u1, sv1 = (i & 2) ? v1h : v1;
            // (col 2i: k 4t..4t+1 | 4t+2..4t+3), (col 2i+1: same); (q - z) exact, then the scale
            const int c = 4 * (2 * e + (i >> 1));
            frag[i & 1][c] = as_u32(__hmul2(
                __hsub2(as_half2(lop3_and_or(su0, mask, 0x64006400u)), zu[i]), su[i]));
            frag[i & 1][c + 1] = as_u32(__hmul2(
                __hsub2(as_half2(lop3_and_or(su1, mask, 0x64006400u)), zu[i]), su[i]));
            frag[i & 1][c + 2] = as_u32(__hmul2(
                __hsub2(as_half2(lop3_and_or(sv0, mask, 0x64006400u)), zv[i]), sv[i]));
            frag[i & 1][c + 3] = as_u32(__hmul2(
                __hsub2(as_half2(lop3_and_or(sv1, mask, 0x64006400u)), zv[i]), sv[i]));
          }
        }
        // half-quarter hq of this warp's lanes; steps 4 h + 2 sp2, + 1; both tiles
        const uint32_t a_slot = tmem + lane_q + kWtColA + (par * 8 + 4 * h + 2 * sp2) * 16;
        tmem_st_16x256b_x4(a_slot, frag[0]);
        tmem_st_16x256b_x4(a_slot + (16u << 16), frag[1]);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      // every lane's TMEM stores are complete and its reads of the stage were consumed; one
      // arrival per warp (hundreds of arrivals on one shared-memory word would serialise)
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(a_full(par));
        mbar_arrive(raw_empty(s));
      }
    }

    // ---------------------------------------------------------------- epilogue
    // warp (q, r): its lane quarter, tokens [r NT / 4, (r + 1) NT / 4) of both tiles ->
    // red[token][column of the slab] (aliases the ring: d_full implies every stage was
    // converted and read by the tensor core)
    if (ok && nst > 0) ok = mbar_wait(d_full, 0, &s_abort, 36);
    if (ok) {
      tc_fence_after();
      const int hp = lane >> 4, odd = (lane >> 3) & 1, gp = lane & 7;
      constexpr int kTok = NT / 4;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int nl = 64 * q + 8 * gp + 2 * (2 * u + hp) + odd;
#pragma unroll
        for (int c0 = 0; c0 < kTok; c0 += 16) {
          uint32_t d[16];
          if (nst > 0) {
            wt_tmem_ld16(tmem + lane_q + (uint32_t)(u * NT + r * kTok + c0), d);
          } else {
#pragma unroll
            for (int m = 0; m < 16; ++m) d[m] = 0u;
          }
#pragma unroll
          for (int m = 0; m < 16; ++m)
            red[(r * kTok + c0 + m) * kWtRedPitch + nl] = __uint_as_float(d[m]);
        }
      }
    }
  }

  // ---- reduction over the cluster ranks through distributed shared memory ----
  tc_fence_before();
  __syncthreads();
  if (S > 1) cluster.sync();  // every rank's partial tile is in its shared memory
  pdl_wait();  // long since satisfied; orders this thread's writes of `out` after the earlier kernel
  if (!s_abort) {
    if (MODE == 0) {
      constexpr int kUnits = kWtBN / 8;
      const int ubeg = (rank * kUnits) / S, uend = ((rank + 1) * kUnits) / S;
      const int nun = uend - ubeg;
      const int n_slab = blockIdx.y * kWtBN;
      for (int idx = tid; idx < nun * NT; idx += kWtThreads) {
        const int u = ubeg + idx % nun, ml = idx / nun;
        const int n = n_slab + u * 8, m = m0 + ml;
        if (m >= p.M || n >= p.N) continue;
        float v[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) v[jj] = 0.f;
        for (int rk = 0; rk < S; ++rk) {
          const float* peer = cluster.map_shared_rank(red, rk) + ml * kWtRedPitch + u * 8;
          const float4 a = *reinterpret_cast<const float4*>(peer);
          const float4 b = *reinterpret_cast<const float4*>(peer + 4);
          v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
          v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
        }
        if (p.bias != nullptr) {
          const uint4 bv = __ldg(reinterpret_cast<const uint4*>(p.bias + n));
          const __half* bh = reinterpret_cast<const __half*>(&bv);
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) v[jj] += __half2float(bh[jj]);
        }
        __align__(16) __half o[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) o[jj] = __float2half_rn(v[jj]);
        *reinterpret_cast<uint4*>(p.out + (size_t)m * p.N + n) = *reinterpret_cast<uint4*>(o);
      }
    } else if (MODE == 1) {
      // act[pos, 128 slab + c] = silu(gate) * up; gate = red[.][c], up = red[.][128 + c]
      for (int idx = tid; idx < 16 * NT; idx += kWtThreads) {
        const int u = idx % 16, ml = idx / 16;
        const int c = blockIdx.y * 128 + u * 8;
        if (c >= p.half_cols) continue;
        const float* gp = red + ml * kWtRedPitch + u * 8;
        __align__(16) __half o[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const float gv = gp[jj];
          o[jj] = __float2half_rn(gv / (1.f + __expf(-gv)) * gp[128 + jj]);
        }
        *reinterpret_cast<uint4*>(p.out + (size_t)(m0 + ml) * p.half_cols + c) =
            *reinterpret_cast<uint4*>(o);
      }
    } else {
      // pair_out[flat pair id, 256 slab + c] = routed weight * D
      for (int idx = tid; idx < 32 * NT; idx += kWtThreads) {
        const int u = idx % 32, ml = idx / 32;
        const int n = blockIdx.y * kWtBN + u * 8;
        const int fid = p.sorted_ids[m0 + ml];
        if (fid >= p.numel || n >= p.N) continue;
        const float rw = __ldg(p.topk_weights + fid);
        const float* src = red + ml * kWtRedPitch + u * 8;
        __align__(16) __half o[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) o[jj] = __float2half_rn(src[jj] * rw);
        *reinterpret_cast<uint4*>(p.out + (size_t)fid * p.N + n) = *reinterpret_cast<uint4*>(o);
      }
    }
  }
  if (S > 1) cluster.sync();  // peers are done reading this CTA's shared memory

  // ---- teardown ----
  tc_fence_before();
  __syncthreads();
  if (warp == kWtProducerWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                 "r"((uint32_t)kWtTmemCols)
                 : "memory");
  }
}

template <int NT, int MODE>
int launch_wt_kernel(const CUtensorMap& map_w, const CUtensorMap& map_x, const WtParams& p, dim3 grid,
                     int S, cudaStream_t stream) {
  using C = WtCfg<NT>;
  static std::atomic<bool> attr_done[64];  // zero-initialised; setting the attribute twice is harmless
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return AWQ_B200_ERR_DEVICE;
  auto kernel = gemm_wt_kernel<NT, MODE>;
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::kSmemBytes) != cudaSuccess)
      return AWQ_B200_ERR_LAUNCH;
    attr_done[dev] = true;
  }
  if (MODE == 0 && S > 1) {
    // the K split only as wide as lets every cluster of the grid be resident at once
    static std::atomic<int> resident[64][9];  // zero-initialised: not asked yet
    const int clusters = (int)(grid.y * grid.z);
    while (S > 1 && resident_clusters(kernel, S, kWtThreads, C::kSmemBytes, resident[dev]) < clusters)
      --S;
    grid.x = S;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kWtThreads, 1, 1);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  // the grouped modes read the routing tables of the kernels before them from their first
  // instruction on and are launched without the attribute
  cfg.numAttrs = MODE == 0 ? add_pdl_attribute(attr, 1) : 1;
  if (cudaLaunchKernelEx(&cfg, kernel, map_w, map_x, p) != cudaSuccess) {
    cudaGetLastError();
    return AWQ_B200_ERR_LAUNCH;
  }
  return AWQ_B200_OK;
}

// packed weights [rows][N / 8 words], box [128 rows x 16 words], 64-byte swizzle;
// activations [a_rows][K], box [NT tokens x 64 k] (rows past the end read as zero), 128-byte swizzle
int make_wt_maps(CUtensorMap* map_w, CUtensorMap* map_x, const uint32_t* qweight, int64_t wrows,
                 int N, const __half* x, int64_t a_rows, int K, int nt) {
  if (int rc = encode_map_2d(map_w, CU_TENSOR_MAP_DATA_TYPE_INT32, qweight, (uint64_t)(N / kPack),
                             (uint64_t)wrows, (uint64_t)(N / kPack) * 4, 16, kWtBK,
                             CU_TENSOR_MAP_SWIZZLE_64B))
    return rc;
  return encode_map_2d(map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x, (uint64_t)K, (uint64_t)a_rows,
                       (uint64_t)K * 2, 64, (uint32_t)nt, CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int NT>
int launch_wt(const uint32_t* qweight, const __half* x, const WtParams& p, cudaStream_t stream) {
  CUtensorMap map_w, map_x;
  if (int rc = make_wt_maps(&map_w, &map_x, qweight, p.K, p.N, x, p.M, p.K, NT)) return rc;
  const int slabs = (p.N + kWtBN - 1) / kWtBN;
  const int mtiles = (p.M + NT - 1) / NT;
  const int KT = p.K / kWtBK;
  // cluster size (K split): only when the tiles alone leave SMs idle (one CTA per SM, and a
  // cluster has to find all its SMs free at once, which costs more than it gains otherwise)
  const int slots = sm_count();
  const int tiles = slabs * mtiles;
  int S = 1;
  if (tiles < slots) {
    S = slots / tiles;
    S = S > 8 ? 8 : S;
    while (S > 1 && KT / S < 4) --S;
  }
  return launch_wt_kernel<NT, 0>(map_w, map_x, p, dim3(S, slabs, mtiles), S, stream);
}

}  // namespace

bool gemm_wt_supported(int M, int N, int K, int group) {
  // N % 32: 16-byte TMA row pitch of the packed weights; K % 128: whole stages = whole groups
  return M >= 1 && N % 32 == 0 && K % kWtBK == 0 && group == 128;
}

int launch_gemm_wt(const __half* x, const uint32_t* qweight, const __half* scales,
                   const uint32_t* qzeros, const __half* bias, __half* out, int M, int N, int K,
                   int group, cudaStream_t stream) {
  if (!gemm_wt_supported(M, N, K, group)) return AWQ_B200_ERR_SHAPE;
  WtParams p{scales, qzeros, bias, out, M, N, K, nullptr, nullptr, nullptr, nullptr, 0, 0};
  return M <= 64 ? launch_wt<64>(qweight, x, p, stream) : launch_wt<128>(qweight, x, p, stream);
}

bool moe_wt_supported(int H, int I, int group) {
  // slabs: 128 gate + 128 up columns (I % 128), 256 hidden columns (H % 256); stage = group = 128
  return H % 256 == 0 && I % 128 == 0 && group == 128;
}

// Grouped expert GEMM of a fused-MoE layer (MODE 1 / 2 of the kernel).  a: activations in
// permuted row order [a_rows, K] (row blocks of 128); w: packed expert weights stacked along the
// rows [experts * K, N / 8].
int launch_wt_grouped(int mode, const __half* a, int64_t a_rows, const uint32_t* w, int experts,
                      const __half* scales, const uint32_t* qzeros, const float* topk_weights,
                      const int32_t* sorted_ids, const int32_t* expert_ids,
                      const int32_t* num_post_pad, __half* out, int numel, int K, int N, int group,
                      int half_cols, int nblk, cudaStream_t stream) {
  if (group != 128 || K % kWtBK != 0 || N % 32 != 0) return AWQ_B200_ERR_SHAPE;
  CUtensorMap map_w, map_x;
  if (int rc = make_wt_maps(&map_w, &map_x, w, (int64_t)experts * K, N, a, a_rows, K, 128)) return rc;
  WtParams p{scales, qzeros, nullptr, out, (int)a_rows, N, K, topk_weights, sorted_ids,
             expert_ids, num_post_pad, numel, half_cols};
  if (mode == 1)
    return launch_wt_kernel<128, 1>(map_w, map_x, p, dim3(1, half_cols / 128, nblk), 1, stream);
  return launch_wt_kernel<128, 2>(map_w, map_x, p, dim3(1, N / kWtBN, nblk), 1, stream);
}

int wt_device_status(int* out, int clear) { return read_tc_status(out, clear); }

}  // namespace awq
