// Decode-size AWQ GEMM (M <= 16) on tcgen05 with the weights going registers -> TMEM.
//
//   D[n, m] = sum_k W[k, n] * x[m, k]          (the transposed product, as in stream_core.cuh)
//
// The int4 weights are unpacked in registers exactly as in the mma.sync streaming kernel (prmt
// pairs two rows, one AND per 32-bit pair, nibbles used as fp16 subnormals), but the fragments are
// not fed to mma.sync: they are written to tensor memory with tcgen05.st.16x256b and become the
// A operand (128 weight columns x 16 k) of tcgen05.mma.kind::f16; the activations are the small
// B operand ([16 tokens x 64 k] K-major, 128-byte swizzle) in shared memory.  The dequantised
// weights never touch shared memory, the 5th-generation tensor core does the arithmetic, and the
// conversion warps execute nothing but the unpack (one instruction per weight).
//
// One CTA per SM (all 512 TMEM columns); slab of 256 output columns = two interleaved 128-lane A
// tiles (tile u = columns 4u..4u+3 of every packed word); stage = 128 weight rows = one
// quantisation group; K range split over a thread-block cluster when the slabs alone would
// leave SMs idle.  Roles, joined by mbarrier rings:
//
//   producer (1 thread)    TMA: packed weights [128 rows x 128 B] + x [16 tokens x 128 k] of a
//                          stage into a 6-deep ring                          raw_full / raw_empty
//   conversion (16 warps)  warp (q, h, par): TMEM lane quarter q, 16-row steps 4h .. 4h + 3 of
//                          the stages of parity par: ld.shared -> unpack -> tcgen05.st into the
//                          A ring.  The ring holds three stages and each parity has its own
//                          warps, so the conversions of consecutive stages overlap and run
//                          ahead of the MMAs                                 a_full / a_empty
//   issue (1 warp)         converged warp, one elected lane: per step one MMA per A tile (weight
//                          tile 0, weight tile 1, constant tile) into the group accumulators
//                          D[b]                                              done[b] / d_empty[b]
//   fold (4 warps)         warp q: tcgen05.ld its lanes of D[b];
//                          tot += scale * (acc - zero * sum_x) in fp32 registers
//
// The constant tile (every k slot = 2^-24) yields sum_k x per token in the same scaling as the
// weight tiles, so the zero point is applied per group without a separate reduction.
//
// Measured on B200 while building this kernel (cycles of the SM clock):
//   * a tcgen05.mma / tcgen05.commit issued by one lane that loops alone (the other 31 lanes of
//     its warp parked at a barrier) costs that lane 45 to 270 cycles depending on how its
//     operands are computed; issued from a converged warp under elect.sync with warp-uniform
//     operands it costs ~23 (M = 128, N = 16, K = 16, A in TMEM);
//   * every mbarrier wait costs its warp ~100 cycles even when the phase is already complete,
//     so the issuing warp probes the barriers of stage j + 1 before the last MMAs of stage j;
//   * with two CTAs per SM (256 TMEM columns each) only one stage of A fits next to the
//     accumulators, conversion of stage j + 1 then waits for the MMAs of stage j and the
//     latencies add up (2.1 - 2.5 TB/s); hence one CTA per SM and a three-stage A ring: the
//     chain  slot free -> convert -> issue -> MMAs complete  (~2100 cycles) has three stage
//     times to close.
//
// TMEM columns: D[2 buffers][3 tiles][16] at 0 .. 95, constant tile at 96 .. 103,
// A[3 stages][8 steps][2 tiles][8] at 128 .. 511.  Lane l of quarter q holds output column
//   64 q + 8 (l % 8) + 2 (2 tile + l / 16) + (l % 16) / 8      of the slab.
//
// All mbarrier waits are bounded (tc_ptx.cuh); a wait that runs out aborts the CTA cleanly.
#include <cooperative_groups.h>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace cg = cooperative_groups;

namespace awq {

namespace {

using namespace tc;

constexpr int kTsBN = 256, kTsBK = 128;
constexpr int kNT = 16;                         // tokens padded to the MMA's N
constexpr int kRing = 6;                        // stages in flight
constexpr int kTsWBytes = kTsBK * (kTsBN / kPack) * 4;  // 16384
constexpr int kTsXBytes = kNT * kTsBK * 2;              // 4096: two [16 x 64] tiles
constexpr int kTsStageBytes = kTsWBytes + kTsXBytes;    // 20480
constexpr int kTsRingBytes = kRing * kTsStageBytes;     // 122880
constexpr int kTsRedPitch = kTsBN + 8;                  // floats
constexpr int kTsSmemBytes = kTsRingBytes + 256 + 1024;  // + barriers + alignment slack
constexpr int kCvWarps = 16, kFoldWarps = 4;
constexpr int kFoldWarp0 = kCvWarps, kIssueWarp = kCvWarps + kFoldWarps;
constexpr int kProducerWarp = kIssueWarp + 1;
constexpr int kTsThreads = 32 * (kProducerWarp + 1);  // 704
constexpr int kTmemColsTs = 512;
constexpr int kColD = 0;      // + buffer * 48 + tile * 16
constexpr int kColOnes = 96;
constexpr int kASlots = 3;     // stages of A held in TMEM
constexpr int kColA = 128;    // + (slot * 8 + step) * 16 + tile * 8
static_assert(kNT * kTsRedPitch * 4 <= kTsRingBytes, "partial tile must fit the idle ring");

struct TsParams {
  const __half* scales;
  const uint32_t* qzeros;
  const __half* bias;
  __half* out;
  int M, N, K;
};

__device__ __forceinline__ void tmem_st_16x256b(uint32_t taddr, uint32_t r0, uint32_t r1,
                                                uint32_t r2, uint32_t r3) {
  asm volatile("tcgen05.st.sync.aligned.16x256b.x1.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr),
               "r"(r0), "r"(r1), "r"(r2), "r"(r3)
               : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7])
      : "r"(taddr)
      : "memory");
}

template <bool EXACT>
__global__ void __launch_bounds__(kTsThreads, 1)
gemm_ts_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const TsParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ volatile int s_abort;
  __shared__ uint32_t s_tmem_base;

  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int S = (int)cluster.num_blocks();

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  float* red = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)));
  const uint32_t bar_base = smem_base + kTsRingBytes;
  auto raw_full = [&](int s) { return bar_base + 8 * s; };
  auto raw_empty = [&](int s) { return bar_base + 8 * (kRing + s); };
  auto a_full = [&](int slot) { return bar_base + 8 * (2 * kRing + slot); };
  auto a_empty = [&](int slot) { return bar_base + 8 * (2 * kRing + 3 + slot); };
  auto done = [&](int par) { return bar_base + 8 * (2 * kRing + 6 + par); };
  auto d_empty = [&](int par) { return bar_base + 8 * (2 * kRing + 8 + par); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int words = p.N / kPack;
  const int word0 = blockIdx.y * (kTsBN / kPack);
  const int KT = p.K / kTsBK;
  const int st_begin = (int)(((long long)rank * KT) / S);
  const int st_end = (int)(((long long)(rank + 1) * KT) / S);
  const int nst = st_end - st_begin;

  // producer thread: TMA loads of local stage j, packed weights and activations
  auto load_w = [&](int j) {
    const int s = j % kRing;
    mbar_arrive_expect_tx(raw_full(s), kTsStageBytes);
    tma_load_2d(smem_base + s * kTsStageBytes, &map_w, word0, (st_begin + j) * kTsBK, raw_full(s));
  };
  auto load_x = [&](int j) {
    const int s = j % kRing;
    const uint32_t dst = smem_base + s * kTsStageBytes + kTsWBytes;
    const int k0 = (st_begin + j) * kTsBK;
    tma_load_2d(dst, &map_x, k0, 0, raw_full(s));
    tma_load_2d(dst + 2048, &map_x, k0 + 64, 0, raw_full(s));
  };
  pdl_launch_dependents();
  if (warp == kProducerWarp && lane == 0) {
    // this thread sets the barriers up and has the first stages in flight before anyone else
    // is through the prologue (the first TMA round trip is the longest latency of a short CTA)
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    s_abort = 0;
    for (int s = 0; s < kRing; ++s) {
      mbar_init(raw_full(s), 1);
      mbar_init(raw_empty(s), kCvWarps / 2 + 1);  // the stage's conversion warps + the issuer's commit
    }
    for (int slot = 0; slot < kASlots; ++slot) {
      mbar_init(a_full(slot), kCvWarps / 2);  // one arrival per conversion warp of the stage
      mbar_init(a_empty(slot), 1);            // commit after the MMAs that read the slot
    }
    for (int par = 0; par < 2; ++par) {
      mbar_init(done(par), 1);                // commit after the MMAs of a stage: D[par] complete
      mbar_init(d_empty(par), kFoldWarps);    // one arrival per fold warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
    // weights first: they do not depend on the kernel before this one in the stream
    for (int j = 0; j < nst && j < kRing; ++j) load_w(j);
    pdl_wait();
    for (int j = 0; j < nst && j < kRing; ++j) load_x(j);
  }
  __syncwarp();
  if (warp == kProducerWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "r"((uint32_t)kTmemColsTs)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ producer: TMA
    // (the first kRing stages were issued in the prologue)
    if (lane == 0) {
      bool ok = true;
      for (int j = kRing; j < nst && ok; ++j) {
        ok = mbar_wait(raw_empty(j % kRing), (uint32_t)((j / kRing - 1) & 1), &s_abort, 21);
        if (ok) {
          load_w(j);
          load_x(j);
        }
      }
    }
  } else if (warp == kIssueWarp) {
    // ------------------------------------------------------------------ MMA issue
    // D fp32, A/B fp16, both K-major, N = 16 tokens, M = 128 weight columns.  The whole warp
    // runs the loop converged, one elected lane issues; the operands are computed from
    // warp-uniform values only (broadcast bases, wrapping counters instead of divisions).
    constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(kNT >> 3) << 17) | (8u << 24);
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
    const uint32_t ring_u = __shfl_sync(0xffffffffu, smem_base, 0);
    bool ok = true;
    int s = 0, slot = 0;               // ring slot and A slot of stage j (wrapping counters)
    uint32_t ring_phase = 0, slot_phase = 0;
    if (nst > 0) {
      ok = mbar_wait(raw_full(0), 0, &s_abort, 11);
      if (ok) ok = mbar_wait(a_full(0), 0, &s_abort, 12);
      ok = __all_sync(0xffffffffu, ok);
    }
    for (int j = 0; j < nst && ok; ++j) {
      const uint32_t xt = ring_u + s * kTsStageBytes + kTsWBytes;
      const int par = j & 1;
      const uint32_t dcol = tmem_u + kColD + par * 48;
      int sn = s + 1, slot_n = slot + 1;
      uint32_t phase_n = ring_phase, slot_phase_n = slot_phase;
      if (sn == kRing) {
        sn = 0;
        phase_n ^= 1u;
      }
      if (slot_n == kASlots) {
        slot_n = 0;
        slot_phase_n ^= 1u;
      }
      auto issue = [&](int first, int last) {  // 16-row steps [first, last] of the stage
#pragma unroll
        for (int step = 0; step < 8; ++step) {
          if (step < first || step > last) continue;
          const uint64_t db = make_desc(xt + (step >> 2) * 2048, 16, 1024) +
                              (uint64_t)(((step & 3) * 32) >> 4);
          const uint32_t acc = step == 0 ? 0u : 1u;
          const uint32_t acol = tmem_u + kColA + (slot * 8 + step) * 16;
          umma_f16_ts(dcol, acol, db, idesc, acc);
          umma_f16_ts(dcol + 16, acol + 8, db, idesc, acc);
          if (!EXACT) umma_f16_ts(dcol + 32, tmem_u + kColOnes, db, idesc, acc);
        }
      };
      tc_fence_after();
      if (elect_one()) issue(0, 5);
      __syncwarp();
      // What stage j + 1 needs is probed while the MMAs just issued run (a wait costs ~100
      // cycles even when the phase is complete).  The probe must not block: the commit of
      // stage j below is what lets the conversion of stage j + 2 start.
      bool ready = true;
      if (j + 1 < nst) {
        ready = mbar_test(raw_full(sn), phase_n);
        ready &= mbar_test(a_full(slot_n), slot_phase_n);
        // D[par ^ 1] was last used by stage j - 1: its sums must have been folded
        if (j >= 1) ready &= mbar_test(d_empty(par ^ 1), (uint32_t)((((j + 1) >> 1) - 1) & 1));
        ready = __all_sync(0xffffffffu, ready);
      }
      if (elect_one()) {
        issue(6, 7);
        umma_commit(a_empty(slot));  // A slot free again
        umma_commit(done(par));      // D[par] complete
        umma_commit(raw_empty(s));   // x tile of the stage read
      }
      __syncwarp();
      if (!ready) {
        ok = mbar_wait(raw_full(sn), phase_n, &s_abort, 11);
        if (ok) ok = mbar_wait(a_full(slot_n), slot_phase_n, &s_abort, 12);
        if (ok && j >= 1)
          ok = mbar_wait(d_empty(par ^ 1), (uint32_t)((((j + 1) >> 1) - 1) & 1), &s_abort, 13);
        ok = __all_sync(0xffffffffu, ok);
      }
      s = sn;
      ring_phase = phase_n;
      slot = slot_n;
      slot_phase = slot_phase_n;
    }
  } else if (warp >= kFoldWarp0) {
    // ------------------------------------------------------------------ fold
    const int q = warp - kFoldWarp0;  // == warp % 4: this warp's TMEM lane quarter
    const uint32_t lane_q = (uint32_t)(q * 32) << 16;
    // this thread's TMEM lane holds one output column per weight tile
    const int hp = lane >> 4, odd = (lane >> 3) & 1, gp = lane & 7;
    const int fold_word = min(word0 + 8 * q + gp, words - 1);
    const int col0 = 2 * hp + odd, col1 = 2 * (2 + hp) + odd;  // column inside the word
    const int nib0 = hp + 4 * odd, nib1 = (2 + hp) + 4 * odd;   // its nibble position
    float tot0[kNT], tot1[kNT];
#pragma unroll
    for (int m = 0; m < kNT; ++m) tot0[m] = tot1[m] = 0.f;

    const __half* sp = p.scales + (size_t)st_begin * p.N + fold_word * 8;
    const uint32_t* zp = p.qzeros + (size_t)st_begin * words + fold_word;
    // scale / zero of the next two groups in registers, of a few more in L2
    __half s0n = __float2half(0.f), s1n = s0n, s0n2 = s0n, s1n2 = s0n;
    uint32_t zwn = 0, zwn2 = 0;
    if (nst > 0) {
      s0n = __ldg(sp + col0);
      s1n = __ldg(sp + col1);
      zwn = __ldg(zp);
    }
    if (nst > 1) {
      s0n2 = __ldg(sp + (size_t)p.N + col0);
      s1n2 = __ldg(sp + (size_t)p.N + col1);
      zwn2 = __ldg(zp + words);
    }
    bool ok = true;
    for (int j = 0; j < nst && ok; ++j) {
      const int b = j & 1;
      const float s0 = __half2float(s0n), s1 = __half2float(s1n);
      const uint32_t zw = zwn;
      s0n = s0n2;
      s1n = s1n2;
      zwn = zwn2;
      if (j + 2 < nst) {
        s0n2 = __ldg(sp + (size_t)(j + 2) * p.N + col0);
        s1n2 = __ldg(sp + (size_t)(j + 2) * p.N + col1);
        zwn2 = __ldg(zp + (size_t)(j + 2) * words);
        if (odd == 0 && hp == 0) {
          const int jp = min(j + 6, nst - 1);
          asm volatile("prefetch.global.L2 [%0];" ::"l"(sp + (size_t)jp * p.N));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(zp + (size_t)jp * words));
        }
      }
      // odd half-quarters hold nibbles kept in place (16 q), so their zero point is 16 z
      const float zf = hp ? 16.f : 1.f;
      const float z0 = zf * (float)((zw >> (4 * nib0)) & 0xF);
      const float z1 = zf * (float)((zw >> (4 * nib1)) & 0xF);
      ok = mbar_wait(done(b), (uint32_t)((j >> 1) & 1), &s_abort, 14);
      if (!ok) break;
      tc_fence_after();
      const uint32_t dcol = tmem + lane_q + kColD + b * 48;
#pragma unroll
      for (int th = 0; th < 2; ++th) {
        uint32_t d0[8], d1[8], dx[8];
        tmem_ld8(dcol + th * 8, d0);
        tmem_ld8(dcol + 16 + th * 8, d1);
        if (!EXACT) tmem_ld8(dcol + 32 + th * 8, dx);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (th == 1) {
          // one arrival per warp: 128 arrivals on one shared-memory word serialise
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(d_empty(b));
        }
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          if (EXACT) {
            tot0[th * 8 + m] = fmaf(s0, __uint_as_float(d0[m]), tot0[th * 8 + m]);
            tot1[th * 8 + m] = fmaf(s1, __uint_as_float(d1[m]), tot1[th * 8 + m]);
          } else {
            const float xs = __uint_as_float(dx[m]);
            tot0[th * 8 + m] = fmaf(s0, fmaf(-z0, xs, __uint_as_float(d0[m])), tot0[th * 8 + m]);
            tot1[th * 8 + m] = fmaf(s1, fmaf(-z1, xs, __uint_as_float(d1[m])), tot1[th * 8 + m]);
          }
        }
      }
    }
    // ---- partial tile to shared memory: red[token][column of the slab] (the ring is idle:
    //      the last done implies every stage was converted and read by the tensor core) ----
    if (ok) {
      const float f = EXACT ? 1.f : (hp ? 1048576.f : 16777216.f);  // undo 2^-20 / 2^-24
      const int nl0 = 64 * q + 8 * gp + col0, nl1 = 64 * q + 8 * gp + col1;
#pragma unroll
      for (int m = 0; m < kNT; ++m) {
        red[m * kTsRedPitch + nl0] = tot0[m] * f;
        red[m * kTsRedPitch + nl1] = tot1[m] * f;
      }
    }
  } else {
    // ------------------------------------------------------------------ conversion warps
    // Warp (q, h, par): TMEM lane quarter q, steps 4 h .. 4 h + 3 of the stages of parity par.
    // A warp's own chain of waits, loads, unpack and TMEM stores takes longer than a stage
    // lasts; with the two parities on different warps the chains of consecutive stages overlap.
    const int g = lane >> 2, t = lane & 3;
    const int q = warp & 3, h = (warp >> 2) & 1, par = warp >> 3;
    const uint32_t lane_q = (uint32_t)(q * 32) << 16;
    // raw tile as TMA leaves it: row k at k * 128, 16-byte chunk c at position c ^ (k % 8).
    // This lane reads word 8 q + g of rows 16 step + 4 t + rr.
    const int chunk_id = 2 * q + (g >> 2);
    uint32_t off[4];
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
      const int row = 4 * t + rr;
      off[rr] = (uint32_t)(row * 128 + ((chunk_id ^ (row & 7)) << 4) + (g & 3) * 4);
    }
    const int conv_word = min(word0 + 8 * q + g, words - 1);

    if (!EXACT && h == 0 && par == 0) {
      // constant A tile: every k slot of every lane = 2^-24 (fp16 subnormal 0x0001); complete
      // before this warp's first arrival on a_full[0]
      tmem_st_16x256b(tmem + lane_q + kColOnes, 0x00010001u, 0x00010001u, 0x00010001u, 0x00010001u);
      tmem_st_16x256b(tmem + lane_q + (16u << 16) + kColOnes, 0x00010001u, 0x00010001u,
                      0x00010001u, 0x00010001u);
    }
    uint32_t zw_n = 0;
    if (EXACT && par < nst) zw_n = __ldg(p.qzeros + (size_t)(st_begin + par) * words + conv_word);

    bool ok = true;
    for (int j = par; j < nst && ok; j += 2) {
      const int s = j % kRing;
      const uint32_t wsm = smem_base + s * kTsStageBytes;
      // EXACT: zero registers of this thread's packed word for the group (= stage)
      __half2 zu[4], zv[4];
      if (EXACT) {
        const uint32_t zw = zw_n;
        if (j + 2 < nst) zw_n = __ldg(p.qzeros + (size_t)(st_begin + j + 2) * words + conv_word);
        const uint32_t uz = prmt(zw, zw, 0x1010), vz = prmt(zw, zw, 0x3232);
        const __half2 m16 = __float2half2_rn(-0.0625f);
        zu[0] = as_half2(lop3_and_or(uz, 0x000F000Fu, 0x64006400u));
        zv[0] = as_half2(lop3_and_or(vz, 0x000F000Fu, 0x64006400u));
        zu[2] = as_half2(lop3_and_or(uz >> 8, 0x000F000Fu, 0x64006400u));
        zv[2] = as_half2(lop3_and_or(vz >> 8, 0x000F000Fu, 0x64006400u));
        zu[1] = __hmul2(as_half2(lop3_and_or(uz, 0x00F000F0u, 0x64006400u)), m16);
        zv[1] = __hmul2(as_half2(lop3_and_or(vz, 0x00F000F0u, 0x64006400u)), m16);
        zu[3] = __hmul2(as_half2(lop3_and_or(uz >> 8, 0x00F000F0u, 0x64006400u)), m16);
        zv[3] = __hmul2(as_half2(lop3_and_or(vz >> 8, 0x00F000F0u, 0x64006400u)), m16);
      }
      ok = mbar_wait(raw_full(s), (uint32_t)((j / kRing) & 1), &s_abort, 15);
      if (!ok) break;
      // all four steps' packed words first: the loads must not queue up behind tcgen05.st
      uint32_t w[4][4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t rowA = wsm + (16 * (4 * h + e)) * 128;
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) w[e][rr] = lds32(rowA + off[rr]);
      }
      // the MMAs of stage j - 3 must have read this slot of the A ring
      const int slot = j % kASlots;
      if (j >= kASlots)
        ok = mbar_wait(a_empty(slot), (uint32_t)((j / kASlots - 1) & 1), &s_abort, 16);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int sp = 0; sp < 2; ++sp) {
        // fragments of two steps: frag[hq][4 * (2 e + tile) + k] -- the two tiles of a step and
        // two consecutive steps are adjacent column groups of the A ring, so one x4 store per
        // half-quarter writes all four
        uint32_t frag[2][16];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t* ww = w[2 * sp + e];
          const uint32_t u0 = prmt(ww[0], ww[1], 0x5410), v0 = prmt(ww[0], ww[1], 0x7632);
          const uint32_t u1 = prmt(ww[2], ww[3], 0x5410), v1 = prmt(ww[2], ww[3], 0x7632);
          const uint32_t u0h = u0 >> 8, v0h = v0 >> 8, u1h = u1 >> 8, v1h = v1 >> 8;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t mask = (i & 1) ? 0x00F000F0u : 0x000F000Fu;
            const uint32_t su0 = (i & 2) ? u0h : u0, sv0 = (i & 2) ? v0h : v0;
            const uint32_t su1 = (i & 2) ? u1h : u1, sv1 = (i & 2) ? v1h : v1;
            uint32_t r0, r1, r2, r3;  // (col 2i: k 4t..4t+1 | 4t+2..4t+3), (col 2i+1: same)
            if (EXACT) {
              const uint32_t e0 = lop3_and_or(su0, mask, 0x64006400u);
              const uint32_t e1 = lop3_and_or(su1, mask, 0x64006400u);
              const uint32_t e2 = lop3_and_or(sv0, mask, 0x64006400u);
              const uint32_t e3 = lop3_and_or(sv1, mask, 0x64006400u);
              if (i & 1) {
                const __half2 r16 = __float2half2_rn(0.0625f);
                r0 = as_u32(__hfma2(as_half2(e0), r16, zu[i]));
                r1 = as_u32(__hfma2(as_half2(e1), r16, zu[i]));
                r2 = as_u32(__hfma2(as_half2(e2), r16, zv[i]));
                r3 = as_u32(__hfma2(as_half2(e3), r16, zv[i]));
              } else {
                r0 = as_u32(__hsub2(as_half2(e0), zu[i]));
                r1 = as_u32(__hsub2(as_half2(e1), zu[i]));
                r2 = as_u32(__hsub2(as_half2(e2), zv[i]));
                r3 = as_u32(__hsub2(as_half2(e3), zv[i]));
              }
            } else {
              r0 = su0 & mask;
              r1 = su1 & mask;
              r2 = sv0 & mask;
              r3 = sv1 & mask;
            }
            // half-quarter i & 1 of this warp's lanes, weight tile i >> 1
            const int c = 4 * (2 * e + (i >> 1));
            frag[i & 1][c] = r0;
            frag[i & 1][c + 1] = r1;
            frag[i & 1][c + 2] = r2;
            frag[i & 1][c + 3] = r3;
          }
        }
        const uint32_t a_slot = tmem + lane_q + kColA + (slot * 8 + 4 * h + 2 * sp) * 16;
        tmem_st_16x256b_x4(a_slot, frag[0]);
        tmem_st_16x256b_x4(a_slot + (16u << 16), frag[1]);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      // every lane's TMEM stores are complete and its reads of the stage were consumed; one
      // arrival per warp (hundreds of arrivals on one shared-memory word would serialise)
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(a_full(slot));
        mbar_arrive(raw_empty(s));
      }
    }
  }

  // ---- reduction over the cluster ranks through distributed shared memory ----
  tc_fence_before();
  __syncthreads();
  if (S > 1) cluster.sync();  // every rank's partial tile is in its shared memory
  pdl_wait();  // long since satisfied; orders this thread's writes of `out` after the earlier kernel
  if (!s_abort) {
    constexpr int kUnits = kTsBN / 8;
    const int ubeg = (rank * kUnits) / S, uend = ((rank + 1) * kUnits) / S;
    const int nun = uend - ubeg;
    const int n_slab = blockIdx.y * kTsBN;
    for (int idx = tid; idx < nun * kNT; idx += kTsThreads) {
      const int u = ubeg + idx % nun, m = idx / nun;
      const int n = n_slab + u * 8;
      if (m >= p.M || n >= p.N) continue;
      float v[8];
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) v[jj] = 0.f;
      for (int rk = 0; rk < S; ++rk) {
        const float* peer = cluster.map_shared_rank(red, rk) + m * kTsRedPitch + u * 8;
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
  }
  if (S > 1) cluster.sync();  // peers are done reading this CTA's shared memory

  // ---- teardown ----
  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                 "r"((uint32_t)kTmemColsTs)
                 : "memory");
  }
}

template <bool EXACT>
int launch_ts(const CUtensorMap& map_w, const CUtensorMap& map_x, const TsParams& p,
              cudaStream_t stream) {
  static std::atomic<bool> attr_done[64];  // zero-initialised; setting the attribute twice is harmless
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return AWQ_B200_ERR_DEVICE;
  auto kernel = gemm_ts_kernel<EXACT>;
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTsSmemBytes) !=
        cudaSuccess)
      return AWQ_B200_ERR_LAUNCH;
    attr_done[dev] = true;
  }
  const int slabs = (p.N + kTsBN - 1) / kTsBN;
  const int KT = p.K / kTsBK;
  // cluster size (K split): only when the slabs alone leave SMs idle (one CTA per SM), and only
  // as large as lets every cluster of the grid be resident at once.  A cluster must find all its
  // SMs free inside one GPC: with 18 - 20 SMs per GPC only two clusters of 7 or three of 5 fit,
  // and a grid that needs more of them runs in two waves (measured at M = 16: K 8192 x N 5120,
  // 20 slabs, 25.2 us with clusters of 7; K 8192 x N 7392, 29 slabs, 28.9 us with clusters of 5).
  const int slots = sm_count();
  int S = 1;
  if (slabs < slots) {
    S = slots / slabs;
    S = S > 8 ? 8 : S;
    while (S > 1 && KT / S < 4) --S;
    static std::atomic<int> resident[64][9];  // zero-initialised: not asked yet
    while (S > 1 && resident_clusters(kernel, S, kTsThreads, kTsSmemBytes, resident[dev]) < slabs) --S;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(S, slabs, 1);
  cfg.blockDim = dim3(kTsThreads, 1, 1);
  cfg.dynamicSmemBytes = kTsSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = add_pdl_attribute(attr, 1);
  if (cudaLaunchKernelEx(&cfg, kernel, map_w, map_x, p) != cudaSuccess) {
    cudaGetLastError();
    return AWQ_B200_ERR_LAUNCH;
  }
  return AWQ_B200_OK;
}

}  // namespace

bool gemm_ts_supported(int M, int N, int K, int group) {
  // N % 32: 16-byte TMA row pitch of the packed weights; K % 128: whole stages
  return M >= 1 && M <= kNT && N % 32 == 0 && K % kTsBK == 0 && group == 128;
}

int launch_gemm_ts(const __half* x, const uint32_t* qweight, const __half* scales,
                   const uint32_t* qzeros, const __half* bias, __half* out, int M, int N, int K,
                   int group, bool exact, cudaStream_t stream) {
  if (!gemm_ts_supported(M, N, K, group)) return AWQ_B200_ERR_SHAPE;
  CUtensorMap map_w, map_x;
  // packed weights [K rows][N / 8 words], box [128 rows x 32 words], 128-byte swizzle
  if (int rc = encode_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_INT32, qweight, (uint64_t)(N / kPack),
                             (uint64_t)K, (uint64_t)(N / kPack) * 4, kTsBN / kPack, kTsBK,
                             CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  // activations [M rows][K], box [16 tokens x 64 k] (rows past M read as zero), 128-byte swizzle
  if (int rc = encode_map_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x, (uint64_t)K, (uint64_t)M,
                             (uint64_t)K * 2, 64, kNT, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  TsParams p{scales, qzeros, bias, out, M, N, K};
  return exact ? launch_ts<true>(map_w, map_x, p, stream) : launch_ts<false>(map_w, map_x, p, stream);
}

int ts_device_status(int* out, int clear) { return read_tc_status(out, clear); }

}  // namespace awq
