// Decode-size AWQ GEMM (M <= 16) on tcgen05 with the weights going registers -> TMEM.
//
//   D[n, m] = sum_k W[k, n] * x[m, k]          (the transposed product, as in stream_core.cuh)
//
// The int4 weights are unpacked in registers exactly as in the mma.sync streaming kernel (prmt
// pairs two rows, one AND per 32-bit pair, nibbles used as fp16 subnormals), but the fragments are
// not fed to mma.sync: they are written to tensor memory with tcgen05.st.16x256b and become the
// A operand (128 weight columns x 16 k) of tcgen05.mma.kind::f16; the activations are the small
// B operand ([16 tokens x 64 k] K-major, 128-byte swizzle) in shared memory.  The dequantised
// weights never touch shared memory and the 5th-generation tensor core does the arithmetic.
//
// The CTA is a pipeline of specialised warps joined by mbarrier rings (slab of 256 output
// columns = two 128-lane A tiles; stage = 128 weight rows = one quantisation group; K range
// split over a thread-block cluster as in gemm_stream.cu):
//
//   producer (1 thread)   TMA: packed weights [128 rows x 128 B] + x [16 tokens x 128 k] of a
//                         stage into a 5-deep shared-memory ring            raw_full / raw_empty
//   conversion (8 warps)  warp (q, p): TMEM lane quarter q, quarter-stages c = p and p + 2.
//                         Per quarter-stage (two 16-row steps): ld.shared -> unpack ->
//                         8 x tcgen05.st into A slot c                      a_full[c] / done0, done1
//   issue (1 warp)        converged warp, one elected lane: per 16-row step one MMA per A tile
//                         (weight tile 0, weight tile 1, constant tile) into the group
//                         accumulators D[b]; two tcgen05.commit per stage   done0, done1[b] / d_empty[b]
//   fold (4 warps)        warp q: tcgen05.ld its lanes of D[b];
//                         tot += scale * (acc - zero * sum_x) in fp32 registers
//
// The constant tile (every k slot = 2^-24) yields sum_k x per token in the same scaling as the
// weight tiles, so the zero point is applied per group without a separate reduction.
//
// Measured on B200 while building this kernel (cycles of the SM clock):
//   * a tcgen05.mma / tcgen05.commit issued by one lane that loops alone (the other 31 lanes of
//     its warp parked at a barrier) costs that lane 45 to 270 cycles depending on how its
//     operands are computed; issued from a converged warp under elect.sync with warp-uniform
//     operands it costs ~23 (M = 128, N = 16, K = 16, A in TMEM);
//   * a tcgen05.commit drains the tensor pipe (~75 cycles in which no MMA starts): with one
//     commit per A slot and per consumer the pipe spent half its time drained, hence two
//     commits per stage and barriers shared by every consumer of the same event;
//   * every mbarrier wait costs its warp ~100 cycles even when the phase is already complete.
// What bounds the kernel now is that TMEM holds only one stage of A next to the accumulators
// (256 columns per CTA, two CTAs per SM): conversion of stage j + 1 cannot start before the MMAs
// of stage j have read the slot, so conversion and MMA latencies add up instead of overlapping.
//
// TMEM columns (256 allocated, two CTAs per SM): D[2 buffers][3 tiles][16] = 96,
// A[4 quarter-stage slots][2 tiles][2 steps][8] = 128, constant tile 8.  Lane l of quarter q holds
// output column  64 q + 8 (l % 8) + 2 (2 tile + l / 16) + (l % 16) / 8  of the slab.
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
constexpr int kRing = 5;                        // stages in flight
constexpr int kTsWBytes = kTsBK * (kTsBN / kPack) * 4;  // 16384
constexpr int kTsXBytes = kNT * kTsBK * 2;              // 4096: two [16 x 64] tiles
constexpr int kTsStageBytes = kTsWBytes + kTsXBytes;    // 20480
constexpr int kTsRingBytes = kRing * kTsStageBytes;     // 102400
constexpr int kTsRedPitch = kTsBN + 8;                  // floats
constexpr int kTsBarBytes = 256;
constexpr int kTsSmemBytes = kTsRingBytes + kTsBarBytes + 1024;  // + alignment slack
constexpr int kCvWarps = 8, kFoldWarps = 4;
constexpr int kFoldWarp0 = kCvWarps, kIssueWarp = kCvWarps + kFoldWarps;
constexpr int kProducerWarp = kIssueWarp + 1;
constexpr int kTsThreads = 32 * (kProducerWarp + 1);  // 448
constexpr int kTmemColsTs = 256;
constexpr int kColD = 0;      // + buffer * 48 + tile * 16
constexpr int kColA = 96;     // + slot * 32 + tile * 16 + step * 8
constexpr int kColOnes = 224;
static_assert(kNT * kTsRedPitch * 4 <= kTsRingBytes, "partial tile must fit the idle ring");

struct TsParams {
  const __half* scales;
  const uint32_t* qzeros;
  const __half* bias;
  __half* out;
  int M, N, K;
};

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
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
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(
          tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

template <bool EXACT>
__global__ void __launch_bounds__(kTsThreads, 2)
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
  auto a_full = [&](int c) { return bar_base + 8 * (2 * kRing + c); };
  auto done0 = [&]() { return bar_base + 8 * (2 * kRing + 4); };
  auto done1 = [&](int b) { return bar_base + 8 * (2 * kRing + 5 + b); };
  auto d_empty = [&](int b) { return bar_base + 8 * (2 * kRing + 7 + b); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int words = p.N / kPack;
  const int word0 = blockIdx.y * (kTsBN / kPack);
  const int KT = p.K / kTsBK;
  const int st_begin = (int)(((long long)rank * KT) / S);
  const int st_end = (int)(((long long)(rank + 1) * KT) / S);
  const int nst = st_end - st_begin;

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < kRing; ++s) {
      mbar_init(raw_full(s), 1);
      mbar_init(raw_empty(s), kCvWarps);
    }
    for (int c = 0; c < 4; ++c)
      mbar_init(a_full(c), 4 * 32);  // the four warps (one per lane quarter) that fill slot c
    mbar_init(done0(), 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(done1(b), 1);
      mbar_init(d_empty(b), kFoldWarps * 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
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
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      bool ok = true;
      for (int j = 0; j < nst && ok; ++j) {
        const int s = j % kRing;
        if (j >= kRing) ok = mbar_wait(raw_empty(s), (uint32_t)((j / kRing - 1) & 1), &s_abort, 21);
        if (!ok) break;
        const uint32_t dst = smem_base + s * kTsStageBytes;
        const int k0 = (st_begin + j) * kTsBK;
        mbar_arrive_expect_tx(raw_full(s), kTsStageBytes);
        tma_load_2d(dst, &map_w, word0, k0, raw_full(s));
        tma_load_2d(dst + kTsWBytes, &map_x, k0, 0, raw_full(s));
        tma_load_2d(dst + kTsWBytes + 2048, &map_x, k0 + 64, 0, raw_full(s));
      }
    }
  } else if (warp == kIssueWarp) {
    // ------------------------------------------------------------------ MMA issue
    // The whole warp runs the loop and stays converged; one elected lane issues (see elect_one).
    // Two commits per stage: done0 after the first half (A slots 0, 1 free again) and done1[b]
    // at the end (A slots 2, 3 free, D[b] complete, x tile of the stage read).
    // D fp32, A/B fp16, both K-major, N = 16 tokens, M = 128 weight columns
    constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(kNT >> 3) << 17) | (8u << 24);
    // Operands of tcgen05 instructions live in uniform registers: keep everything they are
    // computed from provably warp-uniform (broadcast bases, wrapping counters instead of
    // divisions), otherwise every MMA pays for moving its operands across register files.
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
    const uint32_t ring_u = __shfl_sync(0xffffffffu, smem_base, 0);
    bool ok = true;
    int s = 0;
    uint32_t ring_phase = 0;
    for (int j = 0; j < nst && ok; ++j) {
      const int b = j & 1;
      if (j >= 2) ok = mbar_wait(d_empty(b), (uint32_t)(((j >> 1) - 1) & 1), &s_abort, 11);
      if (ok) ok = mbar_wait(raw_full(s), ring_phase, &s_abort, 12);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t xt = ring_u + s * kTsStageBytes + kTsWBytes;
      const uint32_t dcol = tmem_u + kColD + b * 48;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        // slot c converted (the constant tile was written before the first a_full[0])
        ok = mbar_wait(a_full(c), (uint32_t)(j & 1), &s_abort, 13);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int step = 2 * c + e;
            const uint64_t db = make_desc(xt + (step >> 2) * 2048, 16, 1024) +
                                (uint64_t)(((step & 3) * 32) >> 4);
            const uint32_t acc = step == 0 ? 0u : 1u;
            const uint32_t acol = tmem_u + kColA + c * 32 + e * 8;
            umma_f16_ts(dcol, acol, db, idesc, acc);
            umma_f16_ts(dcol + 16, acol + 16, db, idesc, acc);
            if (!EXACT) umma_f16_ts(dcol + 32, tmem_u + kColOnes, db, idesc, acc);
          }
          if (c == 1) umma_commit(done0());
          if (c == 3) umma_commit(done1(b));
        }
        __syncwarp();
      }
      if (++s == kRing) {
        s = 0;
        ring_phase ^= 1u;
      }
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
    __half s0n = __float2half(0.f), s1n = s0n;
    uint32_t zwn = 0;
    if (nst > 0) {
      s0n = __ldg(sp + col0);
      s1n = __ldg(sp + col1);
      zwn = __ldg(zp);
    }
    bool ok = true;
    for (int j = 0; j < nst && ok; ++j) {
      const int b = j & 1;
      const float s0 = __half2float(s0n), s1 = __half2float(s1n);
      const uint32_t zw = zwn;
      if (j + 1 < nst) {
        s0n = __ldg(sp + (size_t)(j + 1) * p.N + col0);
        s1n = __ldg(sp + (size_t)(j + 1) * p.N + col1);
        zwn = __ldg(zp + (size_t)(j + 1) * words);
      }
      // odd half-quarters hold nibbles kept in place (16 q), so their zero point is 16 z
      const float zf = hp ? 16.f : 1.f;
      const float z0 = zf * (float)((zw >> (4 * nib0)) & 0xF);
      const float z1 = zf * (float)((zw >> (4 * nib1)) & 0xF);
      ok = mbar_wait(done1(b), (uint32_t)((j >> 1) & 1), &s_abort, 14);
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
          tc_fence_before();
          mbar_arrive(d_empty(b));
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
    //      the last done1 implies every stage was converted and read by the tensor core) ----
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
    const int g = lane >> 2, t = lane & 3;
    const int q = warp & 3, par = warp >> 2;
    const uint32_t lane_q = (uint32_t)(q * 32) << 16;
    // raw tile as TMA leaves it: row r at r * 128, 16-byte chunk c at position c ^ (r % 8).
    // This lane reads word 8 q + g of rows 16 s + 4 t + rr.
    const int chunk_id = 2 * q + (g >> 2);
    uint32_t off[4];
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
      const int r = 4 * t + rr;
      off[rr] = (uint32_t)(r * 128 + ((chunk_id ^ (r & 7)) << 4) + (g & 3) * 4);
    }
    const int conv_word = min(word0 + 8 * q + g, words - 1);

    if (!EXACT && par == 0) {
      // constant A tile: every k slot of every lane = 2^-24 (fp16 subnormal 0x0001)
      tmem_st_16x256b(tmem + lane_q + kColOnes, 0x00010001u, 0x00010001u, 0x00010001u, 0x00010001u);
      tmem_st_16x256b(tmem + lane_q + (16u << 16) + kColOnes, 0x00010001u, 0x00010001u,
                      0x00010001u, 0x00010001u);
    }
    uint32_t zw_n = 0;
    if (EXACT && nst > 0) zw_n = __ldg(p.qzeros + (size_t)st_begin * words + conv_word);

    bool ok = true;
    for (int j = 0; j < nst && ok; ++j) {
      const int s = j % kRing;
      const uint32_t wsm = smem_base + s * kTsStageBytes;
      // EXACT: zero registers of this thread's packed word for the group (= stage)
      __half2 zu[4], zv[4];
      if (EXACT) {
        const uint32_t zw = zw_n;
        if (j + 1 < nst) zw_n = __ldg(p.qzeros + (size_t)(st_begin + j + 1) * words + conv_word);
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
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = par + 2 * cc;  // quarter-stage = A slot
        // slot c of the previous stage must have been read by the tensor core
        if (j >= 1) {
          if (cc == 0) {
            ok = mbar_wait(done0(), (uint32_t)((j - 1) & 1), &s_abort, 16);
          } else {
            ok = mbar_wait(done1((j - 1) & 1), (uint32_t)(((j - 1) >> 1) & 1), &s_abort, 17);
            // the previous stage is finished with: this warp's reads of its packed weights were
            // consumed by the conversion, the tensor core has read its x tile
            __syncwarp();
            if (ok && lane == 0) mbar_arrive(raw_empty((j - 1) % kRing));
          }
        }
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t rowA = wsm + (16 * (2 * c + e)) * 128;
          const uint32_t w0 = lds32(rowA + off[0]);
          const uint32_t w1 = lds32(rowA + off[1]);
          const uint32_t w2 = lds32(rowA + off[2]);
          const uint32_t w3 = lds32(rowA + off[3]);
          const uint32_t u0 = prmt(w0, w1, 0x5410), v0 = prmt(w0, w1, 0x7632);
          const uint32_t u1 = prmt(w2, w3, 0x5410), v1 = prmt(w2, w3, 0x7632);
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
            tmem_st_16x256b(tmem + lane_q + ((uint32_t)((i & 1) * 16) << 16) + kColA + c * 32 +
                                (i >> 1) * 16 + e * 8,
                            r0, r1, r2, r3);
          }
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        mbar_arrive(a_full(c));
      }
    }
  }

  // ---- reduction over the cluster ranks through distributed shared memory ----
  __syncthreads();
  cluster.sync();
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
      for (int r = 0; r < S; ++r) {
        const float* peer = cluster.map_shared_rank(red, r) + m * kTsRedPitch + u * 8;
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
  cluster.sync();

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
  static bool attr_done[64] = {false};
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
  // cluster size (K split): the one that needs the least time in units of a whole-K CTA,
  // rounds of 2 CTAs per SM times 1 / S; ties go to the smaller cluster
  const int slots = 2 * sm_count();
  int S = 1;
  double best = 1e30;
  for (int s = 1; s <= 8 && KT / s >= 4; ++s) {
    const int rounds = (slabs * s + slots - 1) / slots;
    const double cost = (double)rounds / s + 0.02 * s;
    if (cost < best) {
      best = cost;
      S = s;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(S, slabs, 1);
  cfg.blockDim = dim3(kTsThreads, 1, 1);
  cfg.dynamicSmemBytes = kTsSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
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

int ts_device_status(int* out) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return AWQ_B200_ERR_LAUNCH;
  *out = v;
  return AWQ_B200_OK;
}

}  // namespace awq
