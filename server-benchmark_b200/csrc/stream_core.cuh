// Weight-streaming core shared by the dense small-M GEMM and the grouped MoE GEMMs.
//
// One CTA (4 warps) produces a [8*MT tokens] x [256 columns] fp32 tile of
//   D[n, m] = sum_k W[k, n] * x[m, k]
// over a range of 128-row stages: the int4 weights are the 16-row A operand of
// mma.sync.m16n8k16, the (padded) tokens the 8-wide B operand.
//
//   * Stage = 128 weight rows x 128 B (32 packed words = 256 columns) + 8*MT rows of x,
//     brought in by a 3-deep cp.async ring.  The ring belongs to one warp group (4 warps, 128
//     threads) that synchronises on its own named barrier, so several independent warp groups
//     can share a CTA.
//   * Warp w owns columns [64 w, 64 w + 64) of the slab; lane (g = lane / 4, t = lane % 4) owns
//     packed word g of those 8 words and rows 4t .. 4t+3 of every 16-row step.  The MMA's k
//     slots (2t, 2t+1, 2t+8, 2t+9) are mapped to those four rows -- a sum over k does not care
//     about the order -- so no data moves between lanes and the matching x values are one
//     8-byte shared-memory load.
//
// Register-only unpack (AWQ order): the low 16 bits of a word hold columns 0,2,4,6 and the
// high 16 bits columns 1,3,5,7.  prmt pairs the low halves of two rows (k, k+1) into one
// register u and the high halves into v; (u >> 4i) & 0x000F000F is then the (k, k+1) pair of
// column 2i -- one A-fragment register per AND.  Odd i use the mask 0x00F000F0 without a
// shift; the factor 16 is folded into the column's scale.
//
// Two conversions are compiled:
//   FAST   the masked nibbles are used as fp16 subnormals (value q * 2^-24, exact); the zero
//          point is applied per group as  acc - z * sum_k x  (the sum comes from one extra MMA
//          against a constant fragment) and 2^24 * s multiplies the fp32 group sum.
//   EXACT  nibbles become 1024 + q (OR 0x6400), the zero point is subtracted in fp16 (exact)
//          before the MMA; the scale again multiplies the fp32 group sum.
// Both accumulate every group in fp32 and apply the fp16 scale in fp32.
//
// RP (repacked weights, dequantize.cu::repack_kernel): the four prmt results (u, v of rows
// k, k+1 and of rows k+2, k+3) of every (row quad, word column) are stored as one 16-byte unit,
// [K/4][N/8][4] words.  A stage is then copied as it lies (512 contiguous bytes per row quad)
// and a lane's four registers come from one conflict-free ld.shared.v4: the pairing prmts and
// three of four shared-memory loads leave the loop.
//
// Shared-memory layout of a weight stage: row r (128 B) at r * 128, its 16-byte chunk c stored
// at chunk position c ^ (2 * ((r / 4) % 4) + r % 2) -- conflict-free both for the 16-byte
// cp.async writes and for the 4-byte fragment reads.  x stage: [8 MT rows][128 + 16 halves].
#pragma once

#include "common.cuh"

namespace awq {
namespace stream {

constexpr int kBN = 256;      // columns per CTA slab
constexpr int kBK = 128;      // weight rows per stage
constexpr int kThreads = 128;
constexpr int kWStageBytes = kBK * (kBN / kPack) * 4;  // 16384
constexpr int kXPitch = kBK + 16;                      // halves (row pitch = 8 words mod 32)
constexpr int kRedPitch = kBN + 8;                     // floats
constexpr int kGroupThreads = 128;  // one warp group

template <int MT>
struct Cfg {
  // MT = 2 trades the third stage for a fourth resident CTA per SM (more warps to hide latency)
  static constexpr int kStages = MT <= 2 ? 2 : 3;
  static constexpr int kStageBytes = kWStageBytes + MT * 8 * kXPitch * 2;
  static constexpr int kPipeBytes = kStages * kStageBytes;
  static constexpr int kRedBytes = MT * 8 * kRedPitch * 4;
  static constexpr int kSmemBytes = kPipeBytes > kRedBytes ? kPipeBytes : kRedBytes;
};

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
// barrier among the 128 threads of warp group `wg` (barrier 0 stays __syncthreads)
__device__ __forceinline__ void group_sync(int wg) {
  asm volatile("bar.sync %0, %1;" ::"r"(wg + 1), "n"(kGroupThreads) : "memory");
}
__device__ __forceinline__ uint32_t row_swizzle(int row) {
  return (uint32_t)((((row >> 2) & 3) << 1) | (row & 1));
}

// What one thread needs to know about the operands of its CTA tile.
template <int MT>
struct TileSrc {
  // producer side: this thread copies 16-byte chunk (tid & 7) of weight rows (tid >> 3) + 16 i
  const uint32_t* wsrc;   // address of that chunk in weight row 0 of the matrix
  bool wvalid;            // false: chunk lies past the N edge -> zero fill
  size_t wrow_words;      // weight row pitch in words
  // x rows (tid >> 4) + 8 j, 16-byte chunk (tid & 15) of the stage's 128 columns
  const __half* xsrc[MT];  // address of k = 0 of that chunk (row start + (tid & 15) * 8)
  bool xvalid[MT];
  // consumer side: scales / zeros of this lane's packed word column
  const uint32_t* zsrc;   // qzeros + column, group 0
  const uint4* ssrc;      // scales (as 8-half vectors) + column, group 0
  size_t zpitch;          // words per group row
  size_t spitch;          // uint4 per group row
};

// Runs stages [st_begin, st_begin + nst) and leaves the fp32 tile in `tot`:
//   tot[mt][i][0], [1] = column 2i   of this lane's word, tokens 8 mt + 2t, 8 mt + 2t + 1
//   tot[mt][i][2], [3] = column 2i+1 of this lane's word, same tokens
// GROUP is the quantisation group size when known at compile time (128: loops fully
// unrolled) or 0 to take it from `group` at run time (32 / 64 / 128).
// `tid` is the thread's index inside its warp group `wg`.
template <int MT, bool EXACT, int GROUP, bool RP = false>
__device__ __forceinline__ void mainloop(const TileSrc<MT>& src, uint32_t smem_base, int tid,
                                         int wg, int st_begin, int nst, int group, int ngroups,
                                         float (&tot)[MT][4][4]) {
  constexpr int STAGES = Cfg<MT>::kStages;
  constexpr int STAGE = Cfg<MT>::kStageBytes;
  const int lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  auto issue_w = [&](int st, int buf) {
    const uint32_t wbase = smem_base + buf * STAGE;
    const int k0 = st * kBK;
    if (RP) {
      // repacked weights: row quad q of the stage = 32 word columns x 16 B, copied as it lies;
      // this thread: 16-byte chunk of column tid % 32, quads tid / 32 + 4 i
      const uint32_t* s0 = src.wsrc + (size_t)(k0 / 4 + (tid >> 5)) * src.wrow_words;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        cp_async16(wbase + (tid + 128 * i) * 16, s0 + (size_t)(4 * i) * src.wrow_words, src.wvalid);
    } else {
      const int chunk = tid & 7, rbase = tid >> 3;
      const uint32_t* s0 = src.wsrc + (size_t)k0 * src.wrow_words;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = rbase + 16 * i;
        cp_async16(wbase + row * 128 + ((chunk ^ row_swizzle(row)) << 4),
                   s0 + (size_t)row * src.wrow_words, src.wvalid);
      }
    }
  };
  auto issue_x = [&](int st, int buf) {
    const uint32_t xbase = smem_base + buf * STAGE + kWStageBytes;
    const int k0 = st * kBK;
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      const int row = (tid >> 4) + 8 * j, ch = tid & 15;
      cp_async16(xbase + (row * kXPitch + ch * 8) * 2, src.xsrc[j] + k0, src.xvalid[j]);
    }
  };

  const int chunk_id = 2 * warp + (g >> 2);
  const uint32_t offA = ((chunk_id ^ (2 * t)) << 4) + (g & 3) * 4;      // even rows
  const uint32_t offB = ((chunk_id ^ (2 * t + 1)) << 4) + (g & 3) * 4;  // odd rows
  const int spg = GROUP ? GROUP / 16 : group / 16;   // 16-row steps per quantisation group
  const int gps = GROUP ? kBK / GROUP : kBK / group;  // groups per stage

#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) tot[mt][i][c] = 0.f;

  // scale / zero registers of the next group (prefetched one group ahead)
  uint32_t zw_n = 0;
  uint4 sc_n = make_uint4(0, 0, 0, 0);
  if (nst > 0) {
    const int grp = st_begin * gps;
    zw_n = __ldg(src.zsrc + (size_t)grp * src.zpitch);
    sc_n = __ldg(src.ssrc + (size_t)grp * src.spitch);
  }

  // Prologue: the packed weights of the first stages are requested before pdl_wait (no kernel
  // writes them), the activations after it.  All those weight copies land in the first
  // commit group, so the first iteration waits for the whole prologue's weights.
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s)
    if (s < nst) issue_w(st_begin + s, s);
  pdl_wait();
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < nst) issue_x(st_begin + s, s);
    cp_async_commit();
  }

  for (int it = 0; it < nst; ++it) {
    cp_async_wait<STAGES - 2>();
    group_sync(wg);
    {
      const int nx = it + STAGES - 1;
      if (nx < nst) {
        issue_w(st_begin + nx, nx % STAGES);
        issue_x(st_begin + nx, nx % STAGES);
      }
      cp_async_commit();
    }
    const uint32_t wsm = smem_base + (it % STAGES) * STAGE;
    const uint32_t xsm = wsm + kWStageBytes;

    for (int gi = 0; gi < gps; ++gi) {
      const int grp = (st_begin + it) * gps + gi;
      const uint32_t zw = zw_n;
      const uint4 sc = sc_n;
      {
        const int gn = min(grp + 1, ngroups - 1);
        zw_n = __ldg(src.zsrc + (size_t)gn * src.zpitch);
        sc_n = __ldg(src.ssrc + (size_t)gn * src.spitch);
      }

      float acc[MT][4][4];
      float xs[MT][4];
      const float kZero4[4] = {0.f, 0.f, 0.f, 0.f};

      // EXACT: per-column zero registers, as (z, z) pairs matching the (k, k+1) pairs.
      __half2 zu[4], zv[4];
      if (EXACT) {
        const uint32_t uz = prmt(zw, zw, 0x1010), vz = prmt(zw, zw, 0x3232);
        const __half2 m16 = __float2half2_rn(-0.0625f);
        zu[0] = as_half2(lop3_and_or(uz, 0x000F000Fu, 0x64006400u));
        zv[0] = as_half2(lop3_and_or(vz, 0x000F000Fu, 0x64006400u));
        zu[2] = as_half2(lop3_and_or(uz >> 8, 0x000F000Fu, 0x64006400u));
        zv[2] = as_half2(lop3_and_or(vz >> 8, 0x000F000Fu, 0x64006400u));
        // odd i: nibble kept in place (16 q); -(1024 + 16 z) / 16 = -(64 + z), exact
        zu[1] = __hmul2(as_half2(lop3_and_or(uz, 0x00F000F0u, 0x64006400u)), m16);
        zv[1] = __hmul2(as_half2(lop3_and_or(vz, 0x00F000F0u, 0x64006400u)), m16);
        zu[3] = __hmul2(as_half2(lop3_and_or(uz >> 8, 0x00F000F0u, 0x64006400u)), m16);
        zv[3] = __hmul2(as_half2(lop3_and_or(vz >> 8, 0x00F000F0u, 0x64006400u)), m16);
      }

#pragma unroll
      for (int s2 = 0; s2 < (GROUP ? GROUP / 16 : 8); ++s2) {
        if (!GROUP && s2 >= spg) break;
        const int s = gi * spg + s2;
        uint32_t u0, v0, u1, v1;
        if (RP) {
          // the row pairs were formed when the weights were repacked: one 16-byte load
          const uint4 qd = lds128(wsm + ((4 * s + t) * 32 + 8 * warp + g) * 16);
          u0 = qd.x;
          v0 = qd.y;
          u1 = qd.z;
          v1 = qd.w;
        } else {
          const uint32_t rowA = wsm + (16 * s + 4 * t) * 128;
          const uint32_t w0 = lds32(rowA + offA);
          const uint32_t w1 = lds32(rowA + 128 + offB);
          const uint32_t w2 = lds32(rowA + 2 * 128 + offA);
          const uint32_t w3 = lds32(rowA + 3 * 128 + offB);
          u0 = prmt(w0, w1, 0x5410);
          v0 = prmt(w0, w1, 0x7632);
          u1 = prmt(w2, w3, 0x5410);
          v1 = prmt(w2, w3, 0x7632);
        }
        uint32_t b0[MT], b1[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint2 xv = lds64(xsm + ((mt * 8 + g) * kXPitch + 16 * s + 4 * t) * 2);
          b0[mt] = xv.x;
          b1[mt] = xv.y;
        }
        const uint32_t u0h = u0 >> 8, v0h = v0 >> 8, u1h = u1 >> 8, v1h = v1 >> 8;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t mask = (i & 1) ? 0x00F000F0u : 0x000F000Fu;
          const uint32_t su0 = (i & 2) ? u0h : u0, sv0 = (i & 2) ? v0h : v0;
          const uint32_t su1 = (i & 2) ? u1h : u1, sv1 = (i & 2) ? v1h : v1;
          uint32_t a[4];
          if (EXACT) {
            const uint32_t r0 = lop3_and_or(su0, mask, 0x64006400u);
            const uint32_t r1 = lop3_and_or(sv0, mask, 0x64006400u);
            const uint32_t r2 = lop3_and_or(su1, mask, 0x64006400u);
            const uint32_t r3 = lop3_and_or(sv1, mask, 0x64006400u);
            if (i & 1) {
              const __half2 r16 = __float2half2_rn(0.0625f);
              a[0] = as_u32(__hfma2(as_half2(r0), r16, zu[i]));
              a[1] = as_u32(__hfma2(as_half2(r1), r16, zv[i]));
              a[2] = as_u32(__hfma2(as_half2(r2), r16, zu[i]));
              a[3] = as_u32(__hfma2(as_half2(r3), r16, zv[i]));
            } else {
              a[0] = as_u32(__hsub2(as_half2(r0), zu[i]));
              a[1] = as_u32(__hsub2(as_half2(r1), zv[i]));
              a[2] = as_u32(__hsub2(as_half2(r2), zu[i]));
              a[3] = as_u32(__hsub2(as_half2(r3), zv[i]));
            }
          } else {
            a[0] = su0 & mask;
            a[1] = sv0 & mask;
            a[2] = su1 & mask;
            a[3] = sv1 & mask;
          }
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            // first step of a group starts from zero: no accumulator initialisation needed
            if (s2 == 0) mma16816(acc[mt][i], a, b0[mt], b1[mt], kZero4);
            else mma16816(acc[mt][i], a, b0[mt], b1[mt], acc[mt][i]);
          }
        }
        if (!EXACT) {
          const uint32_t ones[4] = {0x00010001u, 0x00010001u, 0x00010001u, 0x00010001u};
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            if (s2 == 0) mma16816(xs[mt], ones, b0[mt], b1[mt], kZero4);
            else mma16816(xs[mt], ones, b0[mt], b1[mt], xs[mt]);
          }
        }
      }

      // ---- fold the group: tot += scale * (acc - zero * sum_x) ----
      const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 sf = __half22float2(as_half2(scw[i]));  // scales of columns 2i, 2i+1
        const float sa = sf.x, sb = sf.y;
        float za = 0.f, zb = 0.f;
        if (!EXACT) {
          // zero nibbles -> float through the 2^23 mantissa trick (no int-to-float convert);
          // odd i carry the factor 16 of the in-place nibble: take the zero as 16 z as well.
          // The common factor 2^24 (2^20 for odd i) is applied once after the K loop.
          const uint32_t zsa = (i & 1) ? (zw >> (4 * i - 4)) & 0xF0u : (zw >> (4 * i)) & 0xFu;
          const uint32_t zsb = (i & 1) ? (zw >> (4 * i + 12)) & 0xF0u : (zw >> (4 * i + 16)) & 0xFu;
          za = __uint_as_float(zsa | 0x4B000000u) - 8388608.f;
          zb = __uint_as_float(zsb | 0x4B000000u) - 8388608.f;
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          if (EXACT) {
            tot[mt][i][0] = fmaf(sa, acc[mt][i][0], tot[mt][i][0]);
            tot[mt][i][1] = fmaf(sa, acc[mt][i][1], tot[mt][i][1]);
            tot[mt][i][2] = fmaf(sb, acc[mt][i][2], tot[mt][i][2]);
            tot[mt][i][3] = fmaf(sb, acc[mt][i][3], tot[mt][i][3]);
          } else {
            tot[mt][i][0] = fmaf(sa, fmaf(-za, xs[mt][0], acc[mt][i][0]), tot[mt][i][0]);
            tot[mt][i][1] = fmaf(sa, fmaf(-za, xs[mt][1], acc[mt][i][1]), tot[mt][i][1]);
            tot[mt][i][2] = fmaf(sb, fmaf(-zb, xs[mt][0], acc[mt][i][2]), tot[mt][i][2]);
            tot[mt][i][3] = fmaf(sb, fmaf(-zb, xs[mt][1], acc[mt][i][3]), tot[mt][i][3]);
          }
        }
      }
    }
  }
  if (!EXACT) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) tot[mt][i][c] *= (i & 1) ? 1048576.f : 16777216.f;
  }
  cp_async_wait<0>();
  group_sync(wg);  // every warp of the group is done with the ring: the caller may reuse it
}

// Writes the register tile to shared memory as red[m][col] (pitch kRedPitch floats).
template <int MT>
__device__ __forceinline__ void store_tile(float* red, int tid, const float (&tot)[MT][4][4]) {
  const int lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int col = 64 * warp + 8 * g + 2 * i;
      const int m = mt * 8 + 2 * t;
      *reinterpret_cast<float2*>(red + m * kRedPitch + col) =
          make_float2(tot[mt][i][0], tot[mt][i][2]);
      *reinterpret_cast<float2*>(red + (m + 1) * kRedPitch + col) =
          make_float2(tot[mt][i][1], tot[mt][i][3]);
    }
}

}  // namespace stream
}  // namespace awq
