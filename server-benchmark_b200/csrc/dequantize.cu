// awq_dequantize: W fp16 [K, N] = (q - z) * s.  Pure bandwidth: 0.5 B read and 2 B written
// per weight.  One thread owns one packed word column and walks kRows consecutive rows of it,
// so the zero word and the 8 scales are fetched once per kRows rows; each row costs one
// coalesced 4-byte load and one coalesced 16-byte store per thread (512 B per warp).
//
// Also holds the CUDA-core reference GEMM used for shapes the fast kernels do not take.
#include "common.cuh"

namespace awq {

namespace {

constexpr int kDqThreads = 128;
constexpr int kDqRows = 16;

__global__ void __launch_bounds__(kDqThreads)
dequantize_kernel(const uint32_t* __restrict__ qweight, const __half* __restrict__ scales,
                  const uint32_t* __restrict__ qzeros, __half* __restrict__ out, int K, int words,
                  int group) {
  const int c = blockIdx.x * kDqThreads + threadIdx.x;
  if (c >= words) return;
  const int k0 = blockIdx.y * kDqRows;
  const int k1 = min(k0 + kDqRows, K);
  const int N = words * kPack;
  int cur_group = -1;
  uint32_t zmagic[4];
  __half2 s2[4];
  if (group % kDqRows == 0 && k0 + kDqRows <= K) {
    // Whole chunk inside one group: issue all row loads first, then convert and store.
    const int g = k0 / group;
    unpack_word_magic(__ldg(qzeros + (size_t)g * words + c), zmagic);
    const uint4 sv = __ldg(reinterpret_cast<const uint4*>(scales + (size_t)g * N) + c);
    s2[0] = as_half2(sv.x);
    s2[1] = as_half2(sv.y);
    s2[2] = as_half2(sv.z);
    s2[3] = as_half2(sv.w);
    uint32_t w[kDqRows];
#pragma unroll
    for (int i = 0; i < kDqRows; ++i) w[i] = __ldcs(qweight + (size_t)(k0 + i) * words + c);
#pragma unroll
    for (int i = 0; i < kDqRows; ++i)
      __stcs(reinterpret_cast<uint4*>(out + (size_t)(k0 + i) * N) + c,
             dequant_word(w[i], zmagic, s2));
    return;
  }
  for (int k = k0; k < k1; ++k) {
    const int g = k / group;
    if (g != cur_group) {
      cur_group = g;
      unpack_word_magic(__ldg(qzeros + (size_t)g * words + c), zmagic);
      const uint4 sv = __ldg(reinterpret_cast<const uint4*>(scales + (size_t)g * N) + c);
      s2[0] = as_half2(sv.x);
      s2[1] = as_half2(sv.y);
      s2[2] = as_half2(sv.z);
      s2[3] = as_half2(sv.w);
    }
    const uint32_t w = __ldcs(qweight + (size_t)k * words + c);
    const uint4 o = dequant_word(w, zmagic, s2);
    __stcs(reinterpret_cast<uint4*>(out + (size_t)k * N) + c, o);
  }
}

// Reference GEMM on CUDA cores: one thread produces 8 adjacent outputs of one row of y.
constexpr int kGenThreads = 128;

__global__ void __launch_bounds__(kGenThreads)
gemm_generic_kernel(const __half* __restrict__ x, const uint32_t* __restrict__ qweight,
                    const __half* __restrict__ scales, const uint32_t* __restrict__ qzeros,
                    const __half* __restrict__ bias, __half* __restrict__ out, int M, int words,
                    int K, int group) {
  const int c = blockIdx.x * kGenThreads + threadIdx.x;
  const int m = blockIdx.y;
  if (c >= words) return;
  const int N = words * kPack;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  const __half* xr = x + (size_t)m * K;
  for (int g = 0; g * group < K; ++g) {
    const uint32_t zw = __ldg(qzeros + (size_t)g * words + c);
    float part[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) part[j] = 0.f;
    for (int kk = 0; kk < group; ++kk) {
      const int k = g * group + kk;
      const uint32_t w = __ldg(qweight + (size_t)k * words + c);
      const float xv = __half2float(__ldg(xr + k));
#pragma unroll
      for (int j = 0; j < 8; ++j)
        part[j] = fmaf(xv, (float)(nibble_of_col(w, j) - nibble_of_col(zw, j)), part[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      acc[j] = fmaf(part[j], __half2float(__ldg(scales + (size_t)g * N + c * 8 + j)), acc[j]);
  }
  __half o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float v = acc[j];
    if (bias != nullptr) v += __half2float(__ldg(bias + c * 8 + j));
    o[j] = __float2half_rn(v);
  }
  *reinterpret_cast<uint4*>(out + (size_t)m * N + c * 8) = *reinterpret_cast<uint4*>(o);
}

}  // namespace

int launch_dequantize(const uint32_t* qweight, const __half* scales, const uint32_t* qzeros,
                      __half* out, int K, int N, int group, cudaStream_t stream) {
  const int words = N / kPack;
  dim3 grid((words + kDqThreads - 1) / kDqThreads, (K + kDqRows - 1) / kDqRows);
  dequantize_kernel<<<grid, kDqThreads, 0, stream>>>(qweight, scales, qzeros, out, K, words,
                                                     group);
  return cudaGetLastError() == cudaSuccess ? AWQ_B200_OK : AWQ_B200_ERR_LAUNCH;
}

int launch_gemm_generic(const __half* x, const uint32_t* qweight, const __half* scales,
                        const uint32_t* qzeros, const __half* bias, __half* out, int M, int N,
                        int K, int group, cudaStream_t stream) {
  const int words = N / kPack;
  for (int m0 = 0; m0 < M; m0 += 32768) {
    const int rows = min(M - m0, 32768);
    dim3 grid((words + kGenThreads - 1) / kGenThreads, rows);
    gemm_generic_kernel<<<grid, kGenThreads, 0, stream>>>(x + (size_t)m0 * K, qweight, scales,
                                                          qzeros, bias, out + (size_t)m0 * N,
                                                          rows, words, K, group);
    if (cudaGetLastError() != cudaSuccess) return AWQ_B200_ERR_LAUNCH;
  }
  return AWQ_B200_OK;
}

// Load-time repack for the decode kernel (stream_core.cuh, RP): for every row quad and word
// column the four row-pair registers the unpack needs, as one 16-byte unit:
//   out[(kq * words + c) * 4 + {0, 1, 2, 3}] = { lo16(w0) | lo16(w1) << 16, hi16(w0) | hi16(w1) << 16,
//                                               lo16(w2) | lo16(w3) << 16, hi16(w2) | hi16(w3) << 16 }
// with w_r = qweight[(4 kq + r) * words + c].  Same size as qweight; a pure permutation of bits.
namespace {
__global__ void __launch_bounds__(256)
repack_kernel(const uint32_t* __restrict__ qweight, uint4* __restrict__ out, int quads, int words) {
  const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
  if (idx >= (long long)quads * words) return;
  const int kq = (int)(idx / words), c = (int)(idx % words);
  const uint32_t* src = qweight + (size_t)(4 * kq) * words + c;
  const uint32_t w0 = __ldg(src), w1 = __ldg(src + words), w2 = __ldg(src + 2 * (size_t)words),
                 w3 = __ldg(src + 3 * (size_t)words);
  out[idx] = make_uint4(prmt(w0, w1, 0x5410), prmt(w0, w1, 0x7632), prmt(w2, w3, 0x5410),
                        prmt(w2, w3, 0x7632));
}
}  // namespace

int launch_repack_qweight(const uint32_t* qweight, uint32_t* out, int K, int N,
                          cudaStream_t stream) {
  const int words = N / kPack, quads = K / 4;
  const long long total = (long long)quads * words;
  if (total == 0) return AWQ_B200_OK;
  repack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
      qweight, reinterpret_cast<uint4*>(out), quads, words);
  return cudaGetLastError() == cudaSuccess ? AWQ_B200_OK : AWQ_B200_ERR_LAUNCH;
}

}  // namespace awq
