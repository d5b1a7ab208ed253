// Load-time conversion of expert weights from the byte layout of vLLM's MoE WNA16 method
// (quantization/moe_wna16.py:252-324: qweight uint8 [E, N, K/2] with k = 2j in the low nibble,
// zero points uint8 [E, N/2, K/G] with n = 2i in the low nibble, scales [E, N, K/G]) back to the
// AWQ checkpoint layout the expert kernels read (int32 [E, K, N/8] in nibble order
// [0,2,4,6,1,3,5,7], zero points int32 [E, K/G, N/8], scales [E, K/G, N]).  It is the inverse of
// the converter vLLM runs inside that method's weight loader (moe_wna16.py:389-425).
#include "common.cuh"

namespace awq {
namespace {

// AWQ nibble position of column j within its word of 8: [0, 4, 1, 5, 2, 6, 3, 7]
__device__ __forceinline__ int awq_shift(int j) { return 4 * ((j >> 1) + ((j & 1) << 2)); }

constexpr int kTileK2 = 32;  // bytes of K/2 per tile (64 k)
constexpr int kTileN = 32;   // rows of N per tile (4 output words)

// One block converts a tile of 32 rows (n) x 32 bytes (64 k): reads are coalesced along K/2,
// the transposed words are written coalesced along N/8 through shared memory.
__global__ void wna16_qweight_kernel(const uint8_t* __restrict__ w, uint32_t* __restrict__ out,
                                     int N, int K) {
  __shared__ uint8_t tile[kTileN][kTileK2 + 4];
  const int e = blockIdx.z;
  const int n0 = blockIdx.y * kTileN, j0 = blockIdx.x * kTileK2;
  const int half = K / 2;
  const uint8_t* src = w + (size_t)e * N * half;
  for (int i = threadIdx.x; i < kTileN * kTileK2; i += blockDim.x) {
    const int r = i / kTileK2, c = i % kTileK2;
    const int n = n0 + r, j = j0 + c;
    tile[r][c] = (n < N && j < half) ? src[(size_t)n * half + j] : 0;
  }
  __syncthreads();
  // 64 k x 4 words per tile
  uint32_t* dst = out + (size_t)e * K * (N / 8);
  for (int i = threadIdx.x; i < 2 * kTileK2 * (kTileN / 8); i += blockDim.x) {
    const int word = i % (kTileN / 8), kk = i / (kTileN / 8);
    const int k = 2 * j0 + kk, c = n0 / 8 + word;
    if (k >= K || c >= N / 8) continue;
    uint32_t v = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint8_t b = tile[word * 8 + j][kk >> 1];
      v |= (uint32_t)((kk & 1) ? (b >> 4) : (b & 0xF)) << awq_shift(j);
    }
    dst[(size_t)k * (N / 8) + c] = v;
  }
}

// zero points: out word (g, c) gathers n = 8c + j from byte row 4c + j/2, nibble j & 1
__global__ void wna16_qzeros_kernel(const uint8_t* __restrict__ z, uint32_t* __restrict__ out,
                                    int N, int G) {
  const int e = blockIdx.y;
  const int words = N / 8;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= G * words) return;
  const int g = i / words, c = i % words;
  const uint8_t* src = z + (size_t)e * (N / 2) * G;
  uint32_t v = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint8_t b = src[(size_t)(4 * c + (j >> 1)) * G + g];
    v |= (uint32_t)((j & 1) ? (b >> 4) : (b & 0xF)) << awq_shift(j);
  }
  out[(size_t)e * G * words + i] = v;
}

// scales [E, N, G] -> [E, G, N]
__global__ void wna16_scales_kernel(const __half* __restrict__ s, __half* __restrict__ out, int N,
                                    int G) {
  const int e = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= G * N) return;
  const int g = i / N, n = i % N;
  out[(size_t)e * G * N + i] = s[(size_t)e * N * G + (size_t)n * G + g];
}

}  // namespace

int launch_wna16_to_awq(const uint8_t* w, const __half* scales, const uint8_t* zeros,
                        uint32_t* qweight, __half* scales_out, uint32_t* qzeros, int E, int N,
                        int K, int group, cudaStream_t stream) {
  const int G = K / group;
  dim3 grid((K / 2 + kTileK2 - 1) / kTileK2, (N + kTileN - 1) / kTileN, E);
  wna16_qweight_kernel<<<grid, 256, 0, stream>>>(w, qweight, N, K);
  if (cudaGetLastError() != cudaSuccess) return AWQ_B200_ERR_LAUNCH;
  dim3 gz((G * (N / 8) + 255) / 256, E);
  wna16_qzeros_kernel<<<gz, 256, 0, stream>>>(zeros, qzeros, N, G);
  if (cudaGetLastError() != cudaSuccess) return AWQ_B200_ERR_LAUNCH;
  dim3 gs((G * N + 255) / 256, E);
  wna16_scales_kernel<<<gs, 256, 0, stream>>>(scales, scales_out, N, G);
  return cudaGetLastError() == cudaSuccess ? AWQ_B200_OK : AWQ_B200_ERR_LAUNCH;
}

}  // namespace awq
