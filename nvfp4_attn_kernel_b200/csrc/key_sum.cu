// Accumulation of the per-channel K sum that the key-shift calibration averages
// (ref: src/nvfp4_vllm/impl.py:137-144: key[:tokens].double().sum(dim=0) added to an fp64
// accumulator of shape [Hkv][128], once per layer and step).  One launch: the key rows of the
// step are read once (the launch is bound by that read), every thread sums 8 adjacent channels
// of a strided run of tokens in fp64, the token lanes of a CTA are folded through shared memory
// and the CTA's partial sums go to the accumulator with fp64 atomic adds.
//
// Every addend is a BF16 number (8 significant bits), so as long as the magnitudes of a
// channel's values span fewer than 2^44 - true of any activations - every partial sum is
// exactly representable in fp64 and the result does not depend on the order of the additions.
#include <cuda_bf16.h>

#include "nvfp4_kernels.h"

namespace nvfp4 {

constexpr int kSumLanes = 4;      // token lanes per CTA
constexpr int kSumChunks = 128;   // channel groups (8 channels each) per CTA

__global__ void __launch_bounds__(kSumLanes * kSumChunks)
key_sum_kernel(const uint16_t* __restrict__ key, int64_t token_stride, int tokens, int width,
               double* __restrict__ sum) {
  __shared__ double part[kSumLanes][kSumChunks][9];   // 9: no bank conflicts on the fold
  const int chunk = threadIdx.x % kSumChunks, lane = threadIdx.x / kSumChunks;
  const int col = (blockIdx.x * kSumChunks + chunk) * 8;
  double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col < width) {
    const int step = gridDim.y * kSumLanes;
    int t = blockIdx.y * kSumLanes + lane;
    // two tokens in flight per thread
    for (; t + step < tokens; t += 2 * step) {
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(key + (int64_t)t * token_stride + col));
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(key + (int64_t)(t + step) * token_stride + col));
      const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] += (double)__uint_as_float(wa[i] << 16) + (double)__uint_as_float(wb[i] << 16);
        acc[2 * i + 1] += (double)__uint_as_float(wa[i] & 0xffff0000u) + (double)__uint_as_float(wb[i] & 0xffff0000u);
      }
    }
    if (t < tokens) {
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(key + (int64_t)t * token_stride + col));
      const uint32_t wa[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] += (double)__uint_as_float(wa[i] << 16);
        acc[2 * i + 1] += (double)__uint_as_float(wa[i] & 0xffff0000u);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) part[lane][chunk][i] = acc[i];
  __syncthreads();
  // thread (lane, chunk) folds channels `lane` and `lane + 4` of its chunk over the token lanes
  if (col < width) {
#pragma unroll
    for (int c = lane; c < 8; c += kSumLanes) {
      double s = 0;
#pragma unroll
      for (int l = 0; l < kSumLanes; ++l) s += part[l][chunk][c];
      if (s != 0.0) atomicAdd(sum + col + c, s);
    }
  }
}

cudaError_t launch_key_sum(const void* key, int64_t token_stride, int tokens, int heads_kv, double* sum,
                           cudaStream_t stream) {
  static_assert(8 % kSumLanes == 0, "the fold gives each token lane 8 / kSumLanes of a chunk's 8 channels");
  const int width = heads_kv * 128;
  const int col_blocks = (width / 8 + kSumChunks - 1) / kSumChunks;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  // four CTAs of 512 threads per SM; no more token blocks than there are runs of token lanes
  int token_blocks = (4 * sms + col_blocks - 1) / col_blocks;
  const int runs = (tokens + kSumLanes - 1) / kSumLanes;
  if (token_blocks > runs) token_blocks = runs;
  if (token_blocks < 1) token_blocks = 1;
  key_sum_kernel<<<dim3(col_blocks, token_blocks), kSumLanes * kSumChunks, 0, stream>>>(
      static_cast<const uint16_t*>(key), token_stride, tokens, width, sum);
  return cudaGetLastError();
}

}  // namespace nvfp4
