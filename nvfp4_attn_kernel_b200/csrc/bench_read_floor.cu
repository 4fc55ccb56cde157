// Measurement aid, NOT part of libnvfp4_b200.so: built into libnvfp4_bench_read_floor.so, which
// only bench.py loads.  A kernel that does nothing but read a byte range once, as fast as plain
// 16-byte loads from every SM go.  bench.py times it over the same page pools as the decode
// step, so that the decode kernel's duration can be set beside the time the bare read takes
// on the same GPU (the floor for a launch that has to touch those bytes).
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace {

__global__ void __launch_bounds__(1024) read_probe_kernel(const uint4* __restrict__ p, size_t n,
                                                          unsigned* __restrict__ sink) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  unsigned acc = 0;
  for (; i + 3 * stride < n; i += 4 * stride) {
    const uint4 a = p[i], b = p[i + stride], c = p[i + 2 * stride], d = p[i + 3 * stride];
    acc += a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w ^ c.x ^ c.y ^ c.z ^ c.w ^ d.x ^ d.y ^ d.z ^ d.w;
  }
  for (; i < n; i += stride) {
    const uint4 a = p[i];
    acc += a.x ^ a.y ^ a.z ^ a.w;
  }
  // keeps the loads alive; the value is data dependent and practically never equal
  if (acc == 0x9E3779B9u && sink) *sink = acc;
}

}  // namespace

// Returns a cudaError_t as int (0: launched).  ptr: 16-byte aligned device range; sink: nullable
// device word (written only in the practically impossible case that the checksum of the data
// equals a constant; it keeps the loads alive).
extern "C" int bench_read_floor(const void* ptr, size_t bytes, uint32_t* sink, void* stream) {
  if (bytes < 16) return 0;
  if (!ptr || (reinterpret_cast<uintptr_t>(ptr) & 15)) return static_cast<int>(cudaErrorInvalidValue);
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  read_probe_kernel<<<2 * sms, 1024, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(ptr),
                                                                              bytes / 16, sink);
  return static_cast<int>(cudaGetLastError());
}
