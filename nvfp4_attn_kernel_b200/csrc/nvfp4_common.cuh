// Shared device helpers: number-format conversions, scale-block addressing and the
// NVFP4 group quantiser used by every kernel of the library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nvfp4 {

constexpr int kPage = 128;
constexpr int kHeadDim = 128;
constexpr int kGroup = 16;
constexpr int kSfBlockBytes = 1024;  // scale bytes per (page, head): two 512-byte atoms

// Byte offset of (row in [0,128), 16-element group in [0,8)) inside a 1024-byte
// scale block.  This is the ((32,4),(16,4)) atom that tcgen05.cp 32x128b.warpx4
// moves to tensor memory unchanged: 32 rows of 16 bytes, each row holding the
// four scales of rows r, r+32, r+64, r+96.
__host__ __device__ __forceinline__ int sf_offset(int row, int group) {
  return (group >> 2) * 512 + (row & 31) * 16 + (row >> 5) * 4 + (group & 3);
}

// ---- conversions -----------------------------------------------------------

// cvt.rn.satfinite.e4m3x2.f32 d, a, b : a -> upper byte, b -> lower byte.
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ uint8_t f32_to_e4m3(float x) {
  return (uint8_t)(f32x2_to_e4m3x2(x, 0.f) & 0xFF);
}

__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)b));
  return __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFF)));
}

// Eight floats -> eight E2M1 nibbles in one 32-bit word, element i in nibble i.
// cvt.rn.satfinite.e2m1x2.f32 d, a, b : a -> high nibble, b -> low nibble.
__device__ __forceinline__ uint32_t f32x8_to_e2m1x8(float f0, float f1, float f2, float f3,
                                                    float f4, float f5, float f6, float f7) {
  uint32_t r;
  asm("{\n\t"
      ".reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t"
      "}"
      : "=r"(r)
      : "f"(f0), "f"(f1), "f"(f2), "f"(f3), "f"(f4), "f"(f5), "f"(f6), "f"(f7));
  return r;
}

// Four floats -> four E2M1 nibbles in the low 16 bits, element i in nibble i.
__device__ __forceinline__ uint32_t f32x4_to_e2m1x4(float f0, float f1, float f2, float f3) {
  uint32_t r;
  asm("{\n\t"
      ".reg .b8 b0, b1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "mov.b32 %0, {b0, b1, b0, b1};\n\t"
      "}"
      : "=r"(r)
      : "f"(f0), "f"(f1), "f"(f2), "f"(f3));
  return r & 0xFFFFu;
}

// One float -> E2M1 nibble (low 4 bits).
__device__ __forceinline__ uint32_t f32_to_e2m1(float x) {
  uint32_t r;
  asm("{\n\t"
      ".reg .b8 b0;\n\t"
      ".reg .b32 t;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.u32.u8 t, b0;\n\t"
      "and.b32 %0, t, 15;\n\t"
      "}"
      : "=r"(r)
      : "f"(x), "f"(0.f));
  return r;
}

// E2M1 nibble -> float.  Magnitudes {0,.5,1,1.5,2,3,4,6}.
__device__ __forceinline__ float e2m1_to_f32(uint32_t n) {
  const uint32_t e = (n >> 1) & 3u, m = n & 1u;
  // e==0: m*0.5 ; else (1 + m/2) * 2^(e-1)
  float v = e == 0 ? 0.5f * (float)m : __uint_as_float(((126u + e) << 23) | (m << 22));
  return (n & 8u) ? -v : v;
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t lo16) {
  return __uint_as_float(lo16 << 16);
}

// ---- the K/V/Q group quantiser --------------------------------------------
// Arithmetic (must stay exactly this for byte parity with the reference
// quantisers): s = e4m3_rn_satfinite(amax * fp32(1/6)); inv = 1.0f / (float(s) + 1e-30f)
// with IEEE division; nibble = e2m1_rn_satfinite(x * inv).
__device__ __forceinline__ void quantize_group16(const float (&x)[16], uint32_t& lo8, uint32_t& hi8,
                                                 uint8_t& sf) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));
  const float inv6 = 1.0f / 6.0f;  // fp32 constant, as the reference multiplies
  sf = f32_to_e4m3(amax * inv6);
  const float s = e4m3_to_f32(sf);
  const float inv = __fdiv_rn(1.0f, s + 1.0e-30f);
  lo8 = f32x8_to_e2m1x8(x[0] * inv, x[1] * inv, x[2] * inv, x[3] * inv, x[4] * inv, x[5] * inv,
                        x[6] * inv, x[7] * inv);
  hi8 = f32x8_to_e2m1x8(x[8] * inv, x[9] * inv, x[10] * inv, x[11] * inv, x[12] * inv,
                        x[13] * inv, x[14] * inv, x[15] * inv);
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float* out) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

// ---- softmax-probability quantiser ----------------------------------------
// The attention oracle's form: scale = e4m3_rn(group_max / 6) with a true
// division, nibble = e2m1_rn(p / scale) with a true division.
__device__ __forceinline__ uint8_t p_scale_byte(float group_max) {
  return f32_to_e4m3(__fdiv_rn(group_max, 6.0f));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float halfwarp_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace nvfp4
