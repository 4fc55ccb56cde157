// Device and host helpers shared by the tensor-core decode kernels (sm_100a): mbarrier and
// tensor-memory primitives, the block-scaled tcgen05 MMA and its descriptors, TMA and bulk
// loads, the softmax page step with NVFP4 quantisation of the probabilities, and the tensor
// maps of the K and V page arrays.
#pragma once

#include <cuda.h>

#include "decode_common.cuh"

namespace nvfp4 {
namespace sm100 {

constexpr int kTileBytes = 8192;                                  // 128 rows x 64 B
constexpr int kSlotBytes = kTileBytes + kSfBlockBytes;            // a tile and its scale block
constexpr unsigned long long kWaitLimitNs = 2000000000ull;        // 2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait.  Returns false when the CTA is aborting (someone's wait expired).
template <class SM>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, SM& sm, uint32_t* status) {
  if (mbar_try(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  uint32_t spins = 0;
  while (!mbar_try(bar, parity)) {
    if (sm.abort_flag) return false;
    if ((++spins & 1023u) == 0 && global_ns() - t0 > kWaitLimitNs) {
      sm.abort_flag = 1;
      set_status(status, NVFP4_STATUS_WAIT_TIMEOUT);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
      "%14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                 "=r"(r[7])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, K-major, 64-byte swizzle: rows of 64 bytes, eight-row
// groups 512 bytes apart (stride byte offset), descriptor version 1, layout type 4.
__device__ __forceinline__ uint64_t desc_sw64(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(512 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)4 << 61);
}
// Scale atom for tcgen05.cp 32x128b: 32 rows of 16 bytes, no swizzle, eight-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t desc_sf(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}

// Instruction descriptor: E2M1 x E2M1 (format code 1), UE4M3 scales, K-major both, N = NQ, M = 128, K = 64.
template <int NQ>
__device__ __forceinline__ void mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t sfa,
                                         uint32_t sfb, uint32_t accumulate) {
  constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((uint32_t)(NQ >> 3) << 17) | ((128u >> 4) << 24);
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void cp_sf(uint32_t tmem_dst, uint32_t saddr) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(desc_sf(saddr))
               : "memory");
}

__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(dst), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

constexpr int kKProducerWarp = 8;
constexpr int kQkWarp = 9;   // also owns the tensor-memory allocation
constexpr int kPvWarp = 10;
constexpr int kVProducerWarp = 11;

// Barrier over the 256 score and output threads with an AND of a predicate.
__device__ __forceinline__ bool bar_and_256(int bar_id, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 q, %2, 0;\n\t"
      "bar.red.and.pred p, %1, 256, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"(bar_id), "r"((uint32_t)pred)
      : "memory");
  return out != 0;
}

// Barrier over the 128 score threads that also ANDs a predicate across them.
__device__ __forceinline__ bool bar_and_128(int bar_id, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 q, %2, 0;\n\t"
      "bar.red.and.pred p, %1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"(bar_id), "r"((uint32_t)pred)
      : "memory");
  return out != 0;
}

// byte offset of (row, byte column) inside an 8-row, 64-byte-swizzled B tile
__device__ __forceinline__ int sw64_offset(int row, int byte_col) {
  return row * 64 + ((((byte_col >> 4) ^ ((row >> 1) & 3))) << 4) + (byte_col & 15);
}

// Barrier over N threads (a multiple of 32) that also ANDs a predicate across them.
template <int N>
__device__ __forceinline__ bool bar_and(int bar_id, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 q, %2, 0;\n\t"
      "bar.red.and.pred p, %1, %3, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"(bar_id), "r"((uint32_t)pred), "n"(N)
      : "memory");
  return out != 0;
}

// One page of scores for one query head, seen by the 32 lanes of its owner warp (four
// consecutive kv positions per lane): group and page maxima.
struct PageMax { float group, page; };
__device__ __forceinline__ PageMax page_max(const float4& z) {
  float g = fmaxf(fmaxf(z.x, z.y), fmaxf(z.z, z.w));
  g = fmaxf(g, __shfl_xor_sync(0xffffffffu, g, 1));
  g = fmaxf(g, __shfl_xor_sync(0xffffffffu, g, 2));   // the 16-position scale group
  float b = fmaxf(g, __shfl_xor_sync(0xffffffffu, g, 4));
  b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, 8));
  b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, 16));
  return PageMax{g, b};
}

// exp2 of one page against its running maximum, NVFP4 quantisation of the probabilities in
// the oracle's form (scale = e4m3(group max / 6), nibble = e2m1(p / scale)), stores of the
// packed bytes and of the group's scale byte.  A scale that rounds to zero is raised to the
// smallest E4M3 subnormal instead of dropping the group.  The two divisions are a multiply by
// fp32(1/6) and by an approximate reciprocal: that can move a result only when it sits within
// an ulp of a rounding boundary.  Returns the sum of the unquantised probabilities.
__device__ __forceinline__ float quantize_page(const float4& z, float group_max, float m, uint8_t* p_tile,
                                               uint8_t* p_sf, int q, int lane) {
  const float p0 = exp2_rel(z.x, m), p1 = exp2_rel(z.y, m), p2 = exp2_rel(z.z, m), p3 = exp2_rel(z.w, m);
  uint32_t sb = f32_to_e4m3(exp2_rel(group_max, m) * (1.0f / 6.0f));
  sb = sb == 0 ? 1u : sb;
  const float inv = __fdividef(1.0f, e4m3_to_f32((uint8_t)sb));
  const uint32_t packed = f32x4_to_e2m1x4(p0 * inv, p1 * inv, p2 * inv, p3 * inv);
  *reinterpret_cast<uint16_t*>(p_tile + sw64_offset(q, 2 * lane)) = (uint16_t)packed;
  if ((lane & 3) == 0) {
    const int g = lane >> 2;
    p_sf[(g >> 2) * 512 + q * 16 + (g & 3)] = (uint8_t)sb;
  }
  return (p0 + p1) + (p2 + p3);
}

// ---------------------------------------------------------------------------
// host side: tensor maps through the driver entry point (no link-time libcuda)
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

struct MapKey {
  const void* base; int64_t pitch; int64_t pages; int heads; int which;
  bool operator==(const MapKey& o) const {
    return base == o.base && pitch == o.pitch && pages == o.pages && heads == o.heads && which == o.which;
  }
};
struct MapEntry { MapKey key; CUtensorMap map; bool valid; };

// K: bytes [64] x heads x tokens [128] x pages ; V: bytes [64] x channels [128] x heads x pages ;
// which = 2: a BF16 tail cache (pitch unused)
constexpr int kTailBoxRows = 32;   // tokens per box of a tail map
inline cudaError_t make_map(int which, const void* base, int64_t pitch, int64_t pages, int heads,
                            CUtensorMap* out) {
  // four maps per launch (K, V and the two tail caches) and one set per layer of a model: a
  // direct-mapped cache by address, so that an eager step does not encode maps at every call
  constexpr int kCached = 256;
  thread_local MapEntry cache[kCached] = {};
  const MapKey key{base, pitch, pages, heads, which};
  const unsigned long long h =
      (static_cast<unsigned long long>(reinterpret_cast<uintptr_t>(base)) + (unsigned long long)which) *
      0x9E3779B97F4A7C15ull;
  // two candidate places per key: the maps of one launch rarely push each other out
  MapEntry* slot = &cache[(h >> 56) % kCached];
  if (slot->valid && slot->key == key) { *out = slot->map; return cudaSuccess; }
  MapEntry* second = &cache[((h >> 48) ^ 0x55u) % kCached];
  if (second->valid && second->key == key) { *out = second->map; return cudaSuccess; }
  if (slot->valid && !second->valid) slot = second;
  EncodeTiledFn fn = encode_fn();
  if (!fn) return cudaErrorNotSupported;
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
  if (which == 0) {
    dims[0] = 64; dims[1] = heads; dims[2] = 128; dims[3] = pages;
    strides[0] = 64; strides[1] = (cuuint64_t)heads * 64; strides[2] = pitch;
    box[0] = 64; box[1] = 1; box[2] = 128; box[3] = 1;
  } else if (which == 1) {
    dims[0] = 64; dims[1] = 128; dims[2] = heads; dims[3] = pages;
    strides[0] = 64; strides[1] = 128 * 64; strides[2] = pitch;
    box[0] = 64; box[1] = 128; box[2] = 1; box[3] = 1;
  } else {
    // BF16 tail pages, [pages * 128 tokens][heads][128 channels] seen as bytes: a box is half a
    // row (128 of its 256 bytes) of one head for kTailBoxRows tokens, 128-byte swizzle
    // (a map of rank 3)
    dims[0] = 256; dims[1] = heads; dims[2] = (cuuint64_t)pages * 128; dims[3] = 1;
    strides[0] = 256; strides[1] = (cuuint64_t)heads * 256; strides[2] = 0;
    box[0] = 128; box[1] = 1; box[2] = kTailBoxRows; box[3] = 1;
  }
  CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_128B;
  CUtensorMap map;
  CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, which >= 2 ? 3 : 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, which >= 2 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                  promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  *slot = MapEntry{key, map, true};
  *out = map;
  return cudaSuccess;
}

}  // namespace sm100
}  // namespace nvfp4
