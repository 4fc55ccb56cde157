// Write-path kernels: Q quantiser, K/V page quantisers (dense, indexed, per-layer
// destinations, fused key shift), BF16 tail append / reset and the tail flush.
//
// All of them are HBM-bound byte shufflers: every global access is a 16-byte
// vector (8 bytes for packed nibbles), consecutive threads touch consecutive
// addresses, and the V quantiser transposes through shared memory so that both
// its reads (along channels) and its writes (along tokens) are coalesced.
#include "nvfp4_common.cuh"
#include "nvfp4_kernels.h"

namespace nvfp4 {

// ---------------------------------------------------------------------------
// Q quantiser: one thread per 16-element group, 8 threads per head.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
quantize_q_kernel(const __nv_bfloat16* __restrict__ q, int64_t row_stride, int64_t head_stride,
                  const int32_t* __restrict__ row_indices, uint8_t* __restrict__ q_fp4,
                  uint8_t* __restrict__ q_sf, __nv_bfloat16* __restrict__ q_padded, int heads_q,
                  int heads_kv) {
  const int row = blockIdx.x;
  const int src_row = row_indices ? row_indices[row] : row;
  const int gq = heads_q / heads_kv;
  const int items = heads_q * 8;
  for (int it = threadIdx.x; it < items; it += blockDim.x) {
    const int head = it >> 3, g = it & 7;
    const __nv_bfloat16* src = q + (int64_t)src_row * row_stride + (int64_t)head * head_stride + g * 16;
    const uint4 a = *reinterpret_cast<const uint4*>(src);
    const uint4 b = *reinterpret_cast<const uint4*>(src + 8);
    if (q_padded) {
      __nv_bfloat16* dst = q_padded + (((int64_t)row * kPage) * heads_q + head) * kHeadDim + g * 16;
      *reinterpret_cast<uint4*>(dst) = a;
      *reinterpret_cast<uint4*>(dst + 8) = b;
    }
    float x[16];
    unpack_bf16x8(a, x);
    unpack_bf16x8(b, x + 8);
    uint32_t lo, hi;
    uint8_t sf;
    quantize_group16(x, lo, hi, sf);
    *reinterpret_cast<uint2*>(q_fp4 + ((int64_t)row * heads_q + head) * 64 + g * 8) =
        make_uint2(lo, hi);
    const int slot = head % gq, kvh = head / gq;
    q_sf[(int64_t)row * heads_q * kSfBlockBytes + (int64_t)kvh * kSfBlockBytes + sf_offset(slot, g)] = sf;
  }
}

// ---------------------------------------------------------------------------
// K page quantiser.  grid (4 token-chunks, work, layers), 256 threads.
// A block covers 32 tokens x all heads; thread = one 16-channel group.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void
quantize_k_block(int chunk, const __nv_bfloat16* __restrict__ tokens, int64_t token_stride,
                 const __nv_bfloat16* __restrict__ key_shift, uint8_t* __restrict__ packed,
                 int64_t packed_pitch, uint8_t* __restrict__ sf, int64_t sf_pitch,
                 const int32_t* __restrict__ src_tokens, const int32_t* __restrict__ dst_pages,
                 const int64_t* __restrict__ packed_bases, const int64_t* __restrict__ sf_bases,
                 int64_t src_layer_stride, int heads_kv) {
  const int work = blockIdx.y, layer = blockIdx.z;
  const int64_t page = dst_pages ? (int64_t)dst_pages[work] : (int64_t)work;
  if (page < 0) return;
  const int64_t first = (src_tokens ? (int64_t)src_tokens[work] : (int64_t)work * kPage) +
                        (int64_t)layer * src_layer_stride;
  uint8_t* pk = (packed_bases ? reinterpret_cast<uint8_t*>(packed_bases[layer]) : packed) +
                page * packed_pitch;
  uint8_t* ps = (sf_bases ? reinterpret_cast<uint8_t*>(sf_bases[layer]) : sf) + page * sf_pitch;
  const __nv_bfloat16* shift = key_shift ? key_shift + (int64_t)layer * heads_kv * kHeadDim : nullptr;

  const int groups_per_token = heads_kv * 8;
  const int items = 32 * groups_per_token;
  for (int it = threadIdx.x; it < items; it += blockDim.x) {
    const int tl = it / groups_per_token;
    const int rem = it - tl * groups_per_token;  // head*8 + g
    const int head = rem >> 3, g = rem & 7;
    const int tok = chunk * 32 + tl;
    const __nv_bfloat16* src = tokens + (first + tok) * token_stride + rem * 16;
    const uint4 a = *reinterpret_cast<const uint4*>(src);
    const uint4 b = *reinterpret_cast<const uint4*>(src + 8);
    float x[16];
    unpack_bf16x8(a, x);
    unpack_bf16x8(b, x + 8);
    if (shift) {
      const uint4 sa = *reinterpret_cast<const uint4*>(shift + rem * 16);
      const uint4 sb = *reinterpret_cast<const uint4*>(shift + rem * 16 + 8);
      float m[16];
      unpack_bf16x8(sa, m);
      unpack_bf16x8(sb, m + 8);
#pragma unroll
      for (int i = 0; i < 16; ++i)
        x[i] = __bfloat162float(__float2bfloat16_rn(x[i] - m[i]));  // one BF16 subtract
    }
    uint32_t lo, hi;
    uint8_t s;
    quantize_group16(x, lo, hi, s);
    *reinterpret_cast<uint2*>(pk + ((int64_t)tok * heads_kv + head) * 64 + g * 8) = make_uint2(lo, hi);
    ps[head * kSfBlockBytes + sf_offset(tok, g)] = s;
  }
}

__global__ void __launch_bounds__(256)
quantize_k_pages_kernel(const __nv_bfloat16* __restrict__ tokens, int64_t token_stride,
                        const __nv_bfloat16* __restrict__ key_shift, uint8_t* __restrict__ packed,
                        int64_t packed_pitch, uint8_t* __restrict__ sf, int64_t sf_pitch,
                        const int32_t* __restrict__ src_tokens, const int32_t* __restrict__ dst_pages,
                        const int64_t* __restrict__ packed_bases, const int64_t* __restrict__ sf_bases,
                        int64_t src_layer_stride, int heads_kv) {
  quantize_k_block(blockIdx.x, tokens, token_stride, key_shift, packed, packed_pitch, sf, sf_pitch,
                   src_tokens, dst_pages, packed_bases, sf_bases, src_layer_stride, heads_kv);
}

// ---------------------------------------------------------------------------
// V page quantiser.  grid (heads, work, layers), 256 threads.
// The 128x128 BF16 tile of one head goes through shared memory: global reads
// run along channels, the quantiser walks 16 tokens of one channel, and the
// packed rows (64 bytes per channel) leave through a staged, coalesced store.
// ---------------------------------------------------------------------------
constexpr int kVRowWords = 65;  // 128 bf16 = 64 words, +1 word of padding per token row

struct VSmem {
  uint32_t tile[kPage * kVRowWords];        // [tok][65 words]
  __align__(16) uint8_t outp[kHeadDim * 64];  // [d][64 B]
  __align__(16) uint8_t outs[kSfBlockBytes];
};

__device__ __forceinline__ void
quantize_v_block(VSmem& sm, int head, const __nv_bfloat16* __restrict__ tokens, int64_t token_stride,
                 uint8_t* __restrict__ packed, int64_t packed_pitch, uint8_t* __restrict__ sf,
                 int64_t sf_pitch, const int32_t* __restrict__ src_tokens,
                 const int32_t* __restrict__ dst_pages, const int64_t* __restrict__ packed_bases,
                 const int64_t* __restrict__ sf_bases, int64_t src_layer_stride, int heads_kv) {
  uint32_t* tile = sm.tile;
  uint8_t* outp = sm.outp;
  uint8_t* outs = sm.outs;
  const int work = blockIdx.y, layer = blockIdx.z;
  const int64_t page = dst_pages ? (int64_t)dst_pages[work] : (int64_t)work;
  if (page < 0) return;
  const int64_t first = (src_tokens ? (int64_t)src_tokens[work] : (int64_t)work * kPage) +
                        (int64_t)layer * src_layer_stride;
  uint8_t* pk = (packed_bases ? reinterpret_cast<uint8_t*>(packed_bases[layer]) : packed) +
                page * packed_pitch + (int64_t)head * kHeadDim * 64;
  uint8_t* ps = (sf_bases ? reinterpret_cast<uint8_t*>(sf_bases[layer]) : sf) + page * sf_pitch +
                (int64_t)head * kSfBlockBytes;

  // load: 128 tokens x 256 B; 16 threads per token row
  for (int it = threadIdx.x; it < kPage * 16; it += blockDim.x) {
    const int tok = it >> 4, c = it & 15;
    const uint4 v = *reinterpret_cast<const uint4*>(tokens + (first + tok) * token_stride +
                                                    head * kHeadDim + c * 8);
    uint32_t* dst = tile + tok * kVRowWords + c * 4;
    dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
  }
  __syncthreads();
  // quantise: item = (group g, channel d); a warp holds 32 consecutive channels
  for (int it = threadIdx.x; it < 8 * kHeadDim; it += blockDim.x) {
    const int g = it >> 7, d = it & 127;
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t w = tile[(g * 16 + i) * kVRowWords + (d >> 1)];
      x[i] = (d & 1) ? __uint_as_float(w & 0xFFFF0000u) : __uint_as_float(w << 16);
    }
    uint32_t lo, hi;
    uint8_t s;
    quantize_group16(x, lo, hi, s);
    *reinterpret_cast<uint2*>(outp + d * 64 + g * 8) = make_uint2(lo, hi);
    outs[sf_offset(d, g)] = s;
  }
  __syncthreads();
  for (int it = threadIdx.x; it < kHeadDim * 64 / 16; it += blockDim.x)
    reinterpret_cast<uint4*>(pk)[it] = reinterpret_cast<const uint4*>(outp)[it];
  for (int it = threadIdx.x; it < kSfBlockBytes / 16; it += blockDim.x)
    reinterpret_cast<uint4*>(ps)[it] = reinterpret_cast<const uint4*>(outs)[it];
}

__global__ void __launch_bounds__(256)
quantize_v_pages_kernel(const __nv_bfloat16* __restrict__ tokens, int64_t token_stride,
                        uint8_t* __restrict__ packed, int64_t packed_pitch,
                        uint8_t* __restrict__ sf, int64_t sf_pitch,
                        const int32_t* __restrict__ src_tokens, const int32_t* __restrict__ dst_pages,
                        const int64_t* __restrict__ packed_bases, const int64_t* __restrict__ sf_bases,
                        int64_t src_layer_stride, int heads_kv) {
  __shared__ VSmem sm;
  quantize_v_block(sm, blockIdx.x, tokens, token_stride, packed, packed_pitch, sf, sf_pitch,
                   src_tokens, dst_pages, packed_bases, sf_bases, src_layer_stride, heads_kv);
}

// Tail flush: K and V of every (slot, layer) in one launch.
// grid (4 + heads_kv, work, layers): blocks 0..3 quantise K token chunks, the rest one V head each.
__global__ void __launch_bounds__(256)
tail_flush_kernel(const __nv_bfloat16* __restrict__ tail_key, const __nv_bfloat16* __restrict__ tail_value,
                  int64_t src_layer_stride, const int32_t* __restrict__ src_tokens,
                  const int32_t* __restrict__ dst_pages, const int64_t* __restrict__ bases,
                  int64_t k_pitch, int64_t k_sf_pitch, int64_t v_pitch, int64_t v_sf_pitch,
                  int layers, int heads_kv) {
  __shared__ VSmem sm;
  const int64_t token_stride = (int64_t)heads_kv * kHeadDim;
  if (blockIdx.x < 4) {
    quantize_k_block(blockIdx.x, tail_key, token_stride, nullptr, nullptr, k_pitch, nullptr,
                     k_sf_pitch, src_tokens, dst_pages, bases, bases + layers, src_layer_stride,
                     heads_kv);
  } else {
    quantize_v_block(sm, blockIdx.x - 4, tail_value, token_stride, nullptr, v_pitch, nullptr,
                     v_sf_pitch, src_tokens, dst_pages, bases + 2 * layers, bases + 3 * layers,
                     src_layer_stride, heads_kv);
  }
}

// ---------------------------------------------------------------------------
// Tail append: one block per token, 16 bytes per thread and tensor.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void
tail_append_token(int token, const __nv_bfloat16* __restrict__ key, const __nv_bfloat16* __restrict__ value,
                  int64_t key_token_stride, int64_t value_token_stride,
                  const __nv_bfloat16* __restrict__ key_shift, __nv_bfloat16* __restrict__ tail_key,
                  __nv_bfloat16* __restrict__ tail_value, int64_t tail_slot_stride,
                  const int32_t* __restrict__ query_start_loc, const int32_t* __restrict__ seq_lens,
                  const int32_t* __restrict__ seqused_fp4, const int32_t* __restrict__ row_to_slot,
                  int num_reqs, int heads_kv) {
  // the row that owns this token = number of row ends at or before it
  int row = 0;
  for (int r = 0; r < num_reqs; ++r) row += (query_start_loc[r + 1] <= token) ? 1 : 0;
  if (row >= num_reqs) return;
  const int slot = row_to_slot[row];
  const int offset = seq_lens[row] + token - query_start_loc[row + 1] - seqused_fp4[row];
  if (slot < 0 || offset < 0 || offset >= kPage) return;
  const int width = heads_kv * kHeadDim;
  const int64_t dst = (int64_t)slot * tail_slot_stride + (int64_t)offset * width;
  for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
    uint4 k = *reinterpret_cast<const uint4*>(key + (int64_t)token * key_token_stride + c);
    if (key_shift) {
      const uint4 m = *reinterpret_cast<const uint4*>(key_shift + c);
      float x[8], y[8];
      unpack_bf16x8(k, x);
      unpack_bf16x8(m, y);
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_bfloat16 a = __float2bfloat16_rn(x[2 * i] - y[2 * i]);
        const __nv_bfloat16 b = __float2bfloat16_rn(x[2 * i + 1] - y[2 * i + 1]);
        w[i] = (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
      }
      k = make_uint4(w[0], w[1], w[2], w[3]);
    }
    *reinterpret_cast<uint4*>(tail_key + dst + c) = k;
    *reinterpret_cast<uint4*>(tail_value + dst + c) =
        *reinterpret_cast<const uint4*>(value + (int64_t)token * value_token_stride + c);
  }
}

__global__ void __launch_bounds__(128)
tail_append_kernel(const __nv_bfloat16* __restrict__ key, const __nv_bfloat16* __restrict__ value,
                   int64_t key_token_stride, int64_t value_token_stride,
                   const __nv_bfloat16* __restrict__ key_shift, __nv_bfloat16* __restrict__ tail_key,
                   __nv_bfloat16* __restrict__ tail_value, int64_t tail_slot_stride,
                   const int32_t* __restrict__ query_start_loc, const int32_t* __restrict__ seq_lens,
                   const int32_t* __restrict__ seqused_fp4, const int32_t* __restrict__ row_to_slot,
                   int num_reqs, int heads_kv) {
  tail_append_token(blockIdx.x, key, value, key_token_stride, value_token_stride, key_shift, tail_key,
                    tail_value, tail_slot_stride, query_start_loc, seq_lens, seqused_fp4, row_to_slot,
                    num_reqs, heads_kv);
}

// One layer's K/V of a step in ONE launch: full pages quantised into their blocks (key shift
// fused), every other token copied to its row's tail slot.
// grid (4 + heads_kv + tail blocks, max(work, 1)): x < 4 quantises a K token chunk of page-work
// item y, the next heads_kv blocks one V head of it, the rest take one token each.
struct WriteKvArgs {
  const __nv_bfloat16* key; const __nv_bfloat16* value;
  int64_t key_token_stride, value_token_stride;
  const __nv_bfloat16* key_shift;
  uint8_t* k_packed; int64_t k_pitch; uint8_t* k_sf; int64_t k_sf_pitch;
  uint8_t* v_packed; int64_t v_pitch; uint8_t* v_sf; int64_t v_sf_pitch;
  const int32_t* src_tokens; const int32_t* dst_pages; int work;
  __nv_bfloat16* tail_key; __nv_bfloat16* tail_value; int64_t tail_slot_stride;
  const int32_t* query_start_loc; const int32_t* seq_lens; const int32_t* seqused_fp4;
  const int32_t* row_to_slot;
  int num_tokens, num_reqs, heads_kv;
};

__global__ void __launch_bounds__(256) write_kv_kernel(const WriteKvArgs a) {
  __shared__ VSmem sm;
  const int role = blockIdx.x;
  if (role < 4 + a.heads_kv) {
    if ((int)blockIdx.y >= a.work) return;
    if (role < 4)
      quantize_k_block(role, a.key, a.key_token_stride, a.key_shift, a.k_packed, a.k_pitch, a.k_sf,
                       a.k_sf_pitch, a.src_tokens, a.dst_pages, nullptr, nullptr, 0, a.heads_kv);
    else
      quantize_v_block(sm, role - 4, a.value, a.value_token_stride, a.v_packed, a.v_pitch, a.v_sf,
                       a.v_sf_pitch, a.src_tokens, a.dst_pages, nullptr, nullptr, 0, a.heads_kv);
    return;
  }
  const int token = (role - 4 - a.heads_kv) * gridDim.y + blockIdx.y;
  if (token >= a.num_tokens) return;
  tail_append_token(token, a.key, a.value, a.key_token_stride, a.value_token_stride, a.key_shift,
                    a.tail_key, a.tail_value, a.tail_slot_stride, a.query_start_loc, a.seq_lens,
                    a.seqused_fp4, a.row_to_slot, a.num_reqs, a.heads_kv);
}

// ---------------------------------------------------------------------------
// Tail reset: grid (layers, rows, 16 chunks of 8 tokens).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
tail_reset_kernel(__nv_bfloat16* __restrict__ tail_key, __nv_bfloat16* __restrict__ tail_value,
                  int64_t layer_stride, int64_t slot_stride,
                  const int32_t* __restrict__ query_start_loc, const int32_t* __restrict__ seq_lens,
                  const int32_t* __restrict__ row_to_slot, int heads_kv) {
  const int layer = blockIdx.x, row = blockIdx.y, chunk = blockIdx.z;
  const int slot = row_to_slot[row];
  const int qlen = query_start_loc[row + 1] - query_start_loc[row];
  if (slot < 0 || seq_lens[row] > qlen) return;
  const int width = heads_kv * kHeadDim;
  const int64_t base = (int64_t)layer * layer_stride + (int64_t)slot * slot_stride +
                       (int64_t)chunk * 8 * width;
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (int c = threadIdx.x * 8; c < 8 * width; c += blockDim.x * 8) {
    *reinterpret_cast<uint4*>(tail_key + base + c) = z;
    *reinterpret_cast<uint4*>(tail_value + base + c) = z;
  }
}

// ---------------------------------------------------------------------------
// host launchers
// ---------------------------------------------------------------------------
cudaError_t launch_quantize_q(const void* q, int64_t row_stride, int64_t head_stride,
                              const int32_t* row_indices, void* q_fp4, void* q_sf, void* q_padded,
                              int rows, int heads_q, int heads_kv, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  quantize_q_kernel<<<rows, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(q), row_stride, head_stride, row_indices,
      static_cast<uint8_t*>(q_fp4), static_cast<uint8_t*>(q_sf),
      static_cast<__nv_bfloat16*>(q_padded), heads_q, heads_kv);
  return cudaGetLastError();
}

cudaError_t launch_quantize_k(const void* tokens, int64_t token_stride, const void* key_shift,
                              void* packed, int64_t packed_pitch, void* sf, int64_t sf_pitch,
                              const int32_t* src_tokens, const int32_t* dst_pages,
                              const int64_t* packed_bases, const int64_t* sf_bases, int work,
                              int layers, int64_t src_layer_stride, int heads_kv,
                              cudaStream_t stream) {
  if (work == 0 || layers == 0) return cudaSuccess;
  dim3 grid(4, work, layers);
  quantize_k_pages_kernel<<<grid, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(tokens), token_stride,
      static_cast<const __nv_bfloat16*>(key_shift), static_cast<uint8_t*>(packed), packed_pitch,
      static_cast<uint8_t*>(sf), sf_pitch, src_tokens, dst_pages, packed_bases, sf_bases,
      src_layer_stride, heads_kv);
  return cudaGetLastError();
}

cudaError_t launch_quantize_v(const void* tokens, int64_t token_stride, void* packed,
                              int64_t packed_pitch, void* sf, int64_t sf_pitch,
                              const int32_t* src_tokens, const int32_t* dst_pages,
                              const int64_t* packed_bases, const int64_t* sf_bases, int work,
                              int layers, int64_t src_layer_stride, int heads_kv,
                              cudaStream_t stream) {
  if (work == 0 || layers == 0) return cudaSuccess;
  dim3 grid(heads_kv, work, layers);
  quantize_v_pages_kernel<<<grid, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(tokens), token_stride, static_cast<uint8_t*>(packed),
      packed_pitch, static_cast<uint8_t*>(sf), sf_pitch, src_tokens, dst_pages, packed_bases,
      sf_bases, src_layer_stride, heads_kv);
  return cudaGetLastError();
}

cudaError_t launch_tail_append(const void* key, const void* value, int64_t key_token_stride,
                               int64_t value_token_stride, const void* key_shift, void* tail_key,
                               void* tail_value, int64_t tail_slot_stride,
                               const int32_t* query_start_loc, const int32_t* seq_lens,
                               const int32_t* seqused_fp4, const int32_t* row_to_slot,
                               int num_tokens, int num_reqs, int heads_kv, cudaStream_t stream) {
  if (num_tokens == 0) return cudaSuccess;
  tail_append_kernel<<<num_tokens, 128, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(key), static_cast<const __nv_bfloat16*>(value),
      key_token_stride, value_token_stride, static_cast<const __nv_bfloat16*>(key_shift),
      static_cast<__nv_bfloat16*>(tail_key), static_cast<__nv_bfloat16*>(tail_value),
      tail_slot_stride, query_start_loc, seq_lens, seqused_fp4, row_to_slot, num_reqs, heads_kv);
  return cudaGetLastError();
}

cudaError_t launch_write_kv(const void* key, const void* value, int64_t key_token_stride,
                            int64_t value_token_stride, const void* key_shift, void* k_packed,
                            int64_t k_pitch, void* k_sf, int64_t k_sf_pitch, void* v_packed,
                            int64_t v_pitch, void* v_sf, int64_t v_sf_pitch, const int32_t* src_tokens,
                            const int32_t* dst_pages, int work, void* tail_key, void* tail_value,
                            int64_t tail_slot_stride, const int32_t* query_start_loc,
                            const int32_t* seq_lens, const int32_t* seqused_fp4,
                            const int32_t* row_to_slot, int num_tokens, int num_reqs, int heads_kv,
                            cudaStream_t stream) {
  if (num_tokens == 0) return cudaSuccess;
  WriteKvArgs a;
  a.key = static_cast<const __nv_bfloat16*>(key); a.value = static_cast<const __nv_bfloat16*>(value);
  a.key_token_stride = key_token_stride; a.value_token_stride = value_token_stride;
  a.key_shift = static_cast<const __nv_bfloat16*>(key_shift);
  a.k_packed = static_cast<uint8_t*>(k_packed); a.k_pitch = k_pitch;
  a.k_sf = static_cast<uint8_t*>(k_sf); a.k_sf_pitch = k_sf_pitch;
  a.v_packed = static_cast<uint8_t*>(v_packed); a.v_pitch = v_pitch;
  a.v_sf = static_cast<uint8_t*>(v_sf); a.v_sf_pitch = v_sf_pitch;
  a.src_tokens = src_tokens; a.dst_pages = dst_pages; a.work = work;
  a.tail_key = static_cast<__nv_bfloat16*>(tail_key); a.tail_value = static_cast<__nv_bfloat16*>(tail_value);
  a.tail_slot_stride = tail_slot_stride;
  a.query_start_loc = query_start_loc; a.seq_lens = seq_lens; a.seqused_fp4 = seqused_fp4;
  a.row_to_slot = row_to_slot;
  a.num_tokens = num_tokens; a.num_reqs = num_reqs; a.heads_kv = heads_kv;
  const int rows_y = work > 0 ? work : 1;
  const int tail_blocks = (num_tokens + rows_y - 1) / rows_y;
  dim3 grid(4 + heads_kv + tail_blocks, rows_y);
  write_kv_kernel<<<grid, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_tail_reset(void* tail_key, void* tail_value, int64_t layer_stride,
                              int64_t slot_stride, int layers, const int32_t* query_start_loc,
                              const int32_t* seq_lens, const int32_t* row_to_slot, int num_reqs,
                              int heads_kv, cudaStream_t stream) {
  if (layers == 0 || num_reqs == 0) return cudaSuccess;
  dim3 grid(layers, num_reqs, 16);
  tail_reset_kernel<<<grid, 256, 0, stream>>>(
      static_cast<__nv_bfloat16*>(tail_key), static_cast<__nv_bfloat16*>(tail_value), layer_stride,
      slot_stride, query_start_loc, seq_lens, row_to_slot, heads_kv);
  return cudaGetLastError();
}

cudaError_t launch_tail_flush(const void* tail_key, const void* tail_value,
                              int64_t src_layer_stride, const int32_t* src_tokens,
                              const int32_t* dst_pages, const int64_t* bases, int64_t k_pitch,
                              int64_t k_sf_pitch, int64_t v_pitch, int64_t v_sf_pitch, int work,
                              int layers, int heads_kv, cudaStream_t stream) {
  if (work == 0 || layers == 0) return cudaSuccess;
  dim3 grid(4 + heads_kv, work, layers);
  tail_flush_kernel<<<grid, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(tail_key), static_cast<const __nv_bfloat16*>(tail_value),
      src_layer_stride, src_tokens, dst_pages, bases, k_pitch, k_sf_pitch, v_pitch, v_sf_pitch,
      layers, heads_kv);
  return cudaGetLastError();
}

}  // namespace nvfp4
