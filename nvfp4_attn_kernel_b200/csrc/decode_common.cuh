// Pieces shared by the two decode kernels: work decomposition, the BF16 tail
// block (CUDA cores), block-wide reductions over the 128 softmax threads and the
// epilogue.  Thread t of the 128 plays two roles: "kv position t of the current
// block" while scores are formed, and "output channel d = t" while P.V is
// accumulated, so neither role needs a transpose of the G x 128 score tile.
#pragma once

#include "nvfp4_common.cuh"
#include "nvfp4_kernels.h"
#include "../../include/nvfp4_b200.h"

namespace nvfp4 {

constexpr float kLn2 = 0.6931471805599453f;

struct TileWork {
  int row, kvh, split;
  int64_t slot;               // where this CTA's partial goes: index into [slots][heads_q]
  int first_page, last_page;  // logical FP4 pages [first, last) owned by this split
  int tail_len;               // BF16 tail tokens owned by this split (0 if none)
  int tail_id;
};

// ---- system-scope accesses for data and flags that peer GPUs write or read ----
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float ld_relaxed_sys(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(float* p, float v) {
  asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
constexpr unsigned long long kPeerWaitNs = 1000000000ull;  // bound of every wait on a peer GPU: 1 s
constexpr int kInboxStride = 132;  // floats per (source, row, head) slot of an inbox: 128 channels, LSE, padding

__device__ __forceinline__ void set_status(uint32_t* status, uint32_t bit) {
  if (status) atomicOr(status, bit);
}

// Resolve what this CTA owns.  Metadata is device-resident and, on the trusted
// path, unchecked by the host: anything out of range is clamped, flagged in the
// sticky status word and never turned into an address.
// ``what``: which part of the row a piece may own.  The classic split gives the tail to split 0;
// a work list names page pieces and tail pieces separately.
constexpr int kSplitZeroOwnsTail = 0, kPagesOnly = 1, kTailOnly = 2;

__device__ __forceinline__ TileWork resolve_work(const DecodeParams& p, int row, int kvh, int split,
                                                 int num_splits, int64_t slot, int what = kSplitZeroOwnsTail) {
  TileWork w;
  w.row = row; w.kvh = kvh; w.split = split; w.slot = slot;
  // the row's three words are fetched side by side (a length, then the tail's length, then its
  // id, each behind a branch on the one before, were three round trips at the head of every CTA)
  const bool may_own_tail = (what == kTailOnly || (what == kSplitZeroOwnsTail && split == 0)) &&
                            p.tail_key != nullptr && p.seqused_tail != nullptr;
  int fp4 = p.seqused_fp4[row];
  int len = may_own_tail ? p.seqused_tail[row] : 0;
  const int id = may_own_tail && p.tail_ids != nullptr ? p.tail_ids[row] : -1;
  int n = fp4 >> 7;
  if (fp4 < 0 || (fp4 & 127) || n > p.max_pages) {
    set_status(p.status, NVFP4_STATUS_BAD_LENGTH);
    n = fp4 < 0 ? 0 : (n > p.max_pages ? p.max_pages : n);
  }
  const int per = (n + num_splits - 1) / num_splits;
  w.first_page = min(split * per, n);
  w.last_page = min((split + 1) * per, n);
  if (what == kTailOnly) w.first_page = w.last_page = 0;
  w.tail_len = 0;
  w.tail_id = -1;
  if (len > 0) {
    if (len > kPage) { set_status(p.status, NVFP4_STATUS_BAD_LENGTH); len = kPage; }
    if (id < 0 || (int64_t)id >= p.tail_pages) {
      set_status(p.status, NVFP4_STATUS_BAD_TAIL_ID);
    } else {
      w.tail_len = len;
      w.tail_id = id;
    }
  }
  return w;
}

// The classic grid (splits, heads_kv, rows): block (x, y, z) is split x of KV head y of row z.
__device__ __forceinline__ TileWork resolve_grid_work(const DecodeParams& p) {
  return resolve_work(p, blockIdx.z, blockIdx.y, blockIdx.x, p.num_splits,
                      (int64_t)blockIdx.x * p.rows + blockIdx.z);
}

// max over the 128 softmax threads of G per-thread values; red is [4][G] floats.
// Every one of the 128 threads must call; uses barrier `bar_id` with 128 threads.
template <int G>
__device__ __forceinline__ void block_max_128(float (&v)[G], float* red, int tid, int bar_id) {
  const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int q = 0; q < G; ++q) {
    const float w = warp_max(v[q]);
    if (lane == 0) red[warp * G + q] = w;
  }
  asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
#pragma unroll
  for (int q = 0; q < G; ++q)
    v[q] = fmaxf(fmaxf(red[q], red[G + q]), fmaxf(red[2 * G + q], red[3 * G + q]));
  asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
}

template <int G>
__device__ __forceinline__ void block_sum_128(float (&v)[G], float* red, int tid, int bar_id) {
  const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int q = 0; q < G; ++q) {
    const float w = warp_sum(v[q]);
    if (lane == 0) red[warp * G + q] = w;
  }
  asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
#pragma unroll
  for (int q = 0; q < G; ++q) v[q] = (red[q] + red[G + q]) + (red[2 * G + q] + red[3 * G + q]);
  asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
}

// exp2 of (z - m) with the conventions of the oracle: a masked position
// (z = -inf) gives 0 even when the running maximum is still -inf.
__device__ __forceinline__ float exp2_rel(float z, float m) {
  return (m == -INFINITY) ? 0.f : exp2f(z - m);
}

// Value loads (8 bytes: four channels of a position) in flight per thread while the tail is
// walked.  The walk is latency-bound, so this sets its number of round trips to memory; more
// than four in flight costs the tensor-core kernel's main loop registers (measured: 8 in flight
// +0.5 us, 16 in flight +2.8 us on a batch without any tail).
constexpr int kTailValueBatch = 4;

// Loads that say "shared" (through a generic pointer the compiler may not know the address is
// in shared memory, and a generic load costs more than twice the latency).
__device__ __forceinline__ uint32_t shared_address(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint4 lds_u4(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ float4 lds_f4(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ float lds_f1(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
  return v;
}

// A tail staged in shared memory by tensor copies with the 128-byte swizzle: two halves of
// [tokens][128 bytes] (channels 0-63, then 64-127; `half_bytes` apart), the 16-byte chunks of a
// row permuted by the row's low three bits - so a thread per token and a thread per channel
// both read without bank conflicts.  Address of byte `byte` (0..255) of token `t`'s row.
__device__ __forceinline__ const uint8_t* tail_staged_address(const uint8_t* staged, int half_bytes, int t,
                                                              int byte) {
  const int half = byte >> 7, in_half = byte & 127;
  return staged + half * half_bytes + t * 128 + ((((in_half >> 4) ^ (t & 7)) << 4) | (in_half & 15));
}

// The BF16 tail block, first half: thread = kv position.  Seeds the running max m and the
// per-thread partial sums l, and leaves P (rounded to BF16, as floats) in pf[G][128].
//   qb : [G][128] floats, the BF16 query of this KV head's G query heads
//   staged : null, or the tail's key rows already in shared memory in the layout of
//            tail_staged_address (the step's own token, if any, is not among them); P is then
//            left transposed, pf[position][G], for tail_pv_staged
// The code of the tail runs once per CTA, so it is fetched cold: where the rows are in shared
// memory (kStaged) the loop over the row's chunks stays rolled - unrolled, fetching its
// instructions took longer (3 us) than executing them.
template <int G, bool kStaged = false>
__device__ __forceinline__ void tail_scores(const DecodeParams& p, const TileWork& w, const float* qb,
                                            float* pf, float* red, int tid, int bar_id,
                                            float (&m)[G], float (&l)[G], const uint8_t* staged = nullptr,
                                            int half_bytes = 0) {
  const int len = w.tail_len;
  const int64_t tok0 = (int64_t)w.tail_id * kPage;
  float z[G];
#pragma unroll
  for (int q = 0; q < G; ++q) z[q] = -INFINITY;
  if (tid < len) {
    const uint4* krow = reinterpret_cast<const uint4*>(
        p.tail_key + ((tok0 + tid) * p.heads_kv + w.kvh) * kHeadDim);
    // the step's own token sits at the tail's last position: it comes from the source (one BF16
    // subtract of the key shift, as the tail copy does it) and is stored for the steps to come
    const bool fresh = p.append_key != nullptr && tid == len - 1;
    const uint4* ksrc = fresh ? reinterpret_cast<const uint4*>(p.append_key + (int64_t)w.row * p.append_key_stride +
                                                               (int64_t)w.kvh * kHeadDim)
                              : nullptr;
    const uint4* shift = fresh && p.key_shift
                             ? reinterpret_cast<const uint4*>(p.key_shift + (int64_t)w.kvh * kHeadDim)
                             : nullptr;
    float acc[G];
#pragma unroll
    for (int q = 0; q < G; ++q) acc[q] = 0.f;
    if constexpr (kStaged) {
      // Rows in shared memory.  A warp issues in order, so a product right behind its load waits
      // out the load's latency every time (measured: 2.5 us for this loop): per chunk, the next
      // chunk's key load and all the query loads go first, the products after them.
      const uint32_t q_base = shared_address(qb);
      auto key_chunk = [&](int c) {
        uint4 k;
        if (fresh) {
          k = __ldg(ksrc + c);
          if (p.key_shift) {
            float x[8], y[8];
            unpack_bf16x8(k, x);
            unpack_bf16x8(__ldg(shift + c), y);
            uint32_t pk[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const __nv_bfloat16 a = __float2bfloat16_rn(x[2 * i] - y[2 * i]);
              const __nv_bfloat16 b = __float2bfloat16_rn(x[2 * i + 1] - y[2 * i + 1]);
              pk[i] = (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
            }
            k = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
          const_cast<uint4*>(krow)[c] = k;
        } else {
          k = lds_u4(shared_address(tail_staged_address(staged, half_bytes, tid, c * 16)));
        }
        return k;
      };
      constexpr int QC = G < 4 ? G : 4;   // query heads per batch of loads
      uint4 k_now = key_chunk(0);
#pragma unroll 1
      for (int c = 0; c < 16; ++c) {
        const uint4 k_next = c + 1 < 16 ? key_chunk(c + 1) : k_now;
        float kf[8];
        unpack_bf16x8(k_now, kf);
#pragma unroll
        for (int q0 = 0; q0 < G; q0 += QC) {
          float4 qa[QC], qc[QC];
#pragma unroll
          for (int i = 0; i < QC; ++i)
            if (q0 + i < G) {
              qa[i] = lds_f4(q_base + ((q0 + i) * kHeadDim + c * 8) * 4);
              qc[i] = lds_f4(q_base + ((q0 + i) * kHeadDim + c * 8 + 4) * 4);
            }
#pragma unroll
          for (int i = 0; i < QC; ++i)
            if (q0 + i < G) {
              float a = acc[q0 + i];
              a = fmaf(kf[0], qa[i].x, a); a = fmaf(kf[1], qa[i].y, a);
              a = fmaf(kf[2], qa[i].z, a); a = fmaf(kf[3], qa[i].w, a);
              a = fmaf(kf[4], qc[i].x, a); a = fmaf(kf[5], qc[i].y, a);
              a = fmaf(kf[6], qc[i].z, a); a = fmaf(kf[7], qc[i].w, a);
              acc[q0 + i] = a;
            }
        }
        k_now = k_next;
      }
    } else {
  #pragma unroll 4
      for (int c = 0; c < 16; ++c) {
        float kf[8];
        if (fresh) {
          uint4 k = __ldg(ksrc + c);
          if (p.key_shift) {
            float x[8], y[8];
            unpack_bf16x8(k, x);
            unpack_bf16x8(__ldg(shift + c), y);
            uint32_t pk[4];
  #pragma unroll
            for (int i = 0; i < 4; ++i) {
              const __nv_bfloat16 a = __float2bfloat16_rn(x[2 * i] - y[2 * i]);
              const __nv_bfloat16 b = __float2bfloat16_rn(x[2 * i + 1] - y[2 * i + 1]);
              pk[i] = (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
            }
            k = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
          const_cast<uint4*>(krow)[c] = k;
          unpack_bf16x8(k, kf);
        } else {
          unpack_bf16x8(__ldg(krow + c), kf);
        }
  #pragma unroll
        for (int q = 0; q < G; ++q) {
          const float4 qa = *reinterpret_cast<const float4*>(qb + q * kHeadDim + c * 8);
          const float4 qc = *reinterpret_cast<const float4*>(qb + q * kHeadDim + c * 8 + 4);
          acc[q] = fmaf(kf[0], qa.x, acc[q]); acc[q] = fmaf(kf[1], qa.y, acc[q]);
          acc[q] = fmaf(kf[2], qa.z, acc[q]); acc[q] = fmaf(kf[3], qa.w, acc[q]);
          acc[q] = fmaf(kf[4], qc.x, acc[q]); acc[q] = fmaf(kf[5], qc.y, acc[q]);
          acc[q] = fmaf(kf[6], qc.z, acc[q]); acc[q] = fmaf(kf[7], qc.w, acc[q]);
        }
      }
    }
#pragma unroll
    for (int q = 0; q < G; ++q) z[q] = acc[q] * p.scale_log2;
  }
  float bm[G];
#pragma unroll
  for (int q = 0; q < G; ++q) bm[q] = z[q];
  block_max_128<G>(bm, red, tid, bar_id);
#pragma unroll
  for (int q = 0; q < G; ++q) {
    m[q] = bm[q];
    const float pe = exp2_rel(z[q], bm[q]);
    l[q] = pe;
    // P of the tail meets V as BF16
    pf[kStaged ? tid * G + q : q * kHeadDim + tid] = __bfloat162float(__float2bfloat16_rn(pe));
  }
}

// Second half: o[q] = sum_t P[q][t] * V[t][d], and thread tid ends up with channel d = tid.
// The caller orders the pf writes of tail_scores before this; all 32 lanes of every calling
// warp must be here.  The walk is latency-bound, so it is laid out for few round trips: a lane
// takes four channels (8-byte loads) of every fourth position, kTailValueBatch loads in flight
// at a time, and the four position lanes of a channel group are folded by shuffles at the end.
// Positions past the tail length are never read, so stale or non-finite bytes there cannot
// reach the output (their P is zero and their V is taken as zero).
template <int G>
__device__ __forceinline__ void tail_pv_walk(const uint16_t* vbase, int64_t vstride, const uint16_t* vnew,
                                             int len, int fresh, const float* pf, int tid, float (&o)[G]) {
  constexpr int kChunk = G < 4 ? G : 4;   // query heads per pass over the tail
  const int plane = tid & 3;
#pragma unroll
  for (int q0 = 0; q0 < G; q0 += kChunk) {
    float acc[kChunk][4];
#pragma unroll
    for (int q = 0; q < kChunk; ++q)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[q][i] = 0.f;
#pragma unroll 1
    for (int jb = 0; jb < 32 && 4 * jb < len; jb += kTailValueBatch) {
      uint2 v[kTailValueBatch];
#pragma unroll
      for (int j = 0; j < kTailValueBatch; ++j) {
        const int t = plane + 4 * (jb + j);
        v[j] = make_uint2(0u, 0u);
        if (t < len)
          v[j] = __ldg(reinterpret_cast<const uint2*>(t == fresh ? vnew : vbase + t * vstride));
      }
#pragma unroll
      for (int j = 0; j < kTailValueBatch; ++j) {
        const int t = plane + 4 * (jb + j);
        if (q0 == 0 && t == fresh)
          *reinterpret_cast<uint2*>(const_cast<uint16_t*>(vbase) + t * vstride) = v[j];
        const float vf[4] = {__uint_as_float(v[j].x << 16), __uint_as_float(v[j].x & 0xffff0000u),
                             __uint_as_float(v[j].y << 16), __uint_as_float(v[j].y & 0xffff0000u)};
#pragma unroll
        for (int q = 0; q < kChunk; ++q) {
          if (q0 + q >= G) continue;   // a group size that is no multiple of the chunk
          const float pw = pf[(q0 + q) * kHeadDim + t];
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[q][i] = fmaf(pw, vf[i], acc[q][i]);
        }
      }
    }
    // fold the four position lanes; lane `plane` keeps channel ch0 + plane, which is channel tid
    const bool up2 = (plane & 2) != 0, up1 = (plane & 1) != 0;
#pragma unroll
    for (int q = 0; q < kChunk; ++q) {
      float k0 = up2 ? acc[q][2] : acc[q][0], k1 = up2 ? acc[q][3] : acc[q][1];
      const float s0 = up2 ? acc[q][0] : acc[q][2], s1 = up2 ? acc[q][1] : acc[q][3];
      k0 += __shfl_xor_sync(0xffffffffu, s0, 2);
      k1 += __shfl_xor_sync(0xffffffffu, s1, 2);
      float r = up1 ? k1 : k0;
      const float s = up1 ? k0 : k1;
      r += __shfl_xor_sync(0xffffffffu, s, 1);
      if (q0 + q < G) o[q0 + q] = r;
    }
  }
}

template <int G>
__device__ __forceinline__ void tail_pv(const DecodeParams& p, const TileWork& w, const float* pf,
                                        int tid, float (&o)[G]) {
  const int len = w.tail_len;
  const int ch0 = (tid & ~31) + ((tid & 31) >> 2) * 4;
  const int64_t tok0 = (int64_t)w.tail_id * kPage;
  const int64_t vstride = (int64_t)p.heads_kv * kHeadDim;
  const uint16_t* vbase = p.tail_value + (tok0 * p.heads_kv + w.kvh) * kHeadDim + ch0;
  // with the step's own token given, the last position comes from the source and is stored
  const int fresh = p.append_value != nullptr ? len - 1 : -1;
  const uint16_t* vnew = p.append_value != nullptr
                             ? p.append_value + (int64_t)w.row * p.append_value_stride +
                                   (int64_t)w.kvh * kHeadDim + ch0
                             : nullptr;
  tail_pv_walk<G>(vbase, vstride, vnew, len, fresh, pf, tid, o);
}

// The second half out of shared memory: the tail's value rows were staged there in the layout of
// tail_staged_address, P lies transposed (pf[position][G]).  Thread tid is channel tid; the step's
// own token, if any, comes from the source and is stored to the tail page, as in tail_pv.
template <int G>
__device__ __forceinline__ void tail_pv_staged(const DecodeParams& p, const TileWork& w, const float* pf,
                                               const uint8_t* staged, int half_bytes, int tid, float (&o)[G]) {
  const int len = w.tail_len;
  const int fresh = p.append_value != nullptr ? len - 1 : -1;
  float v_fresh = 0.f;
  if (fresh >= 0) {
    const uint16_t raw = __ldg(p.append_value + (int64_t)w.row * p.append_value_stride +
                               (int64_t)w.kvh * kHeadDim + tid);
    const_cast<uint16_t*>(p.tail_value)[(((int64_t)w.tail_id * kPage + fresh) * p.heads_kv + w.kvh) * kHeadDim + tid] = raw;
    v_fresh = __uint_as_float((uint32_t)raw << 16);
  }
#pragma unroll
  for (int q = 0; q < G; ++q) o[q] = 0.f;
  const int body = fresh >= 0 ? len - 1 : len;
  // this thread's two bytes of row t sit at base + t * 128 + ((chunk ^ (t & 7)) << 4): eight
  // rows at a time, so that the permutation is a constant per unrolled step
  const int chunk = (tid & 63) >> 3;
  const uint32_t base = shared_address(staged + (tid >> 6) * half_bytes + (tid & 7) * 2);
  const uint32_t pbase = shared_address(pf);
  // full groups of eight rows: the eight loads first, then the products (with a test per row in
  // between, every row waited for its own load: 100 cycles a row); then the rows left over
  int t0 = 0;
  for (; t0 + 8 <= body; t0 += 8) {
    uint32_t raw[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) raw[j] = lds_u16(base + (t0 + j) * 128 + ((chunk ^ j) << 4));
    if constexpr (G == 4) {
      float4 w4[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) w4[j] = lds_f4(pbase + (t0 + j) * 16);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float vf = __uint_as_float(raw[j] << 16);
        o[0] = fmaf(w4[j].x, vf, o[0]);
        o[1] = fmaf(w4[j].y, vf, o[1]);
        o[2] = fmaf(w4[j].z, vf, o[2]);
        o[3] = fmaf(w4[j].w, vf, o[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float vf = __uint_as_float(raw[j] << 16);
        const uint32_t pw = pbase + (t0 + j) * G * 4;
        float wq[G];
#pragma unroll
        for (int q = 0; q < G; ++q) wq[q] = lds_f1(pw + q * 4);
#pragma unroll
        for (int q = 0; q < G; ++q) o[q] = fmaf(wq[q], vf, o[q]);
      }
    }
  }
#pragma unroll 1
  for (int t = t0; t < body; ++t) {
    const float vf = __uint_as_float(lds_u16(base + t * 128 + ((chunk ^ (t & 7)) << 4)) << 16);
#pragma unroll
    for (int q = 0; q < G; ++q) o[q] = fmaf(lds_f1(pbase + (t * G + q) * 4), vf, o[q]);
  }
  if (fresh >= 0) {
#pragma unroll
    for (int q = 0; q < G; ++q) o[q] = fmaf(pf[fresh * G + q], v_fresh, o[q]);
  }
}

// Both halves on the same 128 threads (the CUDA-core kernel).
template <int G>
__device__ __forceinline__ void tail_block(const DecodeParams& p, const TileWork& w, const float* qb,
                                           float* pf, float* red, int tid, int bar_id,
                                           float (&m)[G], float (&l)[G], float (&o)[G]) {
  tail_scores<G>(p, w, qb, pf, red, tid, bar_id, m, l);
  asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
  tail_pv<G>(p, w, pf, tid, o);
  asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
}

// Normalise and store.  l holds per-thread partial sums; o per-channel sums.
template <int G>
__device__ __forceinline__ void write_output(const DecodeParams& p, const TileWork& w, float* red,
                                             int tid, int bar_id, const float (&m)[G],
                                             float (&l)[G], const float (&o)[G]) {
  block_sum_128<G>(l, red, tid, bar_id);
#pragma unroll
  for (int q = 0; q < G; ++q) {
    const int head = w.kvh * G + q;
    const float val = l[q] > 0.f ? __fdiv_rn(o[q], l[q]) : 0.f;
    if (p.emit_partial) {
      const int64_t idx = w.slot * p.heads_q + head;
      p.o_partial[idx * kHeadDim + tid] = val;
      if (tid == 0)
        p.lse_partial[idx] = l[q] > 0.f ? (m[q] + log2f(l[q])) * kLn2 : -INFINITY;
    } else {
      const int64_t orow = p.out_indices ? (int64_t)p.out_indices[w.row] : (int64_t)w.row;
      p.out[(orow * p.heads_q + head) * kHeadDim + tid] =
          __bfloat16_as_ushort(__float2bfloat16_rn(val));
    }
  }
}

}  // namespace nvfp4
