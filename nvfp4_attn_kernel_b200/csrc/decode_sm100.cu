// Tensor-core decode kernel for sm_100a: block-scaled tcgen05 MMA (kind::mxf4nvf4,
// E2M1 operands with UE4M3 scales per 16 elements), accumulators in tensor memory,
// K/V page tiles staged by TMA through a ring of shared-memory stages.
//
// One CTA of 384 threads per (split, KV head, row):
//   warps 0-3  score threads: read S^T from tensor memory, online softmax, P -> NVFP4
//   warps 4-7  output threads: fold each page's O^T into the running output, epilogue
//   warp  8    K producer: page-table walk, TMA loads of the K tiles, bulk copies of their scales
//   warp  9    issuer of S^T = K . Q^T (one elected lane), owner of the tensor-memory allocation
//   warp 10    issuer of O^T = V^T . P^T (one elected lane)
//   warp 11    V producer: the same walk for the V tiles and their scales
//
// K and V travel through separate rings.  A K slot is handed back as soon as K . Q^T of its
// page has retired, a V slot only after V^T . P^T, two hand-overs later: with one ring a page's
// K would sit in shared memory for all of that time, and the bytes in flight per CTA (which,
// over the memory latency, set the rate a CTA can stream at) would shrink by as much.
//
// The product is formed transposed so that the G query heads of a KV head are the N side of
// the MMA (N = 8 for G <= 8, else N = G = 16 or 32) and nothing is padded to 128:
//   S^T[128 kv, N q] = K_page[128 kv, 128 d] . Q^T            (A = K tile as it lies in the page)
//   O^T[128 d , N q] = V_page^T[128 d, 128 kv] . P^T          (A = V tile as it lies in the page)
// Both page layouts are already K-major A operands, and the 512-byte scale atoms of the
// page format are copied to tensor memory with tcgen05.cp unchanged.
// An output thread is channel t for every query head, so the running output lives in G
// registers per thread and O^T is never rescaled in tensor memory: each page's P.V lands
// in a fresh accumulator and is folded in as o = o * rescale + O_page, exactly the order
// of the attention oracle.
//
// Two forms of the kernel.  The narrow one (kGroups = 1, 384 threads) is built for two CTAs per SM
// and is what a launch that fills the GPU twice over runs on: there the page stream is bound by
// HBM.  A launch with at most one CTA per SM is bound by a CTA's own page period instead - the
// chain scores -> maximum -> exp2 -> quantise -> hand-over through the four score warps - so the
// wide form (kGroups = 2, 640 threads, one CTA per SM, deeper rings, 128 registers per thread)
// has a second pair of issuing threads and a second group of four score warps (measured: with an
// SM to itself a CTA's period was the 1800 cycles per pair of pages that ONE thread needs to issue
// the waits, scale copies, products and commits of V^T . P^T): the hand-overs alternate between
// the two sets of issuers and score warps, and since
// a page's probabilities are quantised against the running maximum of everything walked before
// it, a group passes the maximum on (per warp, through shared memory) as soon as it has its own
// pages' maxima, before it goes on to exp2 and the quantisation.  The rescale factors per page,
// and with them the folded output, are those of the narrow form; only the row sum is kept in two
// parts that are joined at the end.
//
// A tile's BF16 tail is processed first, out of shared memory: its key rows, then its value rows,
// are fetched by tensor copies into the last slots of the V ring (see kTailSlots).  With a work
// list (balanced split) a row's tail is an entry of its own, served by tail_piece without any of
// the page machinery, and the pieces of a row are merged by a later launch or, on request, by
// the piece that finishes last (finish_piece).
//
// Every device-side wait is bounded; on expiry the CTA raises NVFP4_STATUS_WAIT_TIMEOUT,
// drains what it has in flight, frees its tensor memory and returns.
#include <cstring>

#include "sm100_device.cuh"

namespace nvfp4 {

namespace sm100 {

// Ring depths: as many 9 KB slots as two resident CTAs per SM leave room for.  V slots are
// held about two pages longer than K slots, so the V ring is that much deeper.
template <int G, int kGroups> struct KSlots {
  static constexpr int value = kGroups == 2 ? (G <= 8 ? 8 : 6) : G <= 4 ? 4 : G <= 8 ? 3 : 2;
};
template <int G, int kGroups> struct VSlots {
  static constexpr int value = kGroups == 2 ? (G <= 4 ? 12 : G <= 8 ? 10 : G <= 16 ? 8 : 6)
                                            : G <= 4 ? 6 : G <= 8 ? 5 : G <= 16 ? 3 : 2;
};
// pages handled per hand-over: two, except where 32 query slots leave tensor memory for one
template <int G> struct Batch { static constexpr int value = G <= 16 ? 2 : 1; };
// MMA N (query slots): 8 covers every group size up to 8; a group of 16 takes N = 16
template <int G> struct QuerySlots { static constexpr int value = G <= 8 ? 8 : G; };

// tensor-memory column map (32-bit columns); a "set" holds the pages of one hand-over
template <int G, int kGroups>
struct Cols {
  static constexpr int NQ = QuerySlots<G>::value;
  static constexpr int kBatch = Batch<G>::value;
  static constexpr int kSet = kBatch * NQ;       // columns of one set of S^T (or O^T)
  static constexpr int kS = 0;                   // 2 sets x 2 pages x NQ : S^T
  static constexpr int kO = 2 * kSet;            // 2 sets x 2 pages x NQ : per-page O^T
  // scale columns of the operands an issuer copies right before its products: one block of 8
  // (2 k-blocks x 4) per issuer of the kind (the wide form has two of each)
  static constexpr int kSfQ = 4 * kSet;
  static constexpr int kSfK = kSfQ + 8 * kGroups;
  static constexpr int kSfP = kSfK + 8 * kGroups;
  static constexpr int kSfV = kSfP + 16;         // 2 sets x 2 pages x 8 : copied as soon as the V slot has landed
  static constexpr int kUsed = kSfV + 2 * kBatch * 8;
  static constexpr int kAlloc = kUsed <= 128 ? 128 : 256;   // a power of two
  static_assert(kUsed <= 256, "two CTAs per SM leave 256 tensor-memory columns each");
  static_assert(kGroups == 1 || kSfP + 16 >= kSfP + 8 * kGroups, "scale columns of the second P issuer");
};

// The tensor maps of a launch: K and V page tiles, and the BF16 tail caches (unused without tails).
struct TileMaps {
  CUtensorMap k, v, tail_k, tail_v;
};

// The BF16 tail of a tile that also walks pages is staged in shared memory too: its key rows,
// then its value rows, are fetched by bulk copies (one round trip each instead of a dozen
// through registers) into the LAST kTailSlots slots of the V ring, which the V producer leaves
// alone until the tail is consumed.
constexpr int kTailPitch = kHeadDim + 8;   // elements; rows 272 bytes apart: 16-byte aligned, no bank conflicts
constexpr int kTailSlots = (2 * kPage * 128 + kSlotBytes - 1) / kSlotBytes;   // 4: a full tail's 32 KB

template <int G, int kGroups>
struct __align__(1024) Smem {
  static constexpr int kKS = KSlots<G, kGroups>::value, kVS = VSlots<G, kGroups>::value;
  uint8_t k_slot[kKS][kSlotBytes];              // K tile | K scales
  uint8_t v_slot[kVS][kSlotBytes];              // V tile | V scales
  static constexpr int NQ = QuerySlots<G>::value;
  static constexpr int kBatch = Batch<G>::value;
  __align__(1024) uint8_t q_tile[NQ * 64];      // NQ rows x 64 B, 64-byte swizzle
  __align__(1024) uint8_t p_tile[2][kBatch][NQ * 64];
  __align__(512) uint8_t q_sf[kSfBlockBytes];
  __align__(512) uint8_t p_sf[2][kBatch][kSfBlockBytes];
  __align__(16) float qb[G * kHeadDim];         // BF16 query as floats (tail)
  __align__(16) float pf[G * kHeadDim];         // P of the tail block
  __align__(16) float z[2][kBatch][G * kPage];  // scaled scores, [set][page][q][kv position]
  float resc[8][NQ];                            // ring of per-page rescale factors, [page & 7][q]
  float red_io[4 * NQ];                         // reductions of the tail block
  float fin[2][2 * NQ];                         // per score group: row sums and the maxima they refer to
  volatile float m_val[2][NQ];                  // running maximum handed from one score group to the other, [pairs done & 1]
  volatile int m_seq[4];                        // [score warp] pairs whose maximum m_val already holds
  volatile uint8_t page_ok[32];                 // [walk step & 31] 0: the page id was refused
  __align__(8) uint64_t k_full[kKS];
  uint64_t k_empty[kKS], v_full[kVS], v_empty[kVS];
  uint64_t s_full[2], s_free[2], p_full[2], o_full[2], o_free[2];
  uint64_t q_ready, drain[4];
  uint64_t tail_full, tail_done;                // the BF16 tail staged in the V ring's last slots (see kTailSlots)
  uint32_t tmem_base;
  volatile int abort_flag;
  volatile int xchg_last, xchg_ready;           // hand-overs among the output threads during the exchange
};


// Cross-GPU exchange of a finished (row, KV head) tile, run by the 128 output threads (thread t
// is channel t) of the CTA that stored the tile's last split partial.  Local splits are folded in
// index order; the result goes into this tile's slots of every peer's inbox with posted remote
// stores, then one flag per (peer, head); the wait (bounded) is for the peers' flags of the same
// heads only; the merge reads this GPU's own inbox, in rank order, like push_merge_kernel.
template <int G, class SM>
__device__ __forceinline__ void exchange_tile(const DecodeParams& p, const TileWork& w, SM& sm, int t,
                                              bool stored, int epoch) {
  const int tiles = p.rows * p.heads_kv, tile = w.row * p.heads_kv + w.kvh;
  __threadfence();   // this CTA's partial is visible before its arrival is counted
  asm volatile("bar.sync 6, 128;" ::: "memory");
  if (t == 0) {
    // every split counts its arrival, stored or not (a split whose wait expired marks the count
    // failed): the tile always completes, its counter returns to zero and the epoch advances, so
    // one expired wait cannot leave stale counts behind for the launches that follow
    const int seen = atomicAdd(p.xchg_counters + tile, stored ? 1 : 0x10001);
    const bool last = (seen & 0xffff) == p.num_splits - 1;
    sm.xchg_last = last ? (((seen >> 16) == 0 && stored) ? 1 : 2) : 0;   // 2: complete, but a split failed
    sm.xchg_ready = 1;
  }
  asm volatile("bar.sync 6, 128;" ::: "memory");
  if (!sm.xchg_last) return;
  __threadfence();
  if (t == 0) p.xchg_counters[tile] = 0;   // ready for the next launch
  if (sm.xchg_last == 2) {
    // nothing to fold or to push: the status word says why, the peers' waits for this tile run
    // out with a status of their own; the launch still counts the tile as done
    if (t == 0) {
      set_status(p.status, NVFP4_STATUS_WAIT_TIMEOUT);
      if (atomicAdd(p.xchg_epoch_state + 1, 1) == tiles - 1) {
        p.xchg_epoch_state[1] = 0;
        __threadfence();
        *reinterpret_cast<volatile int*>(p.xchg_epoch_state) = epoch;
      }
    }
    return;
  }
  const int rank = p.xchg_rank, world = p.xchg_world;
  const int64_t pairs = (int64_t)p.rows * p.heads_q;
  const int64_t copy_elems = (int64_t)world * pairs * kInboxStride;
  const int64_t idx0 = (int64_t)w.row * p.heads_q + w.kvh * G;   // first of the tile's G (row, head) pairs

  // The splits' LSEs are the same for all 128 threads: each thread fetches one of them into
  // shared memory (one round trip for all), and the partial outputs are loaded a batch at a
  // time (all heads, CH splits) so that their latencies overlap.  The accumulation itself runs
  // in split order with the arithmetic of lse_merge_kernel.
  constexpr int CH = G >= 8 ? 2 : 4;
  float* lse_sh = &sm.z[0][0][0];   // the score buffer is idle by now; room for 128 values and more
  const int n_lse = p.num_splits * G;
  for (int i = t; i < n_lse; i += 128)
    lse_sh[i] = __ldcg(p.lse_partial + (i / G) * pairs + idx0 + (i % G));
  asm volatile("bar.sync 6, 128;" ::: "memory");
  float my_o[G], my_lse[G], mx[G], acc[G], tot[G];
#pragma unroll
  for (int q = 0; q < G; ++q) { mx[q] = -INFINITY; acc[q] = 0.f; tot[q] = 0.f; }
  for (int s = 0; s < p.num_splits; ++s)
#pragma unroll
    for (int q = 0; q < G; ++q) mx[q] = fmaxf(mx[q], lse_sh[s * G + q]);
  for (int s0 = 0; s0 < p.num_splits; s0 += CH) {
    float ov[G][CH];
#pragma unroll
    for (int q = 0; q < G; ++q)
#pragma unroll
      for (int j = 0; j < CH; ++j)
        ov[q][j] = s0 + j < p.num_splits ? __ldcg(p.o_partial + ((s0 + j) * pairs + idx0 + q) * kHeadDim + t) : 0.f;
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      if (s0 + j >= p.num_splits) break;
#pragma unroll
      for (int q = 0; q < G; ++q) {
        const float ls = lse_sh[(s0 + j) * G + q];
        if (ls == -INFINITY) continue;   // an empty split weighs nothing, whatever its O holds
        const float wgt = expf(ls - mx[q]);
        tot[q] += wgt;
        acc[q] = fmaf(wgt, ov[q][j], acc[q]);
      }
    }
  }
#pragma unroll
  for (int q = 0; q < G; ++q) {
    my_o[q] = tot[q] > 0.f ? __fdiv_rn(acc[q], tot[q]) : 0.f;
    my_lse[q] = tot[q] > 0.f ? mx[q] + logf(tot[q]) : -INFINITY;
  }
  const int64_t slot0 = (epoch & 1) * copy_elems + ((int64_t)rank * pairs + idx0) * kInboxStride;
  for (int peer = 0; peer < world; ++peer) {
    if (peer == rank) continue;
    float* dst = p.xchg_inbox[peer] + slot0;
#pragma unroll
    for (int q = 0; q < G; ++q) {
      st_relaxed_sys(dst + q * kInboxStride + t, my_o[q]);
      if (t == 0) st_relaxed_sys(dst + q * kInboxStride + kHeadDim, my_lse[q]);
    }
  }
  asm volatile("bar.sync 6, 128;" ::: "memory");
  // thread j < world * G looks after (peer j / G, head j % G): announce, then wait for its push.
  // The release at system scope is cumulative over what the barrier ordered before it, so the
  // 128 threads' stores above are visible to whoever acquires the flag.
  const int peer = t / G, q_mine = t % G;
  if (peer < world && peer != rank) {
    st_release_sys(p.xchg_flags[peer] + (int64_t)rank * pairs + idx0 + q_mine, epoch);
    const int* flag = p.xchg_flags[rank] + (int64_t)peer * pairs + idx0 + q_mine;
    const unsigned long long t0 = sm100::global_ns();
    // epochs only grow; a peer that is already a step ahead has certainly pushed this one
    while (ld_acquire_sys(flag) - epoch < 0) {
      if (sm100::global_ns() - t0 > kPeerWaitNs) {
        set_status(p.status, NVFP4_STATUS_WAIT_TIMEOUT);
        sm.xchg_ready = 0;
        break;
      }
      __nanosleep(32);
    }
  }
  asm volatile("bar.sync 6, 128;" ::: "memory");
  if (sm.xchg_ready) {   // else the output is left untouched and the status word says why
    const float* mine = p.xchg_inbox[rank] + (epoch & 1) * copy_elems;
    float gm[G], a2[G], t2[G];
#pragma unroll
    for (int q = 0; q < G; ++q) { gm[q] = -INFINITY; a2[q] = 0.f; t2[q] = 0.f; }
    for (int s0 = 0; s0 < world; s0 += CH) {
      float ls[G][CH];
#pragma unroll
      for (int q = 0; q < G; ++q)
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          const int s = s0 + j;
          ls[q][j] = s >= world ? -INFINITY
                     : s == rank ? my_lse[q]
                                 : ld_relaxed_sys(mine + ((int64_t)s * pairs + idx0 + q) * kInboxStride + kHeadDim);
        }
#pragma unroll
      for (int q = 0; q < G; ++q)
#pragma unroll
        for (int j = 0; j < CH; ++j) gm[q] = fmaxf(gm[q], ls[q][j]);
    }
    for (int s0 = 0; s0 < world; s0 += CH) {
      float ls[G][CH], ov[G][CH];
#pragma unroll
      for (int q = 0; q < G; ++q)
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          const int s = s0 + j;
          const float* src = mine + ((int64_t)s * pairs + idx0 + q) * kInboxStride;
          ls[q][j] = s >= world ? -INFINITY : s == rank ? my_lse[q] : ld_relaxed_sys(src + kHeadDim);
          ov[q][j] = s >= world ? 0.f : s == rank ? my_o[q] : ld_relaxed_sys(src + t);
        }
#pragma unroll
      for (int q = 0; q < G; ++q)
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          if (ls[q][j] == -INFINITY) continue;
          const float wgt = expf(ls[q][j] - gm[q]);
          t2[q] += wgt;
          a2[q] = fmaf(wgt, ov[q][j], a2[q]);
        }
    }
#pragma unroll
    for (int q = 0; q < G; ++q) {
      const float val = t2[q] > 0.f ? __fdiv_rn(a2[q], t2[q]) : 0.f;
      const int64_t at = (idx0 + q) * kHeadDim + t;
      if (p.xchg_out_f32) static_cast<float*>(p.xchg_out)[at] = val;
      else static_cast<uint16_t*>(p.xchg_out)[at] = __bfloat16_as_ushort(__float2bfloat16_rn(val));
    }
  }
  if (t == 0 && atomicAdd(p.xchg_epoch_state + 1, 1) == tiles - 1) {
    p.xchg_epoch_state[1] = 0;
    __threadfence();
    *reinterpret_cast<volatile int*>(p.xchg_epoch_state) = epoch;
  }
}

// In-launch merge of a row's pieces (work list only).  Called by 128 threads (thread t is
// channel t) right after they stored their piece's partial: the piece of a (row, KV head) that
// arrives last folds the partials of all the row's pieces into the BF16 output, with the
// arithmetic and in the order of the merge launch (lse_merge_ranges_kernel), so the bits are
// the same whichever piece happens to be last.  No piece waits for another.
template <int G>
__device__ __forceinline__ void finish_piece(const DecodeParams& p, int row, int kvh, int t,
                                             volatile int& last_arrival) {
  __threadfence();   // this piece's partial is visible before its arrival is counted
  asm volatile("bar.sync 6, 128;" ::: "memory");
  const int count = __ldg(p.list_row_count + row);
  if (t == 0) {
    int* counter = p.list_counters + row * p.heads_kv + kvh;
    const int seen = atomicAdd(counter, 1);
    last_arrival = seen == count - 1;
    if (last_arrival) *counter = 0;   // ready for the next launch that reuses the list
  }
  asm volatile("bar.sync 6, 128;" ::: "memory");
  if (!last_arrival) return;
  __threadfence();
  const int first = __ldg(p.list_row_offset + row);
  const int64_t orow = p.out_indices ? (int64_t)p.out_indices[row] : (int64_t)row;
#pragma unroll 1
  for (int q = 0; q < G; ++q) {
    const int head = kvh * G + q;
    float mx = -INFINITY;
#pragma unroll 4
    for (int s = 0; s < count; ++s) mx = fmaxf(mx, __ldcg(p.lse_partial + (int64_t)(first + s) * p.heads_q + head));
    float acc = 0.f, tot = 0.f;
    if (mx != -INFINITY) {
#pragma unroll 4
      for (int s = 0; s < count; ++s) {
        const int64_t idx = (int64_t)(first + s) * p.heads_q + head;
        const float ls = __ldcg(p.lse_partial + idx);
        const float ov = __ldcg(p.o_partial + idx * kHeadDim + t);
        if (ls == -INFINITY) continue;
        const float wgt = expf(ls - mx);
        tot += wgt;
        acc = fmaf(wgt, ov, acc);
      }
    }
    const float val = tot > 0.f ? __fdiv_rn(acc, tot) : 0.f;
    p.out[(orow * p.heads_q + head) * kHeadDim + t] = __bfloat16_as_ushort(__float2bfloat16_rn(val));
  }
}

// ---- a work-list piece that holds nothing but a row's BF16 tail ----
// The balanced split lists a row's tail as a piece of its own.  Its CTA needs none of the page
// machinery (no ring, no tensor memory): every K and V row of the tail is fetched into shared
// memory with one bulk copy each, all of them in flight at once (one round trip to memory
// instead of the dozen a walk with loads into registers takes), and the scores, the softmax
// and P . V run out of shared memory.  Arithmetic as in tail_scores / tail_pv: BF16 query
// against BF16 keys, P rounded to BF16 before it meets V, the row sum over the unrounded P.

template <int G>
struct __align__(128) TailSmem {
  __align__(16) uint16_t k[kPage][kTailPitch];
  __align__(16) uint16_t v[kPage][kTailPitch];
  __align__(16) float qb[G * kHeadDim];   // the query as floats
  __align__(16) float pt[kPage * G];      // P, [position][query head]
  __align__(16) float o2[G * kHeadDim];   // the odd positions' share of the output
  float red[4 * G];
  float m[G], l[G];
  volatile int last_arrival;
  __align__(8) uint64_t bar;
};

template <int G, int kThreads>
__device__ __noinline__ void tail_piece(const DecodeParams& p, const TileWork& w, TailSmem<G>& ts) {
  static_assert(kThreads >= 384, "the copies, the fresh token and the query are spread over 384 threads");
  const int tid = threadIdx.x, len = w.tail_len;
  const int64_t tok0 = (int64_t)w.tail_id * kPage;
  // with the step's own token given, the tail's last position comes from the source (one BF16
  // subtract of the key shift, as the tail copy does it) and is stored for the steps to come
  const bool has_fresh = p.append_key != nullptr;
  const int copied = has_fresh ? len - 1 : len;
  if (tid == 0) {
    mbar_init(&ts.bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (copied > 0) mbar_expect_tx(&ts.bar, (uint32_t)copied * 2u * kHeadDim * 2u);
    else mbar_arrive(&ts.bar);
  }
  __syncthreads();
  if (tid < 2 * kPage) {
    const int t = tid & (kPage - 1);
    const bool is_v = tid >= kPage;
    if (t < copied) {
      const uint16_t* src = (is_v ? p.tail_value : p.tail_key) + ((tok0 + t) * p.heads_kv + w.kvh) * kHeadDim;
      bulk_load(smem_u32(is_v ? &ts.v[t][0] : &ts.k[t][0]), src, kHeadDim * 2, &ts.bar);
    }
  } else if (tid < 2 * kPage + 32) {
    if (has_fresh) {
      const int c = tid & 15;
      if (tid < 2 * kPage + 16) {
        uint4 k = __ldg(reinterpret_cast<const uint4*>(p.append_key + (int64_t)w.row * p.append_key_stride +
                                                       (int64_t)w.kvh * kHeadDim) + c);
        if (p.key_shift) {
          float x[8], y[8];
          unpack_bf16x8(k, x);
          unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(p.key_shift + (int64_t)w.kvh * kHeadDim) + c), y);
          uint32_t pk[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const __nv_bfloat16 a = __float2bfloat16_rn(x[2 * i] - y[2 * i]);
            const __nv_bfloat16 b = __float2bfloat16_rn(x[2 * i + 1] - y[2 * i + 1]);
            pk[i] = (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
          }
          k = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        reinterpret_cast<uint4*>(const_cast<uint16_t*>(p.tail_key) +
                                 ((tok0 + len - 1) * p.heads_kv + w.kvh) * kHeadDim)[c] = k;
        reinterpret_cast<uint4*>(&ts.k[len - 1][0])[c] = k;
      } else {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.append_value + (int64_t)w.row * p.append_value_stride +
                                                             (int64_t)w.kvh * kHeadDim) + c);
        reinterpret_cast<uint4*>(const_cast<uint16_t*>(p.tail_value) +
                                 ((tok0 + len - 1) * p.heads_kv + w.kvh) * kHeadDim)[c] = v;
        reinterpret_cast<uint4*>(&ts.v[len - 1][0])[c] = v;
      }
    }
  } else {
    for (int it = tid - (2 * kPage + 32); it < G * 16; it += kThreads - (2 * kPage + 32)) {
      const int q = it >> 4, c = it & 15;
      float f[8];
      if (p.q_bf16) {
        unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(p.q_bf16 + (int64_t)w.row * p.q_row_stride +
                                                           (int64_t)(w.kvh * G + q) * p.q_head_stride + c * 8)), f);
      } else {
        // no BF16 query supplied: the tail meets the dequantised NVFP4 query
        const uint32_t pk = *reinterpret_cast<const uint32_t*>(
            p.q_fp4 + ((int64_t)w.row * p.heads_q + w.kvh * G + q) * 64 + c * 4);
        const float sc = e4m3_to_f32(p.q_sf[(int64_t)w.row * p.heads_q * kSfBlockBytes +
                                            (int64_t)w.kvh * kSfBlockBytes + sf_offset(q, c >> 1)]);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = e2m1_to_f32((pk >> (4 * i)) & 15u) * sc;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ts.qb[q * kHeadDim + c * 8 + i] = f[i];
    }
  }
  // bounded wait for the copies; a CTA whose wait expired stores the empty partial
  bool landed = mbar_try(&ts.bar, 0);
  if (!landed) {
    const unsigned long long t0 = global_ns();
    uint32_t spins = 0;
    while (!(landed = mbar_try(&ts.bar, 0)))
      if ((++spins & 1023u) == 0 && global_ns() - t0 > kWaitLimitNs) break;
  }
  landed = __syncthreads_and(landed) != 0;   // also: query and fresh rows visible
  if (!landed) {
    if (tid == 0) set_status(p.status, NVFP4_STATUS_WAIT_TIMEOUT);
    if (tid < kHeadDim) {
#pragma unroll
      for (int q = 0; q < G; ++q) {
        const int64_t idx = w.slot * p.heads_q + w.kvh * G + q;
        p.o_partial[idx * kHeadDim + tid] = 0.f;
        if (tid == 0) p.lse_partial[idx] = -INFINITY;
      }
      if (p.list_counters) finish_piece<G>(p, w.row, w.kvh, tid, ts.last_arrival);
    }
    return;
  }
  if (tid < kPage) {   // thread = position
    float z[G];
#pragma unroll
    for (int q = 0; q < G; ++q) z[q] = -INFINITY;
    if (tid < len) {
      float acc[G];
#pragma unroll
      for (int q = 0; q < G; ++q) acc[q] = 0.f;
#pragma unroll 4
      for (int c = 0; c < 16; ++c) {
        float kf[8];
        unpack_bf16x8(*reinterpret_cast<const uint4*>(&ts.k[tid][c * 8]), kf);
#pragma unroll
        for (int q = 0; q < G; ++q) {
          const float4 qa = *reinterpret_cast<const float4*>(ts.qb + q * kHeadDim + c * 8);
          const float4 qc = *reinterpret_cast<const float4*>(ts.qb + q * kHeadDim + c * 8 + 4);
          acc[q] = fmaf(kf[0], qa.x, acc[q]); acc[q] = fmaf(kf[1], qa.y, acc[q]);
          acc[q] = fmaf(kf[2], qa.z, acc[q]); acc[q] = fmaf(kf[3], qa.w, acc[q]);
          acc[q] = fmaf(kf[4], qc.x, acc[q]); acc[q] = fmaf(kf[5], qc.y, acc[q]);
          acc[q] = fmaf(kf[6], qc.z, acc[q]); acc[q] = fmaf(kf[7], qc.w, acc[q]);
        }
      }
#pragma unroll
      for (int q = 0; q < G; ++q) z[q] = acc[q] * p.scale_log2;
    }
    float m[G], l[G];
#pragma unroll
    for (int q = 0; q < G; ++q) m[q] = z[q];
    block_max_128<G>(m, ts.red, tid, 1);
#pragma unroll
    for (int q = 0; q < G; ++q) {
      const float pe = exp2_rel(z[q], m[q]);
      l[q] = pe;
      ts.pt[tid * G + q] = __bfloat162float(__float2bfloat16_rn(pe));   // P of the tail meets V as BF16
    }
    block_sum_128<G>(l, ts.red, tid, 1);
    if (tid == 0) {
#pragma unroll
      for (int q = 0; q < G; ++q) { ts.m[q] = m[q]; ts.l[q] = l[q]; }
    }
  }
  __syncthreads();
  // P . V: thread (half, channel) takes every other position; the halves are joined below
  const int half = tid >> 7, d = tid & (kHeadDim - 1);
  float o[G];
#pragma unroll
  for (int q = 0; q < G; ++q) o[q] = 0.f;
  if (half < 2) {
    for (int t = half; t < len; t += 2) {
      const float vf = __uint_as_float((uint32_t)ts.v[t][d] << 16);
#pragma unroll
      for (int q = 0; q < G; ++q) o[q] = fmaf(ts.pt[t * G + q], vf, o[q]);
    }
    if (half == 1) {
#pragma unroll
      for (int q = 0; q < G; ++q) ts.o2[q * kHeadDim + d] = o[q];
    }
  }
  __syncthreads();
  if (half == 0) {
#pragma unroll
    for (int q = 0; q < G; ++q) {
      const float lq = ts.l[q];
      const float val = lq > 0.f ? __fdiv_rn(o[q] + ts.o2[q * kHeadDim + d], lq) : 0.f;
      const int64_t idx = w.slot * p.heads_q + w.kvh * G + q;
      p.o_partial[idx * kHeadDim + d] = val;
      if (d == 0) p.lse_partial[idx] = lq > 0.f ? (ts.m[q] + log2f(lq)) * kLn2 : -INFINITY;
    }
    if (p.list_counters) finish_piece<G>(p, w.row, w.kvh, d, ts.last_arrival);
  }
}

// narrow: 12 warps; wide: plus a second group of four score warps (12-15), a second pair of
// issuers (16, 17) and a second pair of producers (18, 19)
// The wide form's second producers and issuers shorten the page period of a CTA whose score work
// is light; with 16 or 32 query heads per KV head the score threads bound the period, and what
// those instantiations need is registers: they run without the four extra warps, 512 threads at
// 128 registers instead of 640 at 96.
template <int G, int kGroups> struct SecondSet { static constexpr bool value = kGroups == 2 && G < 16; };
template <int G, int kGroups> struct ThreadsOf {
  static constexpr int value = kGroups == 1 ? 384 : SecondSet<G, kGroups>::value ? 640 : 512;
};

template <int G, int kGroups>
__global__ void __launch_bounds__(ThreadsOf<G, kGroups>::value, kGroups == 1 ? 2 : 1)
decode_sm100_kernel(const __grid_constant__ TileMaps maps, const __grid_constant__ DecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  Smem<G, kGroups>& sm =
      *reinterpret_cast<Smem<G, kGroups>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kThreads = ThreadsOf<G, kGroups>::value;
  constexpr bool kSecond = SecondSet<G, kGroups>::value;   // second producers (warps 18, 19) and issuers (16, 17)
  constexpr int kIssuers = kSecond ? 2 : 1;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int kKS = KSlots<G, kGroups>::value, kVS = VSlots<G, kGroups>::value;
  constexpr int NQ = QuerySlots<G>::value;
  constexpr int kBatch = Batch<G>::value;
  using C = Cols<G, kGroups>;

  // Which work this CTA has.  With a work list (balanced split) the entry says so; otherwise the
  // block index does.  row_of_block is what the early page-table fetch below may use before the
  // row's lengths are known.
  int row_of_block = blockIdx.z;
  int4 entry = make_int4(0, 0, 0, 0);
  if (p.work_list) {
    entry = __ldg(p.work_list + blockIdx.y);   // the grid is (KV heads, list entries)
    if (entry.x < 0) return;   // past the end of the list
    row_of_block = entry.x;
  }
  // a work-list entry is either some of a row's pages (entry.w = 0) or the row's tail alone (1)
  auto resolve = [&]() {
    return p.work_list ? resolve_work(p, entry.x, blockIdx.x, entry.y, entry.z, (int64_t)blockIdx.y,
                                      entry.w ? kTailOnly : kPagesOnly)
                       : resolve_grid_work(p);
  };
  // A split of a short row often owns no page at all (the split count follows the longest row of
  // the batch): such a CTA stores the empty partial and leaves before any set-up.  Only on the
  // split path without the cross-GPU exchange, which counts the arrival of every split.
  if ((p.num_splits > 1 || p.work_list) && p.emit_partial && !p.xchg_inbox) {
    const TileWork w0 = resolve();
    if (w0.last_page == w0.first_page && w0.tail_len == 0) {
      if (tid < kHeadDim) {
#pragma unroll
        for (int q = 0; q < G; ++q) {
          const int64_t idx = w0.slot * p.heads_q + w0.kvh * G + q;
          p.o_partial[idx * kHeadDim + tid] = 0.f;
          if (tid == 0) p.lse_partial[idx] = -INFINITY;
        }
        if (p.work_list && p.list_counters) finish_piece<G>(p, w0.row, w0.kvh, tid, sm.xchg_last);
      }
      return;
    }
    if (p.work_list && entry.w) {
      static_assert(sizeof(TailSmem<G>) <= sizeof(Smem<G, kGroups>), "the tail piece lives in the ring's memory");
      tail_piece<G, kThreads>(p, w0, *reinterpret_cast<TailSmem<G>*>(&sm));
      return;
    }
  }

  // ---- set-up: barriers, tensor memory, zeroed operand tiles ----
  // Each producer warp prepares its own ring barriers and starts fetching before the CTA-wide
  // set-up barrier, so the first page tiles are in flight while tensor memory is allocated.
  // (the wide form's second producers, warps 18 / 19, take the odd walk steps; they join in after
  // the set-up barrier)
  const bool is_k_producer = warp == kKProducerWarp || (kSecond && warp == 18);
  const bool is_v_producer = warp == kVProducerWarp || (kSecond && warp == 19);
  const bool is_producer = is_k_producer || is_v_producer;
  const bool second_producer = kSecond && warp >= 18;
  int spec[4] = {-1, -1, -1, -1};
  if (is_producer && !second_producer) {
    if (lane == 0) {
      if (is_k_producer) {
        for (int s = 0; s < kKS; ++s) { mbar_init(&sm.k_full[s], 1); mbar_init(&sm.k_empty[s], 1); }
        sm.abort_flag = 0;
      } else {
        for (int s = 0; s < kVS; ++s) { mbar_init(&sm.v_full[s], 1); mbar_init(&sm.v_empty[s], 1); }
        sm.abort_flag = 0;   // both producers clear it: either may be the first to wait
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    // a producer only signals the set-up barrier (it needs nothing the others prepare)
    asm volatile("bar.arrive 4, %0;" ::"n"(kThreads) : "memory");
    // Page-table columns are fetched before the row's length is known (the loads run beside
    // the length's).  Reading a column is harmless even when it lies past the used prefix;
    // its value is only used, and range-checked, if the length says the column is live.
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = lane + 32 * j;
      if (col < p.max_pages) spec[j] = __ldg(p.page_table + (int64_t)row_of_block * p.page_table_row_stride + col);
    }
  }
  if (tid == 0) {
    for (int wq = 0; wq < 4; ++wq) sm.m_seq[wq] = 0;
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.s_full[b], 1); mbar_init(&sm.s_free[b], 128);
      mbar_init(&sm.p_full[b], 128);
      mbar_init(&sm.o_full[b], 1); mbar_init(&sm.o_free[b], 128);
    }
    mbar_init(&sm.q_ready, 128);
    for (int b = 0; b < 4; ++b) mbar_init(&sm.drain[b], 1);
    mbar_init(&sm.tail_full, 1);
    mbar_init(&sm.tail_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kQkWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&sm.tmem_base)),
                 "r"(C::kAlloc)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // rows G..7 of the N = 8 operands and their scale rows stay zero for the whole kernel
  if (!is_producer) {
    constexpr int kWorkers = kThreads - 64 * kIssuers;   // all but the producer warps
    // warps 0-7, 9, 10 -> 0..319, the second score group's warps 12-15 -> 320..447
    const int wt = tid < kKProducerWarp * 32 ? tid : tid < kVProducerWarp * 32 ? tid - 32 : tid - 64;
    for (int i = wt; i < NQ * 64 / 16; i += kWorkers) reinterpret_cast<uint4*>(sm.q_tile)[i] = make_uint4(0, 0, 0, 0);
    for (int i = wt; i < 2 * kBatch * NQ * 64 / 16; i += kWorkers)
      reinterpret_cast<uint4*>(sm.p_tile)[i] = make_uint4(0, 0, 0, 0);
    for (int i = wt; i < 2 * kBatch * kSfBlockBytes / 16; i += kWorkers)
      reinterpret_cast<uint4*>(sm.p_sf)[i] = make_uint4(0, 0, 0, 0);
    if (!p.q_fp4)
      for (int i = wt; i < kSfBlockBytes / 16; i += kWorkers) reinterpret_cast<uint4*>(sm.q_sf)[i] = make_uint4(0, 0, 0, 0);
  }
  const TileWork w = resolve();
  const int n_pages = w.last_page - w.first_page;
  const int n_batches = (n_pages + kBatch - 1) / kBatch;

  // one slot of a ring: the K (or V) tile of a page and its scale block, or a masked stand-in
  auto issue_slot = [&](bool is_k, int s, int step, int64_t pid) {
    uint8_t* st = is_k ? sm.k_slot[s] : sm.v_slot[s];
    uint64_t* bar = is_k ? &sm.k_full[s] : &sm.v_full[s];
    if (is_k) sm.page_ok[step & 31] = pid >= 0 ? 1 : 0;   // by walk step: a K slot is reused before its scores are read
    if (pid >= 0) {
      mbar_expect_tx(bar, kSlotBytes);
      if (is_k) {
        tma_load_4d(smem_u32(st), &maps.k, bar, 0, w.kvh, 0, (int)pid);
        bulk_load(smem_u32(st + kTileBytes), p.k_sf + pid * p.k_sf_pitch + (int64_t)w.kvh * kSfBlockBytes,
                  kSfBlockBytes, bar);
      } else {
        tma_load_4d(smem_u32(st), &maps.v, bar, 0, 0, w.kvh, (int)pid);
        bulk_load(smem_u32(st + kTileBytes), p.v_sf + pid * p.v_sf_pitch + (int64_t)w.kvh * kSfBlockBytes,
                  kSfBlockBytes, bar);
      }
    } else {
      // a page id outside the cache is never turned into an address: the slot gets zero
      // scales (so its product is zero) and the score threads mask its scores
      for (int j = 0; j < kSfBlockBytes / 16; ++j)
        reinterpret_cast<uint4*>(st + kTileBytes)[j] = make_uint4(0, 0, 0, 0);
      fence_proxy_async();
      mbar_arrive(bar);
    }
  };
  static_assert(kVS > kTailSlots, "the V producer keeps at least one slot while the tail is staged");
  const bool has_tail = w.tail_len > 0;
  // Tail staging geometry: boxes of kTailBoxRows tokens; a half (64 channels) of the staged keys
  // is tail_half bytes long.  Up to two boxes (64 tokens) keys AND values fit side by side and
  // are fetched together; a longer tail's values follow its keys into the same place.
  const int tail_copied = p.append_key != nullptr ? w.tail_len - 1 : w.tail_len;   // the step's own token is not in the cache yet
  const int tail_boxes = (tail_copied + kTailBoxRows - 1) / kTailBoxRows;
  const int tail_half = tail_boxes * kTailBoxRows * 128;
  const bool tail_together = tail_boxes <= 2;
  // slots a producer may fill at once at the start: all of its ring, except that the V ring's
  // last slots hold the tail until tail_done - as many as this tail needs, at most kTailSlots
  const int tail_bytes = (tail_together ? 4 : 2) * tail_half;
  const int tail_slots = (tail_bytes + kSlotBytes - 1) / kSlotBytes;
  uint8_t* const tail_rows = sm.v_slot[kVS - kTailSlots] + (kTailSlots * kSlotBytes - tail_slots * kSlotBytes);
  const int open_slots = is_k_producer ? kKS : (has_tail ? kVS - tail_slots : kVS);
  // ids: lane l of a producer warp holds the page id of walk step 32c + l of the current chunk c
  int ids = -1, issued = 0;
  if (second_producer) issued = n_pages < open_slots ? n_pages : open_slots;
  if (is_producer && !second_producer) {
    const int slots = is_k_producer ? kKS : kVS;
    // chunk 0 out of the columns fetched ahead; every lane executes the same four shuffles
    const int idx0 = w.last_page - 1 - lane;  // pages are walked from the last to the first
    const bool live = idx0 >= w.first_page;
    const int src = live ? (idx0 & 31) : 0;
    int v = -1;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int got = __shfl_sync(0xffffffffu, spec[j], src);
      if (live && (idx0 >> 5) == j) v = got;
    }
    if (live && idx0 >= 128) v = p.page_table[(int64_t)w.row * p.page_table_row_stride + idx0];
    ids = v;
    const int first = n_pages < open_slots ? n_pages : open_slots;
    for (int i = 0; i < first; ++i) {
      int64_t pid = __shfl_sync(0xffffffffu, ids, i);
      if (pid < 0 || pid >= p.num_pages) {
        if (lane == 0 && is_k_producer) set_status(p.status, NVFP4_STATUS_BAD_PAGE_ID);
        pid = -1;
      }
      if (lane == 0) issue_slot(is_k_producer, i, i, pid);
    }
    issued = first;
  }
  uint32_t tmem = 0;
  if (!is_producer || second_producer) {
    tc_fence_before();
    asm volatile("bar.sync 4, %0;" ::"n"(kThreads) : "memory");
    tc_fence_after();
    tmem = sm.tmem_base;
  }

  if (warp < 4 || (warp >= 12 && warp < 16)) {
    // =====================  score threads  =====================
    // Pages are handed over in pairs.  While a pair's scores are processed, warp w owns query
    // heads q = w, w + 4 (< G) over ALL 128 kv positions of each page, four consecutive
    // positions per lane: the page maximum is a warp reduction, a 16-position scale group is
    // four adjacent lanes and the packed E2M1 bytes of P are formed without any exchange.
    // In the wide form a second group of four warps (warps 12-15) takes every other hand-over:
    // group g works on set g of the score, P and output buffers.
    const int grp = warp < 4 ? 0 : 1;
    const int stid = tid & 127, swarp = stid >> 5;   // thread and warp within the group
    const int bar_id = grp == 0 ? 1 : 7;             // the group's own named barrier
    const uint32_t lane_off = (uint32_t)(swarp * 32) << 16;
    // Under a programmatic launch everything up to here, and the producers' and issuers' work,
    // may run while the previous kernel drains.  The query and the tail may be that kernel's
    // output: wait for it, and only then let this launch's own dependents go.
    if (p.pdl) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      if (tid == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    constexpr int QPW = (G + 3) / 4;
    float m_w[QPW], l_w[QPW];
#pragma unroll
    for (int k = 0; k < QPW; ++k) { m_w[k] = -INFINITY; l_w[k] = 0.f; }
    if (grp == 0) {
    // query operand: G packed rows, swizzled; its scale block; the BF16 copy for the tail
    if (p.q_fp4) {
      if (tid < G * 4) {
        const int q = tid >> 2, c = tid & 3;
        const uint4 v = *reinterpret_cast<const uint4*>(
            p.q_fp4 + ((int64_t)w.row * p.heads_q + w.kvh * G + q) * 64 + c * 16);
        *reinterpret_cast<uint4*>(sm.q_tile + sw64_offset(q, c * 16)) = v;
      }
      if (tid < 64) {   // after the rows above (a thread may have both jobs when G = 16)
        reinterpret_cast<uint4*>(sm.q_sf)[tid] = *(reinterpret_cast<const uint4*>(
            p.q_sf + (int64_t)w.row * p.heads_q * kSfBlockBytes + (int64_t)w.kvh * kSfBlockBytes) + tid);
      }
    } else for (int it = tid; it < G * 8; it += 128) {
      // no quantised query was supplied: quantise the BF16 rows of this KV head here, one
      // 16-channel group per thread and pass, with the arithmetic of the stand-alone query
      // quantiser (the scale block was zeroed during set-up)
      const int q = it >> 3, g = it & 7;
      const uint16_t* src = p.q_bf16 + (int64_t)w.row * p.q_row_stride +
                            (int64_t)(w.kvh * G + q) * p.q_head_stride + g * 16;
      float x[16];
      unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(src)), x);
      unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(src) + 1), x + 8);
      uint32_t lo, hi;
      uint8_t sf;
      quantize_group16(x, lo, hi, sf);
      *reinterpret_cast<uint2*>(sm.q_tile + sw64_offset(q, g * 8)) = make_uint2(lo, hi);
      sm.q_sf[sf_offset(q, g)] = sf;
      if (has_tail) {   // the same BF16 values meet the tail: kept as floats, no second fetch
#pragma unroll
        for (int i = 0; i < 16; ++i) sm.qb[q * kHeadDim + g * 16 + i] = x[i];
      }
    }
    fence_proxy_async();
    mbar_arrive(&sm.q_ready);

    if (w.tail_len > 0) {
      if (p.q_fp4) for (int it = tid; it < G * 16; it += 128) {
        const int q = it >> 4, c = it & 15;
        float f[8];
        if (p.q_bf16) {
          unpack_bf16x8(*reinterpret_cast<const uint4*>(p.q_bf16 + (int64_t)w.row * p.q_row_stride +
                                                        (int64_t)(w.kvh * G + q) * p.q_head_stride + c * 8), f);
        } else {
          // no BF16 query supplied: the tail meets the dequantised NVFP4 query
          const uint32_t pk = *reinterpret_cast<const uint32_t*>(
              p.q_fp4 + ((int64_t)w.row * p.heads_q + w.kvh * G + q) * 64 + c * 4);
          const float sc = e4m3_to_f32(p.q_sf[(int64_t)w.row * p.heads_q * kSfBlockBytes +
                                              (int64_t)w.kvh * kSfBlockBytes + sf_offset(q, c >> 1)]);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = e2m1_to_f32((pk >> (4 * i)) & 15u) * sc;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) sm.qb[q * kHeadDim + c * 8 + i] = f[i];
      }
      float m[G], l[G];
      asm volatile("bar.sync 1, 128;" ::: "memory");  // qb visible
      // the key rows were staged by the first output warp; a wait that expires leaves the
      // status word set and the launch aborting, whatever is computed here
      mbar_wait(&sm.tail_full, 0, sm, p.status);
      tail_scores<G, true>(p, w, sm.qb, sm.pf, sm.red_io, tid, 1, m, l, tail_rows, tail_half);
      asm volatile("bar.sync 2, 256;" ::: "memory");  // P of the tail visible to the output threads
      block_sum_128<G>(l, sm.red_io, tid, 1);
#pragma unroll
      for (int k = 0; k < QPW; ++k) {
        const int q = warp + 4 * k;
#pragma unroll
        for (int qq = 0; qq < G; ++qq)
          if (qq == q) { m_w[k] = m[qq]; l_w[k] = lane == 0 ? l[qq] : 0.f; }
      }
    }
    }   // group 0: query and tail

    // A thread whose wait expired keeps walking the loop's barrier points with ok = false, so
    // the 128 threads of a group always leave the loop together.
    bool alive = true;
    for (int kb = grp; kb < n_batches; kb += kGroups) {
      const int set = kb & 1, i0 = kb * kBatch;
      const bool two = kBatch == 2 && i0 + 1 < n_pages;
      const bool ok = alive && mbar_wait(&sm.s_full[set], (kb >> 1) & 1, sm, p.status);
      if (ok) {
        tc_fence_after();
        uint32_t r[C::kSet];
#pragma unroll
        for (int c = 0; c < C::kSet; c += 16)
          tmem_ld16(tmem + lane_off + C::kS + set * C::kSet + c, *reinterpret_cast<uint32_t(*)[16]>(&r[c]));
        tc_fence_before();
        mbar_arrive(&sm.s_free[set]);
        const bool ok0 = sm.page_ok[i0 & 31] != 0;
        const bool ok1 = two && sm.page_ok[(i0 + 1) & 31] != 0;
#pragma unroll
        for (int q = 0; q < G; ++q) {
          sm.z[set][0][q * kPage + stid] = ok0 ? __uint_as_float(r[q]) * p.scale_log2 : -INFINITY;
          if constexpr (kBatch == 2)
            sm.z[set][1][q * kPage + stid] = ok1 ? __uint_as_float(r[NQ + q]) * p.scale_log2 : -INFINITY;
        }
      }
      if (!bar_and<128>(bar_id, ok)) { alive = false; break; }
      // P.V of the pair two hand-overs back has retired: its P tiles, their scale rows and the
      // rescale slots of the pair four hand-overs back may be overwritten
      if (kb >= 2 && !mbar_wait(&sm.o_full[set], ((kb - 2) >> 1) & 1, sm, p.status)) alive = false;
      // the page maxima first: in the wide form the other group is waiting for them
      // (with many heads per warp the scores are read from shared memory again further down
      // rather than kept in registers)
      constexpr bool kKeepZ = QPW <= 2;
      float4 za[kKeepZ ? QPW : 1], zb[kKeepZ ? QPW : 1];
      PageMax ma[QPW], mb[QPW];
#pragma unroll
      for (int k = 0; k < QPW; ++k) {
        const int q = swarp + 4 * k;
        if (q < G) {
          const float4 a = *reinterpret_cast<const float4*>(&sm.z[set][0][q * kPage + 4 * lane]);
          ma[k] = page_max(a);
          if constexpr (kKeepZ) za[k] = a;
          if constexpr (kBatch == 2) {
            const float4 b = *reinterpret_cast<const float4*>(&sm.z[set][1][q * kPage + 4 * lane]);
            mb[k] = page_max(b);
            if constexpr (kKeepZ) zb[k] = b;
          }
        }
      }
      float m_before[QPW];   // running maximum of everything walked before this pair
#pragma unroll
      for (int k = 0; k < QPW; ++k) m_before[k] = m_w[k];
      if constexpr (kGroups == 2) {
        if (kb > 0) {
          // the other group publishes the maximum after pair kb - 1 for this warp's heads
          if (lane == 0) {
            const unsigned long long t0 = global_ns();
            uint32_t spins = 0;
            while (sm.m_seq[swarp] < kb) {
              if (sm.abort_flag) break;
              if ((++spins & 1023u) == 0 && global_ns() - t0 > kWaitLimitNs) {
                sm.abort_flag = 1;
                set_status(p.status, NVFP4_STATUS_WAIT_TIMEOUT);
                break;
              }
            }
          }
          __syncwarp();
#pragma unroll
          for (int k = 0; k < QPW; ++k) {
            const int q = swarp + 4 * k;
            if (q < G) m_before[k] = sm.m_val[kb & 1][q];
          }
        }
      }
      float m1[QPW], m2[QPW];
#pragma unroll
      for (int k = 0; k < QPW; ++k) {
        const int q = swarp + 4 * k;
        if (q < G) {
          // the pages are walked in order: the first page of a pair is quantised against the
          // maximum up to and including itself, the second against the maximum including both
          m1[k] = fmaxf(m_before[k], ma[k].page);
          m2[k] = m1[k];
          if constexpr (kBatch == 2) m2[k] = fmaxf(m1[k], mb[k].page);
          if constexpr (kGroups == 2)
            if (lane == 0) sm.m_val[(kb + 1) & 1][q] = m2[k];
        }
      }
      if constexpr (kGroups == 2) {
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          sm.m_seq[swarp] = kb + 1;   // the other group may go on
        }
      }
#pragma unroll
      for (int k = 0; k < QPW; ++k) {
        const int q = swarp + 4 * k;
        if (q < G) {
          // this group's part of the row sum refers to its own last maximum: bring it to the
          // maximum before this pair (the other group's pair may have raised it)
          if constexpr (kGroups == 2)
            if (m_w[k] != -INFINITY && m_before[k] != m_w[k]) l_w[k] *= exp2f(m_w[k] - m_before[k]);
          const float ra = (m_before[k] == -INFINITY) ? 0.f : exp2f(m_before[k] - m1[k]);
          float4 a;
          if constexpr (kKeepZ) a = za[k];
          else a = *reinterpret_cast<const float4*>(&sm.z[set][0][q * kPage + 4 * lane]);
          const float sa = quantize_page(a, ma[k].group, m1[k], sm.p_tile[set][0], sm.p_sf[set][0], q, lane);
          if constexpr (kBatch == 2) {
            const float rb = (m1[k] == -INFINITY) ? 0.f : exp2f(m1[k] - m2[k]);
            float4 b;
            if constexpr (kKeepZ) b = zb[k];
            else b = *reinterpret_cast<const float4*>(&sm.z[set][1][q * kPage + 4 * lane]);
            const float sb = quantize_page(b, mb[k].group, m2[k], sm.p_tile[set][1], sm.p_sf[set][1], q, lane);
            l_w[k] = fmaf(fmaf(l_w[k], ra, sa), rb, sb);
            if (lane == 0) {
              sm.resc[i0 & 7][q] = ra;
              sm.resc[(i0 + 1) & 7][q] = rb;
            }
          } else {
            l_w[k] = fmaf(l_w[k], ra, sa);
            if (lane == 0) sm.resc[i0 & 7][q] = ra;
          }
          m_w[k] = m2[k];
        }
      }
      fence_proxy_async();
      mbar_arrive(&sm.p_full[set]);
    }
    // the group's part of the row sums and the maxima they refer to, for the output threads
#pragma unroll
    for (int k = 0; k < QPW; ++k) {
      const int q = swarp + 4 * k;
      if (q < G) {
        const float ls = warp_sum(l_w[k]);
        if (lane == 0) { sm.fin[grp][q] = ls; sm.fin[grp][NQ + q] = m_w[k]; }
      }
    }
    bar_and<128 * (kGroups + 1)>(3, alive);
  } else if (warp < 8) {
    // =====================  output threads: thread t = channel t  =====================
    const int t = tid - 128;
    const uint32_t lane_off = (uint32_t)((warp - 4) * 32) << 16;
    // the epoch of this launch's exchange: read now, long before the last tile of the launch
    // advances it (no CTA of the next launch can run before that)
    const int xchg_epoch = p.xchg_inbox ? *reinterpret_cast<volatile int*>(p.xchg_epoch_state) + 1 : 0;
    if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");   // before the tail is read or anything is stored
    float o[G];
#pragma unroll
    for (int q = 0; q < G; ++q) o[q] = 0.f;
    if (w.tail_len > 0) {
      // The tail's rows come into shared memory by tensor copies (boxes of kTailBoxRows tokens x
      // half a row, 128-byte swizzle; a copy per row was tried first: the copy engine takes
      // some 35 ns per instruction, 9 us for a full tail), issued by this group's first warp:
      // the key rows at once; the value rows into the same place as soon as the score threads
      // are done with the keys (the barrier below).  The step's own token is not in the cache
      // yet: it is taken from the source by the threads that handle its position.
      uint8_t* const value_rows = tail_together ? tail_rows + 2 * tail_half : tail_rows;
      auto stage = [&](const CUtensorMap* map, uint8_t* dst) {
        if (lane < 2 * tail_boxes) {
          const int half = lane & 1, b = lane >> 1;
          tma_load_3d(smem_u32(dst + half * tail_half + b * kTailBoxRows * 128), map, &sm.tail_full,
                      half * 128, w.kvh, w.tail_id * kPage + b * kTailBoxRows);
        }
      };
      auto expect = [&](int parts) {   // parts: 1 = keys or values, 2 = both
        if (lane == 0) {
          if (tail_boxes > 0) mbar_expect_tx(&sm.tail_full, (uint32_t)(parts * 2 * tail_half));
          else mbar_arrive(&sm.tail_full);
        }
        __syncwarp();
      };
      if (warp == 4) {
        expect(tail_together ? 2 : 1);
        stage(&maps.tail_k, tail_rows);
        if (tail_together) stage(&maps.tail_v, value_rows);
      }
      asm volatile("bar.sync 2, 256;" ::: "memory");   // P of the tail is there; the keys are no longer read
      if (!tail_together) {
        if (warp == 4) {
          fence_proxy_async();
          expect(1);
          stage(&maps.tail_v, value_rows);
        }
        mbar_wait(&sm.tail_full, 1, sm, p.status);
      } else {
        mbar_wait(&sm.tail_full, 0, sm, p.status);
      }
      tail_pv_staged<G>(p, w, sm.pf, value_rows, tail_half, t, o);
      asm volatile("bar.sync 6, 128;" ::: "memory");   // every output thread is done with the rows
      if (t == 0) mbar_arrive(&sm.tail_done);           // the V producer may have the slots
    }
    bool alive = true;
    for (int kb = 0; kb < n_batches && alive; ++kb) {
      // fold the pair: o = o * rescale(j) + O_page(j), page by page
      const int set = kb & 1, j0 = kb * kBatch;
      const bool two = kBatch == 2 && j0 + 1 < n_pages;
      if (mbar_wait(&sm.o_full[set], (kb >> 1) & 1, sm, p.status)) {
        tc_fence_after();
        uint32_t ro[C::kSet];
#pragma unroll
        for (int c = 0; c < C::kSet; c += 16)
          tmem_ld16(tmem + lane_off + C::kO + set * C::kSet + c, *reinterpret_cast<uint32_t(*)[16]>(&ro[c]));
        tc_fence_before();
        mbar_arrive(&sm.o_free[set]);
#pragma unroll
        for (int q = 0; q < G; ++q) {
          o[q] = fmaf(o[q], sm.resc[j0 & 7][q], __uint_as_float(ro[q]));
          if constexpr (kBatch == 2)
            if (two) o[q] = fmaf(o[q], sm.resc[(j0 + 1) & 7][q], __uint_as_float(ro[NQ + q]));
        }
      } else {
        alive = false;
      }
    }
    const bool stored = bar_and<128 * (kGroups + 1)>(3, alive);
    if (stored) {
#pragma unroll
      for (int q = 0; q < G; ++q) {
        float lq = sm.fin[0][q], mq = sm.fin[0][NQ + q];
        if constexpr (kGroups == 2) {
          // join the two groups' parts of the row sum at the larger (the final) maximum
          const float l1 = sm.fin[1][q], mq1 = sm.fin[1][NQ + q];
          const float mf = fmaxf(mq, mq1);
          const float a0 = mq == -INFINITY ? 0.f : lq * exp2f(mq - mf);
          const float a1 = mq1 == -INFINITY ? 0.f : l1 * exp2f(mq1 - mf);
          lq = a0 + a1;
          mq = mf;
        }
        const int head = w.kvh * G + q;
        const float val = lq > 0.f ? __fdiv_rn(o[q], lq) : 0.f;
        if (p.emit_partial) {
          const int64_t idx = w.slot * p.heads_q + head;
          p.o_partial[idx * kHeadDim + t] = val;
          if (t == 0) p.lse_partial[idx] = lq > 0.f ? (mq + log2f(lq)) * kLn2 : -INFINITY;
        } else {
          const int64_t orow = p.out_indices ? (int64_t)p.out_indices[w.row] : (int64_t)w.row;
          p.out[(orow * p.heads_q + head) * kHeadDim + t] = __bfloat16_as_ushort(__float2bfloat16_rn(val));
        }
      }
    }
    // The exchange serves up to eight query heads per KV head (its fold keeps five values per
    // head and thread in registers; at sixteen and more heads that code spilled, and the spill
    // slots were the only stack these instantiations had).  The host refuses the combination.
    if constexpr (G <= 8) {
      if (p.xchg_inbox) exchange_tile<G>(p, w, sm, t, stored, xchg_epoch);
      else if (p.work_list && p.list_counters) finish_piece<G>(p, w.row, w.kvh, t, sm.xchg_last);
    } else {
      if (p.work_list && p.list_counters) finish_piece<G>(p, w.row, w.kvh, t, sm.xchg_last);
    }
  } else if (is_producer) {
    // =====================  producers (K ring: warp 8, V ring: warp 11)  =====================
    if constexpr (kGroups == 1) {
      // Narrow form (two CTAs per SM, the page stream bound by HBM): lane 0 walks the table
      // itself, reading its entries one step ahead of their use.
      if (lane == 0) {
        const int slots = is_k_producer ? kKS : kVS;
        const int32_t* table = p.page_table + (int64_t)w.row * p.page_table_row_stride;
        int i = issued;
        int64_t next = i < n_pages ? table[w.last_page - 1 - i] : -1;
        for (; i < n_pages; ++i) {
          int64_t pid = next;
          if (i + 1 < n_pages) next = table[w.last_page - 1 - (i + 1)];
          if (pid < 0 || pid >= p.num_pages) {
            if (is_k_producer) set_status(p.status, NVFP4_STATUS_BAD_PAGE_ID);
            pid = -1;
          }
          const int s = i % slots;
          if (has_tail && !is_k_producer && i < slots && s >= open_slots) {
            // first use of a slot that held the tail: wait until the tail is consumed
            if (!mbar_wait(&sm.tail_done, 0, sm, p.status)) break;
            fence_proxy_async();
          }
          uint64_t* freed = is_k_producer ? &sm.k_empty[s] : &sm.v_empty[s];
          if (!mbar_wait(freed, ((i / slots) & 1) ^ 1, sm, p.status)) break;
          issue_slot(is_k_producer, s, i, pid);
        }
      }
    } else {
    // Wide form (a CTA with an SM to itself, bound by its own page period): the page ids of a
    // walk are read 32 at a time, one per lane and one chunk ahead of their use - a load per
    // page in the issuing thread's own loop costs it a memory round trip per page, and the ring
    // then fills at two pages a microsecond whatever its depth - and two producers of each kind
    // take the walk steps alternately; lane 0 of each takes its ids by shuffle and issues.
    {
      const int slots = is_k_producer ? kKS : kVS;
      const int32_t* table = p.page_table + (int64_t)w.row * p.page_table_row_stride;
      auto chunk_ids = [&](int base) {   // lane l: the page id of walk step base + l, or -1 past the end
        const int idx = w.last_page - 1 - (base + lane);
        return idx >= w.first_page ? __ldg(table + idx) : -1;
      };
      int alive = 1;
      if (second_producer) ids = chunk_ids(0);
      int ids_next = n_pages > 32 ? chunk_ids(32) : -1;
      const int parity = second_producer ? 1 : 0;
      for (int base = 0; base < n_pages && alive; base += 32) {
        if (base > 0) {
          ids = ids_next;
          if (base + 32 < n_pages) ids_next = chunk_ids(base + 32);
        }
        const int in_chunk = min(32, n_pages - base);
        for (int j = (base == 0 ? issued : 0); j < in_chunk; ++j) {
          if (kSecond && (j & 1) != parity) continue;   // the other producer of the kind takes it
          int64_t pid = __shfl_sync(0xffffffffu, ids, j);
          if (lane == 0) {
            if (pid < 0 || pid >= p.num_pages) {
              if (is_k_producer) set_status(p.status, NVFP4_STATUS_BAD_PAGE_ID);
              pid = -1;
            }
            const int i = base + j, s = i % slots;
            if (has_tail && !is_k_producer && i < slots && s >= open_slots) {
              if (!mbar_wait(&sm.tail_done, 0, sm, p.status)) alive = 0;
              fence_proxy_async();
            }
            uint64_t* freed = is_k_producer ? &sm.k_empty[s] : &sm.v_empty[s];
            if (!alive || !mbar_wait(freed, ((i / slots) & 1) ^ 1, sm, p.status)) alive = 0;
            else issue_slot(is_k_producer, s, i, pid);
          }
          alive = __shfl_sync(0xffffffffu, alive, 0);
          if (!alive) break;
        }
      }
    }
    }
    __syncwarp();
  } else if (warp == kQkWarp || (kSecond && warp == 16)) {
    // =====================  MMA issuer 1: S^T = K . Q^T  =====================
    // Issuing a tcgen05 instruction costs the issuing thread some 60 cycles and a barrier
    // wait about twice that, so the two products of a page are issued by two threads - and in
    // the wide form, where a CTA has an SM to itself and the issue rate is what bounds its page
    // period, by two threads each: issuer ig takes the hand-overs kb = ig, ig + 2, ... (set ig of
    // the buffers) with scale columns of its own.
    const int ig = warp == kQkWarp ? 0 : 1;
    if (lane == 0 && n_pages > 0) {
      bool alive = mbar_wait(&sm.q_ready, 0, sm, p.status);
      const uint32_t sfq = tmem + C::kSfQ + 8 * ig, sfk = tmem + C::kSfK + 8 * ig;
      if (alive) {
        tc_fence_after();
        cp_sf(sfq, smem_u32(sm.q_sf));
        cp_sf(sfq + 4, smem_u32(sm.q_sf + 512));
      }
      const uint64_t q_desc = desc_sw64(smem_u32(sm.q_tile));
      for (int kb = ig; kb < n_batches && alive; kb += kIssuers) {
        const int set = kb & 1;
        alive = mbar_wait(&sm.s_free[set], ((kb >> 1) & 1) ^ 1, sm, p.status);
        for (int u = 0; u < kBatch && alive; ++u) {
          const int i = kb * kBatch + u;
          if (i >= n_pages) break;
          const int s = i % kKS;
          alive = mbar_wait(&sm.k_full[s], (i / kKS) & 1, sm, p.status);
          if (!alive) break;
          tc_fence_after();
          const uint32_t st = smem_u32(sm.k_slot[s]);
          cp_sf(sfk, st + kTileBytes);
          cp_sf(sfk + 4, st + kTileBytes + 512);
          const uint64_t k_desc = desc_sw64(st);
          const uint32_t d = tmem + C::kS + set * C::kSet + u * NQ;
          mma_nvf4<NQ>(d, k_desc, q_desc, sfk, sfq, 0);
          mma_nvf4<NQ>(d, k_desc + 2, q_desc + 2, sfk + 4, sfq + 4, 1);
          mma_commit(&sm.k_empty[s]);   // the K slot goes back once this page's product has retired
        }
        if (alive) mma_commit(&sm.s_full[set]);
      }
      // everything this thread issued must have retired before tensor memory is freed
      mma_commit(&sm.drain[ig]);
      mbar_wait(&sm.drain[ig], 0, sm, p.status);
    }
    __syncwarp();
  } else if (warp == kPvWarp || (kSecond && warp == 17)) {
    // =====================  MMA issuer 2: O^T = V^T . P^T  =====================
    const int ig = warp == kPvWarp ? 0 : 1;
    if (lane == 0 && n_pages > 0) {
      bool alive = true;
      const uint32_t sfp = tmem + C::kSfP + 8 * ig;
      for (int kb = ig; kb < n_batches && alive; kb += kIssuers) {
        const int set = kb & 1;
        // The V slots of a pair land long before its probabilities are ready: their scale
        // blocks go to tensor memory now (columns of their own per page of the pair), which
        // keeps four copies off the path between P being ready and O^T being done.
        for (int u = 0; u < kBatch && alive; ++u) {
          const int j = kb * kBatch + u;
          if (j >= n_pages) break;
          const int s = j % kVS;
          alive = mbar_wait(&sm.v_full[s], (j / kVS) & 1, sm, p.status);
          if (!alive) break;
          tc_fence_after();
          const uint32_t st = smem_u32(sm.v_slot[s]);
          const uint32_t c = tmem + C::kSfV + (set * kBatch + u) * 8;
          cp_sf(c, st + kTileBytes);
          cp_sf(c + 4, st + kTileBytes + 512);
        }
        alive = alive && mbar_wait(&sm.p_full[set], (kb >> 1) & 1, sm, p.status) &&
                mbar_wait(&sm.o_free[set], ((kb >> 1) & 1) ^ 1, sm, p.status);
        if (!alive) break;
        tc_fence_after();
        for (int u = 0; u < kBatch; ++u) {
          const int j = kb * kBatch + u;
          if (j >= n_pages) break;
          const int s = j % kVS;
          const uint32_t c = tmem + C::kSfV + (set * kBatch + u) * 8;
          cp_sf(sfp, smem_u32(sm.p_sf[set][u]));
          cp_sf(sfp + 4, smem_u32(sm.p_sf[set][u] + 512));
          const uint64_t v_desc = desc_sw64(smem_u32(sm.v_slot[s]));
          const uint64_t p_desc = desc_sw64(smem_u32(sm.p_tile[set][u]));
          const uint32_t d = tmem + C::kO + set * C::kSet + u * NQ;
          mma_nvf4<NQ>(d, v_desc, p_desc, c, sfp, 0);
          mma_nvf4<NQ>(d, v_desc + 2, p_desc + 2, c + 4, sfp + 4, 1);
          mma_commit(&sm.v_empty[s]);   // the V slot goes back once this page's product has retired
        }
        mma_commit(&sm.o_full[set]);
      }
      mma_commit(&sm.drain[2 + ig]);
      mbar_wait(&sm.drain[2 + ig], 0, sm, p.status);
    }
    __syncwarp();
  }

  // ---- teardown ----
  tc_fence_before();
  __syncthreads();
  if (is_producer && !second_producer && lane == 0 && sm.abort_flag) {
    // copies still in flight must land before the CTA's shared memory is handed on
    const int slots = is_k_producer ? kKS : kVS;
    for (int s = 0; s < slots; ++s) {
      uint64_t* bar = is_k_producer ? &sm.k_full[s] : &sm.v_full[s];
      const unsigned long long t0 = global_ns();
      while (!mbar_try(bar, 0) && !mbar_try(bar, 1) && global_ns() - t0 < 200000000ull) {}
    }
  }
  __syncthreads();
  if (warp == kQkWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::kAlloc)
                 : "memory");
  }
}


template <int G, int kGroups>
static cudaError_t launch_g(const DecodeParams& p, const TileMaps& maps,
                            cudaStream_t stream) {
  const size_t smem = sizeof(Smem<G, kGroups>) + 1024;
  static_assert(sizeof(Smem<G, kGroups>) + 1024 <= (kGroups == 1 ? 115712 : 232448),
                "shared memory of one CTA (two per SM in the narrow form)");
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    e = cudaFuncSetAttribute(decode_sm100_kernel<G, kGroups>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(decode_sm100_kernel<G, kGroups>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    // The narrow form is built for two CTAs per SM: 2 x (shared memory of a CTA + 1 KB the
    // system keeps per CTA) must fit the SM's 228 KB.  A static shared variable anywhere in the
    // kernel counts too, and 16 bytes of it once halved the residency (and the page stream)
    // unnoticed: checked once per device, refused loudly.  (The occupancy calculator is no help:
    // it answers 1 for this kernel at any size.)
    if constexpr (kGroups == 1) {
      cudaFuncAttributes fa{};
      e = cudaFuncGetAttributes(&fa, decode_sm100_kernel<G, kGroups>);
      if (e != cudaSuccess) return e;
      if (fa.sharedSizeBytes + smem > 115712) return cudaErrorLaunchOutOfResources;
    }
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  dim3 grid(p.num_splits, p.heads_kv, p.rows);
  // CTAs start in the order of their linear index, x fastest: all KV heads of the first list
  // entry, then of the second, ... - and the list holds the longest pieces first
  if (p.work_list) grid = dim3(p.heads_kv, p.work_capacity, 1);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(ThreadsOf<G, kGroups>::value);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, decode_sm100_kernel<G, kGroups>, maps, p);
}

// The wide form pays when a CTA's own page period, not HBM, bounds the launch: at most one CTA
// per SM.  Sixteen and more query heads per KV head always take it (their score threads need its
// register budget).
template <int G>
static cudaError_t launch_form(const DecodeParams& p, const TileMaps& maps,
                               cudaStream_t stream) {
  static int sms[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  int n = 148;
  if (dev >= 0 && dev < 64) {
    if (!sms[dev] && cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms[dev] = 148;
    n = sms[dev];
  }
  const int64_t ctas = p.work_list ? (int64_t)p.heads_kv * p.work_capacity
                                   : (int64_t)p.num_splits * p.heads_kv * p.rows;
  // 16 and 32 query heads per KV head exist in the wide form only
  if constexpr (G >= 16) {
    return launch_g<G, 2>(p, maps, stream);
  } else {
    const bool wide = ctas <= n || p.wide_hint;
    return wide ? launch_g<G, 2>(p, maps, stream) : launch_g<G, 1>(p, maps, stream);
  }
}

}  // namespace sm100

bool decode_sm100_supports(const DecodeParams& p) {
  if (p.heads_kv < 1 || p.heads_q % p.heads_kv) return false;
  const int g = p.heads_q / p.heads_kv;
  return (g >= 1 && g <= 8) || g == 16 || g == 32;
}

cudaError_t launch_decode_sm100(const DecodeParams& p, cudaStream_t stream) {
  if (p.rows == 0) return cudaSuccess;
  if (!decode_sm100_supports(p)) return cudaErrorNotSupported;
  if (p.num_pages < 1 || p.num_pages > 0x7FFFFFFF) return cudaErrorInvalidValue;
  sm100::TileMaps maps;
  std::memset(&maps, 0, sizeof(maps));
  cudaError_t e = sm100::make_map(0, p.k_packed, p.k_pitch, p.num_pages, p.heads_kv, &maps.k);
  if (e != cudaSuccess) return e;
  e = sm100::make_map(1, p.v_packed, p.v_pitch, p.num_pages, p.heads_kv, &maps.v);
  if (e != cudaSuccess) return e;
  if (p.tail_key != nullptr && p.tail_value != nullptr && p.tail_pages > 0) {
    if (p.tail_pages > (int64_t)0x7FFFFFFF / 128) return cudaErrorInvalidValue;
    e = sm100::make_map(2, p.tail_key, 0, p.tail_pages, p.heads_kv, &maps.tail_k);
    if (e != cudaSuccess) return e;
    e = sm100::make_map(2, p.tail_value, 0, p.tail_pages, p.heads_kv, &maps.tail_v);
    if (e != cudaSuccess) return e;
  }
  switch (p.heads_q / p.heads_kv) {
    case 1: return sm100::launch_form<1>(p, maps, stream);
    case 2: return sm100::launch_form<2>(p, maps, stream);
    case 3: return sm100::launch_form<3>(p, maps, stream);
    case 4: return sm100::launch_form<4>(p, maps, stream);
    case 5: return sm100::launch_form<5>(p, maps, stream);
    case 6: return sm100::launch_form<6>(p, maps, stream);
    case 7: return sm100::launch_form<7>(p, maps, stream);
    case 8: return sm100::launch_form<8>(p, maps, stream);
    case 16: return sm100::launch_form<16>(p, maps, stream);
    case 32: return sm100::launch_form<32>(p, maps, stream);
    default: return cudaErrorNotSupported;
  }
}

}  // namespace nvfp4
