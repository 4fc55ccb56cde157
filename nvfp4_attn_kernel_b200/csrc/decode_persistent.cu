// Persistent tensor-core decode kernel for sm_100a: the whole step is cut into equal shares of
// page tiles, one share per resident CTA (two CTAs per SM), and a CTA pays its set-up - barriers,
// tensor memory, zeroed operand tiles - once, then walks the pieces of its share back to back.
//
// Schedule.  A row costs C = max(1, FP4 pages + tail units) units; the rows are laid end to end
// and the CTAs form groups of heads_kv: group j of Ce owns units [floor(j T / Ce),
// floor((j + 1) T / Ce)) and its CTA h walks KV head h of them, so the heads of a page, which a
// K page interleaves 64 bytes at a time, are read together.  Every CTA derives the same schedule
// from the device-resident lengths (one warp: prefix sums over the rows), so nothing is launched
// ahead of the kernel and a captured graph follows the lengths of every replay.  A row's unit 0
// stands for its BF16 tail (tail units long, indivisible, so it goes with the piece that holds
// unit 0 - the reference gives the tail to split 0, fp4_decode_kernel.py:159), the units after
// it for logical pages 0, 1, ...
//
// A piece that covers its whole row stores the BF16 output row directly.  A row cut over several
// groups is folded by the group that holds its first unit.  Rows lie in order, so every other
// group meets the row as the FIRST piece of its share: it stores a partial (normalised fp32 O and
// natural-log LSE, the split format of the reference, fp4_decode_kernel.py:5186-5196) into the
// CTA's scratch slot, every value together with the launch's tag in one 8-byte word, and waits
// for nothing: no fence, no counter.  The folding group meets the row as the LAST piece of its
// share: by then the others have normally arrived, it fetches their words while its own last
// pages are in flight and folds them with its own values out of registers, in group order and
// with the arithmetic of the LSE merge kernel.  Only for words still missing at its very end does
// it wait (bounded) - for CTAs of higher index only, whose first piece depends on nobody, so the
// wait cannot be circular.
//
// Inside a CTA the roles are those of the one-tile kernel (decode_sm100.cu): warps 0-3 score
// threads, 4-7 output threads, 8 / 11 K and V producers, 9 / 10 the two MMA issuers.  The rings,
// the hand-over counters and the tensor-memory sets run on across piece boundaries, so the
// producers are a ring depth ahead into the next piece while the last pages of the current one
// are still being folded.  What changes at a boundary: the query operand (two shared-memory
// buffers; the next piece's rows are fetched with cp.async while the current piece runs), the
// softmax state, and the output threads' epilogue.
//
// Every device-side wait is bounded; on expiry the CTA raises NVFP4_STATUS_WAIT_TIMEOUT, keeps
// walking its schedule without touching data (a storing piece marks its partial failed and the
// folding piece then leaves the row alone), drains its copies, frees tensor memory and returns.
#include "sm100_device.cuh"

namespace nvfp4 {
namespace sm100p {

using namespace sm100;

constexpr int kThreads = 384;
constexpr int kMaxSeg = 48;        // pieces one CTA may hold; the host refuses shapes that could exceed it
constexpr int kMinShare = 4;       // units: a step this small uses fewer CTAs rather than thinner shares
constexpr int kBatch = 2;          // pages per hand-over
constexpr int NQ = 8;              // MMA N: query slots (G <= 8 live)
constexpr int kKProducerWarp = 8, kQkWarp = 9, kPvWarp = 10, kVProducerWarp = 11;

// Cost of a BF16 tail in units of one NVFP4 page (the tail is walked on CUDA cores).
__host__ __device__ __forceinline__ int tail_units(int len) { return len > 0 ? 4 + (len >> 3) : 0; }

template <int G> struct KSlots { static constexpr int value = G <= 4 ? 4 : 3; };
template <int G> struct VSlots { static constexpr int value = 5; };

// tensor-memory columns (32-bit); a "set" holds the two pages of one hand-over
struct Cols {
  static constexpr int kSet = kBatch * NQ;
  static constexpr int kS = 0;                   // 2 sets : S^T
  static constexpr int kO = 2 * kSet;            // 2 sets : per-page O^T
  static constexpr int kSfQ = 4 * kSet;          // 8
  static constexpr int kSfK = kSfQ + 8;          // 8
  static constexpr int kSfP = kSfK + 8;          // 8 (+ 8 spare)
  static constexpr int kSfV = kSfP + 16;         // 2 sets x 2 pages x 8
  static constexpr int kAlloc = 128;
  static_assert(kSfV + 2 * kBatch * 8 <= kAlloc, "tensor-memory columns");
};

struct Seg {
  int row, kvh;
  int first_page, last_page;   // logical FP4 pages [first, last), walked from the last to the first
  int tail_len, tail_id;       // BF16 tail of this piece (0, -1: none)
  int slot;                    // scratch slot of the partial, or -1: the piece is its whole tile
  int c_first, c_last;         // groups of CTAs that hold the row's first and last unit
  int pad;
};

template <int G>
struct __align__(1024) Smem {
  static constexpr int kKS = KSlots<G>::value, kVS = VSlots<G>::value;
  uint8_t k_slot[kKS][kSlotBytes];              // K tile | K scales
  uint8_t v_slot[kVS][kSlotBytes];              // V tile | V scales
  __align__(1024) uint8_t q_tile[2][NQ * 64];   // NQ rows x 64 B, 64-byte swizzle; [piece parity]
  __align__(1024) uint8_t p_tile[2][kBatch][NQ * 64];
  __align__(512) uint8_t q_sf[2][kSfBlockBytes];
  __align__(512) uint8_t p_sf[2][kBatch][kSfBlockBytes];
  __align__(16) uint16_t q_stage[2][G * kHeadDim];   // BF16 query rows of a piece, as fetched
  __align__(16) float qb[G * kHeadDim];         // BF16 query as floats (tail)
  __align__(16) float pf[G * kHeadDim];         // P of the tail block
  __align__(16) float z[2][kBatch][G * kPage];  // scaled scores, [set][page][q][kv position]
  float resc[8][NQ];                            // ring of per-page rescale factors, [page & 7][q]
  float fin[8][2 * NQ];                         // ring of per-piece row sums and maxima, [piece & 7]
  float red_tail[4 * NQ];                       // reductions inside the tail block
  volatile int page_ok[32];                     // [walk step & 31] 0: the page id was refused
  Seg seg[kMaxSeg];
  int nseg;
  __align__(8) uint64_t k_full[kKS];
  uint64_t k_empty[kKS], v_full[kVS], v_empty[kVS];
  uint64_t s_full[2], s_free[2], p_full[2], o_full[2], o_free[2];
  uint64_t q_full[2], seg_done[8], drain[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ int warp_sum_int(int v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.wait_all;" ::: "memory");
}

// One warp builds the CTA's list of pieces.  Returns through sm.seg / sm.nseg.
template <int G, class SM>
__device__ __forceinline__ void build_schedule(const DecodeParams& p, SM& sm, int lane) {
  const int rows = p.rows, hkv = p.heads_kv;
  const bool has_tail = p.tail_key != nullptr && p.seqused_tail != nullptr;
  const bool report = blockIdx.x == 0;
  // a row's pages, tail length and tail id as every CTA will see them (clamped, never trusted)
  auto row_info = [&](int r, int& n, int& tl, int& tid) {
    const int fp4 = __ldg(p.seqused_fp4 + r);
    n = fp4 >> 7;
    if (fp4 < 0 || (fp4 & 127) || n > p.max_pages) {
      if (report) set_status(p.status, NVFP4_STATUS_BAD_LENGTH);
      n = fp4 < 0 ? 0 : (n > p.max_pages ? p.max_pages : n);
    }
    tl = 0; tid = -1;
    if (has_tail) {
      int len = __ldg(p.seqused_tail + r);
      if (len > 0) {
        if (len > kPage) { if (report) set_status(p.status, NVFP4_STATUS_BAD_LENGTH); len = kPage; }
        const int id = __ldg(p.tail_ids + r);
        if (id < 0 || (int64_t)id >= p.tail_pages) { if (report) set_status(p.status, NVFP4_STATUS_BAD_TAIL_ID); }
        else { tl = len; tid = id; }
      }
    }
  };
  // pass 1: total units of the rows (every KV head of a row costs the same)
  int64_t T = 0;
  for (int r0 = 0; r0 < rows; r0 += 32) {
    int c = 0;
    if (r0 + lane < rows) {
      int n, tl, tid;
      row_info(r0 + lane, n, tl, tid);
      c = max(1, n + tail_units(tl));
    }
    T += warp_sum_int(c);
  }
  // Groups of heads_kv CTAs: group j owns a share of the rows' units and its CTA h walks KV head
  // h of that share, so the heads_kv CTAs of a group read the same pages at about the same time
  // (a K page interleaves its heads 64 bytes at a time: read apart, every 64 bytes would be a
  // DRAM access of their own).
  int64_t ce = (T + kMinShare - 1) / kMinShare;
  const int64_t groups = (int64_t)gridDim.x / hkv;
  ce = ce < groups ? ce : groups;
  const int64_t c = blockIdx.x / hkv;      // this CTA's group
  const int h = blockIdx.x % hkv;          // and its KV head
  int count = 0;
  if (c < ce) {
    const int64_t u0 = c * T / ce, u1 = (c + 1) * T / ce;
    // pass 2: the rows that meet [u0, u1), in unit order
    int64_t before = 0;   // units of the rows before this chunk
    for (int r0 = 0; r0 < rows && before < u1; r0 += 32) {
      const int r = r0 + lane;
      int n = 0, tl = 0, tid = -1, cost = 0;
      if (r < rows) { row_info(r, n, tl, tid); cost = max(1, n + tail_units(tl)); }
      int incl = cost;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += v;
      }
      const int64_t U = before + incl - cost;   // first unit of this row
      const bool mine = r < rows && U < u1 && U + cost > u0;
      const unsigned ballot = __ballot_sync(0xffffffffu, mine);
      const int pos = count + __popc(ballot & ((1u << lane) - 1));
      if (mine) {
        if (pos >= kMaxSeg) {
          set_status(p.status, NVFP4_STATUS_BAD_LENGTH);
        } else {
          const int tw = tail_units(tl);
          const int lo = (int)(max(u0, U) - U), hi = (int)(min(u1, U + cost) - U);
          Seg s;
          s.row = r; s.kvh = h;
          s.first_page = min(max(lo, tw) - tw, n);
          s.last_page = min(max(hi, tw) - tw, n);
          const bool owns_tail = tl > 0 && lo == 0;
          s.tail_len = owns_tail ? tl : 0;
          s.tail_id = owns_tail ? tid : -1;
          s.c_first = (int)(((U + 1) * ce - 1) / T);       // groups that hold the row's first and last unit
          s.c_last = (int)(((U + cost) * ce - 1) / T);
          s.slot = (lo == 0 && hi == cost) ? -1 : (int)blockIdx.x;
          s.pad = 0;
          sm.seg[pos] = s;
        }
      }
      count = min(count + __popc(ballot), kMaxSeg);
      before += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  if (lane == 0) sm.nseg = count;
}

// ---- the scratch slots: values that carry their own arrival flag ----
// A storing piece writes every value of its partial as an 8-byte word {value bits, tag}, the tag
// being this launch's number.  An 8-byte store lands whole, so a reader that finds the tag it
// expects has the value: the writer needs neither a fence nor a counter and never waits, and a
// slot never has to be cleared (the next launch expects the next tag).  A piece that failed
// writes its LSE words with kFailBit set instead.
constexpr uint32_t kFailBit = 0x80000000u;

// slot of the partial that group `group` stores for KV head kvh: one per CTA, a CTA stores at most
// one partial (the row that began in an earlier group)
__device__ __forceinline__ int slot_of(const DecodeParams& p, int kvh, int group) { return group * p.heads_kv + kvh; }

// word `i` of slot `slot`: words [0, G * 128) the normalised O, [G * 128, G * 129) the LSEs
template <int G>
__device__ __forceinline__ uint2* slot_word(const DecodeParams& p, int slot, int i) {
  return reinterpret_cast<uint2*>(p.o_partial) + (int64_t)slot * (G * (kHeadDim + 1)) + i;
}
__device__ __forceinline__ void st_word(uint2* at, float v, uint32_t tag) {
  asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %2};" ::"l"(at), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const uint2* at) {
  uint2 v;
  asm volatile("ld.relaxed.gpu.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(at) : "memory");
  return v;
}
// The value of a word once it carries `tag` (bounded wait).  *bad is set when the writer marked
// the piece failed or the wait ran out.
__device__ __forceinline__ float wait_word(const uint2* at, uint2 have, uint32_t tag, uint32_t* status, bool* bad) {
  if (have.y == tag) return __uint_as_float(have.x);
  const unsigned long long t0 = global_ns();
  for (;;) {
    if (have.y == tag) return __uint_as_float(have.x);
    if (have.y == (tag | kFailBit)) { *bad = true; return 0.f; }
    if (global_ns() - t0 > kWaitLimitNs) {
      set_status(status, NVFP4_STATUS_WAIT_TIMEOUT);
      *bad = true;
      return 0.f;
    }
    __nanosleep(40);
    have = ld_word(at);
  }
}

// Pieces other than the folding one whose values are fetched ahead into registers; a row cut into
// more pieces is folded with loads at the end.
template <int G> struct DirectOthers { static constexpr int value = G <= 4 ? 2 : 1; };

// Values of the other pieces of a row, fetched by an output thread (thread t = channel t) while
// its own piece's last pages are in flight.
template <int G>
struct Others {
  float o[G][DirectOthers<G>::value], lse[G][DirectOthers<G>::value];
};

// Returns true if every word carried the tag (the values are then in `ot`); else the fold loads
// them again at its end, and waits.
template <int G>
__device__ __forceinline__ bool fetch_others(const DecodeParams& p, const Seg& sg, int t, uint32_t tag, Others<G>& ot) {
  // the folding piece lies in group c_first: the others are c_first + 1 .. c_last
  bool all = true;
#pragma unroll
  for (int jj = 0; jj < DirectOthers<G>::value; ++jj) {
    const int c = sg.c_first + 1 + jj;
    if (c > sg.c_last) break;
    const int slot = slot_of(p, sg.kvh, c);
    uint2 wl[G], wo[G];
#pragma unroll
    for (int q = 0; q < G; ++q) {
      wl[q] = ld_word(slot_word<G>(p, slot, G * kHeadDim + q));
      wo[q] = ld_word(slot_word<G>(p, slot, q * kHeadDim + t));
    }
#pragma unroll
    for (int q = 0; q < G; ++q) {
      all = all && wl[q].y == tag && wo[q].y == tag;
      ot.lse[q][jj] = __uint_as_float(wl[q].x);
      ot.o[q][jj] = __uint_as_float(wo[q].x);
    }
  }
  return all;
}

// Fold a row: this piece (group c_first, values in registers) and the pieces of the groups after
// it, in group order, with the arithmetic of the LSE merge kernel; store the BF16 row.  Values
// not fetched ahead are loaded now, waiting (bounded) for words that have not arrived.  Returns
// false, storing nothing, if a piece failed.
template <int G>
__device__ __forceinline__ bool fold_row(const DecodeParams& p, const Seg& sg, int t, uint32_t tag,
                                         const float (&val)[G], const float (&lse)[G], const Others<G>& ot,
                                         bool fetched) {
  const int64_t orow = p.out_indices ? (int64_t)p.out_indices[sg.row] : (int64_t)sg.row;
  const int others = sg.c_last - sg.c_first;
  bool bad = false;
  float mx[G], tot[G], acc[G];
#pragma unroll
  for (int q = 0; q < G; ++q) mx[q] = lse[q];
  if (fetched) {
#pragma unroll
    for (int jj = 0; jj < DirectOthers<G>::value; ++jj)
      if (jj < others) {
#pragma unroll
        for (int q = 0; q < G; ++q) mx[q] = fmaxf(mx[q], ot.lse[q][jj]);
      }
  } else {
    for (int j = 0; j < others; ++j) {
      const int slot = slot_of(p, sg.kvh, sg.c_first + 1 + j);
      uint2 w[G];
#pragma unroll
      for (int q = 0; q < G; ++q) w[q] = ld_word(slot_word<G>(p, slot, G * kHeadDim + q));
#pragma unroll
      for (int q = 0; q < G; ++q)
        mx[q] = fmaxf(mx[q], wait_word(slot_word<G>(p, slot, G * kHeadDim + q), w[q], tag, p.status, &bad));
    }
  }
#pragma unroll
  for (int q = 0; q < G; ++q) {
    tot[q] = 0.f; acc[q] = 0.f;
    if (lse[q] != -INFINITY) {   // an empty piece weighs nothing, whatever its O holds
      const float wgt = expf(lse[q] - mx[q]);
      tot[q] = wgt;
      acc[q] = wgt * val[q];
    }
  }
  if (fetched) {
#pragma unroll
    for (int jj = 0; jj < DirectOthers<G>::value; ++jj)
      if (jj < others) {
#pragma unroll
        for (int q = 0; q < G; ++q) {
          if (ot.lse[q][jj] == -INFINITY) continue;
          const float wgt = expf(ot.lse[q][jj] - mx[q]);
          tot[q] += wgt;
          acc[q] = fmaf(wgt, ot.o[q][jj], acc[q]);
        }
      }
  } else {
    for (int j = 0; j < others; ++j) {
      const int slot = slot_of(p, sg.kvh, sg.c_first + 1 + j);
      uint2 wl[G], wo[G];
#pragma unroll
      for (int q = 0; q < G; ++q) {
        wl[q] = ld_word(slot_word<G>(p, slot, G * kHeadDim + q));
        wo[q] = ld_word(slot_word<G>(p, slot, q * kHeadDim + t));
      }
#pragma unroll
      for (int q = 0; q < G; ++q) {
        const float ls = wait_word(slot_word<G>(p, slot, G * kHeadDim + q), wl[q], tag, p.status, &bad);
        const float ov = wait_word(slot_word<G>(p, slot, q * kHeadDim + t), wo[q], tag, p.status, &bad);
        if (ls == -INFINITY) continue;
        const float wgt = expf(ls - mx[q]);
        tot[q] += wgt;
        acc[q] = fmaf(wgt, ov, acc[q]);
      }
    }
  }
  if (bad) return false;
#pragma unroll
  for (int q = 0; q < G; ++q) {
    const float r = tot[q] > 0.f ? __fdiv_rn(acc[q], tot[q]) : 0.f;
    p.out[(orow * p.heads_q + sg.kvh * G + q) * kHeadDim + t] = __bfloat16_as_ushort(__float2bfloat16_rn(r));
  }
  return true;
}

template <int G>
__global__ void __launch_bounds__(kThreads, 2)
decode_persistent_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                         const DecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  Smem<G>& sm = *reinterpret_cast<Smem<G>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int kKS = KSlots<G>::value, kVS = VSlots<G>::value;
  using C = Cols;

  // ---- set-up: schedule (K producer warp), barriers, tensor memory, zeroed operand tiles ----
  const bool is_k_producer = warp == kKProducerWarp, is_v_producer = warp == kVProducerWarp;
  const bool is_producer = is_k_producer || is_v_producer;
  if (is_k_producer) {
    if (lane == 0) {
      for (int s = 0; s < kKS; ++s) { mbar_init(&sm.k_full[s], 1); mbar_init(&sm.k_empty[s], 1); }
      for (int s = 0; s < kVS; ++s) { mbar_init(&sm.v_full[s], 1); mbar_init(&sm.v_empty[s], 1); }
      sm.abort_flag = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    build_schedule<G>(p, sm, lane);
    __syncwarp();
  }
  if (tid == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.s_full[b], 1); mbar_init(&sm.s_free[b], 128);
      mbar_init(&sm.p_full[b], 128);
      mbar_init(&sm.o_full[b], 1); mbar_init(&sm.o_free[b], 128);
      mbar_init(&sm.q_full[b], 128);
      mbar_init(&sm.drain[b], 1);
    }
    for (int b = 0; b < 8; ++b) mbar_init(&sm.seg_done[b], 128);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kQkWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&sm.tmem_base)),
                 "r"(C::kAlloc)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (!is_producer) {
    // rows G..7 of the N = 8 operands and their scale rows stay zero for the whole kernel
    constexpr int kWorkers = kThreads - 64;
    const int wt = tid < kKProducerWarp * 32 ? tid : tid - 32;   // warps 0-7, 9, 10 -> 0..319
    for (int i = wt; i < 2 * NQ * 64 / 16; i += kWorkers) reinterpret_cast<uint4*>(sm.q_tile)[i] = make_uint4(0, 0, 0, 0);
    for (int i = wt; i < 2 * kBatch * NQ * 64 / 16; i += kWorkers)
      reinterpret_cast<uint4*>(sm.p_tile)[i] = make_uint4(0, 0, 0, 0);
    for (int i = wt; i < 2 * kBatch * kSfBlockBytes / 16; i += kWorkers)
      reinterpret_cast<uint4*>(sm.p_sf)[i] = make_uint4(0, 0, 0, 0);
    if (!p.q_fp4)
      for (int i = wt; i < 2 * kSfBlockBytes / 16; i += kWorkers) reinterpret_cast<uint4*>(sm.q_sf)[i] = make_uint4(0, 0, 0, 0);
  }
  // the K producer needs nothing the others prepare: it only signals the set-up barrier
  tc_fence_before();
  if (is_k_producer) asm volatile("bar.arrive 4, %0;" ::"n"(kThreads) : "memory");
  else asm volatile("bar.sync 4, %0;" ::"n"(kThreads) : "memory");
  tc_fence_after();
  const uint32_t tmem = is_k_producer ? 0u : sm.tmem_base;
  const int nseg = sm.nseg;   // no share of this step (nseg 0): every role falls through its loop

  if (warp < 4) {
    // =====================  score threads  =====================
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    if (p.pdl) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      if (tid == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    // Query operand of a piece, in two steps so that the fetch runs under the previous piece:
    // fetch (cp.async: the packed rows and their scale block straight into place, or the BF16
    // rows into the staging buffer), then, once landed, quantise the staged rows if need be
    // and hand the operand to the issuer.
    auto fetch_query = [&](const Seg& sg, int buf) {
      if (p.q_fp4) {
        if (tid < G * 4) {
          const int q = tid >> 2, c = tid & 3;
          cp_async16(sm.q_tile[buf] + sw64_offset(q, c * 16),
                     p.q_fp4 + ((int64_t)sg.row * p.heads_q + sg.kvh * G + q) * 64 + c * 16);
        }
        if (tid >= 64)
          cp_async16(sm.q_sf[buf] + (tid - 64) * 16,
                     p.q_sf + (int64_t)sg.row * p.heads_q * kSfBlockBytes + (int64_t)sg.kvh * kSfBlockBytes +
                         (tid - 64) * 16);
      } else {
        for (int it = tid; it < G * 16; it += 128) {
          const int q = it >> 4, c = it & 15;
          cp_async16(sm.q_stage[buf] + q * kHeadDim + c * 8,
                     p.q_bf16 + (int64_t)sg.row * p.q_row_stride + (int64_t)(sg.kvh * G + q) * p.q_head_stride + c * 8);
        }
      }
    };
    auto publish_query = [&](int buf) {
      cp_async_wait_all();
      if (!p.q_fp4) {
        asm volatile("bar.sync 1, 128;" ::: "memory");   // every thread's staged bytes are visible
        for (int it = tid; it < G * 8; it += 128) {
          // one 16-channel group per thread, with the arithmetic of the stand-alone query quantiser
          const int q = it >> 3, g = it & 7;
          float x[16];
          unpack_bf16x8(*reinterpret_cast<const uint4*>(sm.q_stage[buf] + q * kHeadDim + g * 16), x);
          unpack_bf16x8(*reinterpret_cast<const uint4*>(sm.q_stage[buf] + q * kHeadDim + g * 16 + 8), x + 8);
          uint32_t lo, hi;
          uint8_t sf;
          quantize_group16(x, lo, hi, sf);
          *reinterpret_cast<uint2*>(sm.q_tile[buf] + sw64_offset(q, g * 8)) = make_uint2(lo, hi);
          sm.q_sf[buf][sf_offset(q, g)] = sf;
        }
      }
      fence_proxy_async();
      mbar_arrive(&sm.q_full[buf]);
    };
    // the pieces with pages, in order: qi counts them; next_q finds the one after a given index
    auto next_with_pages = [&](int from) {
      int s = from;
      while (s < nseg && sm.seg[s].last_page == sm.seg[s].first_page) ++s;
      return s;
    };
    int qi = 0;                                 // pieces with pages seen so far
    int s_fetch = next_with_pages(0);           // piece whose query is fetched but not yet published
    if (s_fetch < nseg) {
      fetch_query(sm.seg[s_fetch], 0);
      publish_query(0);
      s_fetch = next_with_pages(s_fetch + 1);
      if (s_fetch < nseg) fetch_query(sm.seg[s_fetch], 1);
    }
    constexpr int QPW = (G + 3) / 4;
    bool alive = true;
    int page_g = 0, kb_g = 0, tails_seen = 0, ai = 0;
    for (int s = 0; s < nseg; ++s) {
      const Seg& sg = sm.seg[s];
      const int n_pages = sg.last_page - sg.first_page;
      if (n_pages == 0 && sg.tail_len == 0) continue;   // the output threads deal with an empty piece
      float m_w[QPW], l_w[QPW];
#pragma unroll
      for (int k = 0; k < QPW; ++k) { m_w[k] = -INFINITY; l_w[k] = 0.f; }
      if (sg.tail_len > 0) {
        // the previous tail's P must have been consumed before this one's is written
        if (tails_seen > 0) asm volatile("bar.sync 5, 256;" ::: "memory");
        ++tails_seen;
        TileWork w;
        w.row = sg.row; w.kvh = sg.kvh; w.split = 0; w.slot = 0; w.first_page = sg.first_page;
        w.last_page = sg.last_page; w.tail_len = sg.tail_len; w.tail_id = sg.tail_id;
        for (int it = tid; it < G * 16; it += 128) {
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
        tail_scores<G>(p, w, sm.qb, sm.pf, sm.red_tail, tid, 1, m, l);
        asm volatile("bar.sync 2, 256;" ::: "memory");  // P of the tail visible to the output threads
        block_sum_128<G>(l, sm.red_tail, tid, 1);
#pragma unroll
        for (int k = 0; k < QPW; ++k) {
          const int q = warp + 4 * k;
#pragma unroll
          for (int qq = 0; qq < G; ++qq)
            if (qq == q) { m_w[k] = m[qq]; l_w[k] = lane == 0 ? l[qq] : 0.f; }
        }
      }
      const int n_batches = (n_pages + kBatch - 1) / kBatch;
      for (int kb = 0; kb < n_batches; ++kb, ++kb_g) {
        const int set = kb_g & 1, i0 = page_g + kb * kBatch;
        const bool two = kb * kBatch + 1 < n_pages;
        const bool ok = alive && mbar_wait(&sm.s_full[set], (kb_g >> 1) & 1, sm, p.status);
        if (ok) {
          tc_fence_after();
          uint32_t r[C::kSet];
          tmem_ld16(tmem + lane_off + C::kS + set * C::kSet, r);
          tc_fence_before();
          mbar_arrive(&sm.s_free[set]);
          const bool ok0 = sm.page_ok[i0 & 31] != 0;
          const bool ok1 = two && sm.page_ok[(i0 + 1) & 31] != 0;
#pragma unroll
          for (int q = 0; q < G; ++q) {
            sm.z[set][0][q * kPage + tid] = ok0 ? __uint_as_float(r[q]) * p.scale_log2 : -INFINITY;
            sm.z[set][1][q * kPage + tid] = ok1 ? __uint_as_float(r[NQ + q]) * p.scale_log2 : -INFINITY;
          }
        }
        if (!bar_and_128(1, ok)) alive = false;
        if (alive) {
          // P.V of the pair two hand-overs back has retired: its P tiles, their scale rows and the
          // rescale slots of the pair four hand-overs back may be overwritten
          if (kb_g >= 2 && !mbar_wait(&sm.o_full[set], ((kb_g - 2) >> 1) & 1, sm, p.status)) alive = false;
#pragma unroll
          for (int k = 0; k < QPW; ++k) {
            const int q = warp + 4 * k;
            if (q < G) {
              const float4 za = *reinterpret_cast<const float4*>(&sm.z[set][0][q * kPage + 4 * lane]);
              const PageMax ma = page_max(za);
              const float m1 = fmaxf(m_w[k], ma.page);
              const float ra = (m_w[k] == -INFINITY) ? 0.f : exp2f(m_w[k] - m1);
              const float sa = quantize_page(za, ma.group, m1, sm.p_tile[set][0], sm.p_sf[set][0], q, lane);
              const float4 zb = *reinterpret_cast<const float4*>(&sm.z[set][1][q * kPage + 4 * lane]);
              const PageMax mb = page_max(zb);
              const float m2 = fmaxf(m1, mb.page);
              const float rb = (m1 == -INFINITY) ? 0.f : exp2f(m1 - m2);
              const float sb = quantize_page(zb, mb.group, m2, sm.p_tile[set][1], sm.p_sf[set][1], q, lane);
              m_w[k] = m2;
              l_w[k] = fmaf(fmaf(l_w[k], ra, sa), rb, sb);
              if (lane == 0) {
                sm.resc[i0 & 7][q] = ra;
                sm.resc[(i0 + 1) & 7][q] = rb;
              }
            }
          }
          fence_proxy_async();
          mbar_arrive(&sm.p_full[set]);
        }
        // the next piece's query has landed by now: quantise it and hand it to the issuer
        if (kb == 0 && s_fetch < nseg && s_fetch > s) {
          publish_query((qi + 1) & 1);
          s_fetch = nseg;   // published; the fetch after it starts with the next piece
        }
      }
      page_g += n_pages;
      // row sums and final maxima of every query head, for the output threads
#pragma unroll
      for (int k = 0; k < QPW; ++k) {
        const int q = warp + 4 * k;
        if (q < G) {
          const float ls = warp_sum(l_w[k]);
          if (lane == 0) { sm.fin[ai & 7][q] = ls; sm.fin[ai & 7][NQ + q] = m_w[k]; }
        }
      }
      mbar_arrive(&sm.seg_done[ai & 7]);
      ++ai;
      if (n_pages > 0) {
        ++qi;
        // start fetching the query of the piece after the next one with pages (its buffer was
        // last used by this piece, whose products have all retired)
        const int nxt = next_with_pages(s + 1);
        if (nxt < nseg) {
          const int after = next_with_pages(nxt + 1);
          if (after < nseg) { fetch_query(sm.seg[after], (qi + 1) & 1); s_fetch = after; }
        }
      }
    }
    if (tails_seen > 0) asm volatile("bar.sync 5, 256;" ::: "memory");
  } else if (warp < 8) {
    // =====================  output threads: thread t = channel t  =====================
    const int t = tid - 128;
    const uint32_t lane_off = (uint32_t)((warp - 4) * 32) << 16;
    if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");   // before the tail is read or anything is stored
    bool alive = true;
    int page_g = 0, kb_g = 0, ai = 0;
    const int my_group = (int)blockIdx.x / p.heads_kv;
    // this launch's tag for the scratch slots: one more than the launches that completed on them
    const uint32_t tag = (uint32_t)(*reinterpret_cast<volatile int*>(p.tile_counters) + 1) & ~kFailBit;
    for (int s = 0; s < nseg; ++s) {
      const Seg& sg = sm.seg[s];
      const int n_pages = sg.last_page - sg.first_page;
      float o[G], lse[G];
#pragma unroll
      for (int q = 0; q < G; ++q) { o[q] = 0.f; lse[q] = -INFINITY; }
      // A row cut over several groups is folded by the group that holds its first unit: every
      // other group walks its piece of the row FIRST (rows lie in order) and stores its partial,
      // waiting for nothing; the folding group walks its piece LAST, so the others have normally
      // arrived long before it ends.  It fetches their words one hand-over before its last, while
      // its last pages are folded, and only waits (bounded) for words still missing at its end.
      const bool is_cut = sg.slot >= 0;
      const bool folds = is_cut && my_group == sg.c_first;
      const int others = sg.c_last - sg.c_first;
      const int n_batches = (n_pages + kBatch - 1) / kBatch;
      bool fetched = false;
      Others<G> ot;
      auto look = [&]() {
        if (others <= DirectOthers<G>::value) fetched = fetch_others<G>(p, sg, t, tag, ot);
      };
      if (folds && n_batches < 2) look();
      if (sg.tail_len > 0) {
        TileWork w;
        w.row = sg.row; w.kvh = sg.kvh; w.split = 0; w.slot = 0; w.first_page = sg.first_page;
        w.last_page = sg.last_page; w.tail_len = sg.tail_len; w.tail_id = sg.tail_id;
        asm volatile("bar.sync 2, 256;" ::: "memory");
        tail_pv<G>(p, w, sm.pf, t, o);
        asm volatile("bar.arrive 5, 256;" ::: "memory");   // P of this tail has been consumed
      }
      for (int kb = 0; kb < n_batches; ++kb, ++kb_g) {
        const int set = kb_g & 1, j0 = page_g + kb * kBatch;
        const bool two = kb * kBatch + 1 < n_pages;
        if (folds && kb == n_batches - 2) look();
        if (alive && mbar_wait(&sm.o_full[set], (kb_g >> 1) & 1, sm, p.status)) {
          tc_fence_after();
          uint32_t ro[C::kSet];
          tmem_ld16(tmem + lane_off + C::kO + set * C::kSet, ro);
          tc_fence_before();
          float ra[G], rb[G];
#pragma unroll
          for (int q = 0; q < G; ++q) { ra[q] = sm.resc[j0 & 7][q]; rb[q] = sm.resc[(j0 + 1) & 7][q]; }
          mbar_arrive(&sm.o_free[set]);
#pragma unroll
          for (int q = 0; q < G; ++q) {
            o[q] = fmaf(o[q], ra[q], __uint_as_float(ro[q]));
            if (two) o[q] = fmaf(o[q], rb[q], __uint_as_float(ro[NQ + q]));
          }
        } else {
          alive = false;
        }
      }
      page_g += n_pages;
      float val[G];
      if (n_pages > 0 || sg.tail_len > 0) {
        if (alive && !mbar_wait(&sm.seg_done[ai & 7], (ai >> 3) & 1, sm, p.status)) alive = false;
#pragma unroll
        for (int q = 0; q < G; ++q) {
          const float lq = sm.fin[ai & 7][q], mq = sm.fin[ai & 7][NQ + q];
          val[q] = lq > 0.f ? __fdiv_rn(o[q], lq) : 0.f;
          lse[q] = lq > 0.f ? (mq + log2f(lq)) * kLn2 : -INFINITY;
        }
        ++ai;
      } else {   // an empty piece: a zero row, or an empty partial
#pragma unroll
        for (int q = 0; q < G; ++q) val[q] = 0.f;
      }
      const bool ok = alive && !sm.abort_flag;
      // ---- end of the piece ----
      if (!is_cut) {
        if (ok) {
          const int64_t orow = p.out_indices ? (int64_t)p.out_indices[sg.row] : (int64_t)sg.row;
#pragma unroll
          for (int q = 0; q < G; ++q)
            p.out[(orow * p.heads_q + sg.kvh * G + q) * kHeadDim + t] =
                __bfloat16_as_ushort(__float2bfloat16_rn(val[q]));
        }
      } else if (!folds) {
        // a failed piece marks its LSE words, so that the folding piece leaves the row alone
#pragma unroll
        for (int q = 0; q < G; ++q) {
          if (ok) st_word(slot_word<G>(p, sg.slot, q * kHeadDim + t), val[q], tag);
          if (t == 0) st_word(slot_word<G>(p, sg.slot, G * kHeadDim + q), lse[q], ok ? tag : (tag | kFailBit));
        }
      } else if (ok) {
        fold_row<G>(p, sg, t, tag, val, lse, ot, fetched);
      }
    }
  } else if (is_producer) {
    // =====================  producers (K ring: warp 8, V ring: warp 11)  =====================
    // The pages of all pieces form one sequence of walk steps.  Lane l looks up the page id of
    // step 32 c + l of chunk c (one chunk ahead of its use); lane 0 issues the loads.
    const int slots = is_k_producer ? kKS : kVS;
    int total = 0;
    for (int s = 0; s < nseg; ++s) total += sm.seg[s].last_page - sm.seg[s].first_page;
    auto lookup = [&](int step, int& kvh) -> int {
      int pid = -1;
      kvh = 0;
      if (step < total) {
        int acc = 0;
        for (int s = 0; s < nseg; ++s) {
          const int n = sm.seg[s].last_page - sm.seg[s].first_page;
          if (step < acc + n) {
            const int page = sm.seg[s].last_page - 1 - (step - acc);
            pid = __ldg(p.page_table + (int64_t)sm.seg[s].row * p.page_table_row_stride + page);
            kvh = sm.seg[s].kvh;
            if (pid < 0 || (int64_t)pid >= p.num_pages) {
              if (is_k_producer) set_status(p.status, NVFP4_STATUS_BAD_PAGE_ID);
              pid = -1;
            }
            break;
          }
          acc += n;
        }
      }
      return pid;
    };
    int kvh_cur, kvh_next = 0;
    int id_cur = lookup(lane, kvh_cur), id_next = -1;
    int alive = 1;
    for (int base = 0; base < total && alive; base += 32) {
      if (base + 32 < total) id_next = lookup(base + 32 + lane, kvh_next);
      const int in_chunk = min(32, total - base);
      for (int j = 0; j < in_chunk; ++j) {
        const int pid = __shfl_sync(0xffffffffu, id_cur, j);
        const int kvh = __shfl_sync(0xffffffffu, kvh_cur, j);
        if (lane == 0) {
          const int i = base + j, s = i % slots;
          uint8_t* st = is_k_producer ? sm.k_slot[s] : sm.v_slot[s];
          uint64_t* bar = is_k_producer ? &sm.k_full[s] : &sm.v_full[s];
          uint64_t* freed = is_k_producer ? &sm.k_empty[s] : &sm.v_empty[s];
          if (i >= slots && !mbar_wait(freed, ((i / slots) & 1) ^ 1, sm, p.status)) {
            alive = 0;
          } else {
            if (is_k_producer) sm.page_ok[i & 31] = pid >= 0 ? 1 : 0;
            if (pid >= 0) {
              mbar_expect_tx(bar, kSlotBytes);
              if (is_k_producer) {
                tma_load_4d(smem_u32(st), &k_map, bar, 0, kvh, 0, pid);
                bulk_load(smem_u32(st + kTileBytes), p.k_sf + (int64_t)pid * p.k_sf_pitch + (int64_t)kvh * kSfBlockBytes,
                          kSfBlockBytes, bar);
              } else {
                tma_load_4d(smem_u32(st), &v_map, bar, 0, 0, kvh, pid);
                bulk_load(smem_u32(st + kTileBytes), p.v_sf + (int64_t)pid * p.v_sf_pitch + (int64_t)kvh * kSfBlockBytes,
                          kSfBlockBytes, bar);
              }
            } else {
              // a page id outside the cache is never turned into an address: the slot gets zero
              // scales (so its product is zero) and the score threads mask its scores
              for (int k = 0; k < kSfBlockBytes / 16; ++k)
                reinterpret_cast<uint4*>(st + kTileBytes)[k] = make_uint4(0, 0, 0, 0);
              fence_proxy_async();
              mbar_arrive(bar);
            }
          }
        }
        alive = __shfl_sync(0xffffffffu, alive, 0);
        if (!alive) break;
      }
      id_cur = id_next; kvh_cur = kvh_next;
    }
  } else if (warp == kQkWarp) {
    // =====================  MMA issuer 1: S^T = K . Q^T  =====================
    if (lane == 0) {
      bool alive = true;
      int i = 0, kb_g = 0, qi = 0;
      for (int s = 0; s < nseg && alive; ++s) {
        const int n_pages = sm.seg[s].last_page - sm.seg[s].first_page;
        if (n_pages == 0) continue;
        const int buf = qi & 1;
        alive = mbar_wait(&sm.q_full[buf], (qi >> 1) & 1, sm, p.status);
        if (!alive) break;
        ++qi;
        tc_fence_after();
        cp_sf(tmem + C::kSfQ, smem_u32(sm.q_sf[buf]));
        cp_sf(tmem + C::kSfQ + 4, smem_u32(sm.q_sf[buf] + 512));
        const uint64_t q_desc = desc_sw64(smem_u32(sm.q_tile[buf]));
        const int n_batches = (n_pages + kBatch - 1) / kBatch;
        for (int kb = 0; kb < n_batches && alive; ++kb, ++kb_g) {
          const int set = kb_g & 1;
          alive = mbar_wait(&sm.s_free[set], ((kb_g >> 1) & 1) ^ 1, sm, p.status);
          for (int u = 0; u < kBatch && alive; ++u) {
            if (kb * kBatch + u >= n_pages) break;
            const int sl = i % kKS;
            alive = mbar_wait(&sm.k_full[sl], (i / kKS) & 1, sm, p.status);
            if (!alive) break;
            tc_fence_after();
            const uint32_t st = smem_u32(sm.k_slot[sl]);
            cp_sf(tmem + C::kSfK, st + kTileBytes);
            cp_sf(tmem + C::kSfK + 4, st + kTileBytes + 512);
            const uint64_t k_desc = desc_sw64(st);
            const uint32_t d = tmem + C::kS + set * C::kSet + u * NQ;
            mma_nvf4<NQ>(d, k_desc, q_desc, tmem + C::kSfK, tmem + C::kSfQ, 0);
            mma_nvf4<NQ>(d, k_desc + 2, q_desc + 2, tmem + C::kSfK + 4, tmem + C::kSfQ + 4, 1);
            mma_commit(&sm.k_empty[sl]);   // the K slot goes back once this page's product has retired
            ++i;
          }
          if (alive) mma_commit(&sm.s_full[set]);
        }
      }
      // everything this thread issued must have retired before tensor memory is freed
      mma_commit(&sm.drain[0]);
      mbar_wait(&sm.drain[0], 0, sm, p.status);
    }
    __syncwarp();
  } else if (warp == kPvWarp) {
    // =====================  MMA issuer 2: O^T = V^T . P^T  =====================
    if (lane == 0) {
      bool alive = true;
      int j = 0, kb_g = 0;
      for (int s = 0; s < nseg && alive; ++s) {
        const int n_pages = sm.seg[s].last_page - sm.seg[s].first_page;
        const int n_batches = (n_pages + kBatch - 1) / kBatch;
        for (int kb = 0; kb < n_batches && alive; ++kb, ++kb_g) {
          const int set = kb_g & 1;
          // the V scale blocks of the pair go to tensor memory as soon as their slots have landed
          for (int u = 0; u < kBatch && alive; ++u) {
            if (kb * kBatch + u >= n_pages) break;
            const int sl = (j + u) % kVS;
            alive = mbar_wait(&sm.v_full[sl], ((j + u) / kVS) & 1, sm, p.status);
            if (!alive) break;
            tc_fence_after();
            const uint32_t st = smem_u32(sm.v_slot[sl]);
            const uint32_t c = tmem + C::kSfV + (set * kBatch + u) * 8;
            cp_sf(c, st + kTileBytes);
            cp_sf(c + 4, st + kTileBytes + 512);
          }
          alive = alive && mbar_wait(&sm.p_full[set], (kb_g >> 1) & 1, sm, p.status) &&
                  mbar_wait(&sm.o_free[set], ((kb_g >> 1) & 1) ^ 1, sm, p.status);
          if (!alive) break;
          tc_fence_after();
          for (int u = 0; u < kBatch; ++u) {
            if (kb * kBatch + u >= n_pages) break;
            const int sl = j % kVS;
            const uint32_t c = tmem + C::kSfV + (set * kBatch + u) * 8;
            cp_sf(tmem + C::kSfP, smem_u32(sm.p_sf[set][u]));
            cp_sf(tmem + C::kSfP + 4, smem_u32(sm.p_sf[set][u] + 512));
            const uint64_t v_desc = desc_sw64(smem_u32(sm.v_slot[sl]));
            const uint64_t p_desc = desc_sw64(smem_u32(sm.p_tile[set][u]));
            const uint32_t d = tmem + C::kO + set * C::kSet + u * NQ;
            mma_nvf4<NQ>(d, v_desc, p_desc, c, tmem + C::kSfP, 0);
            mma_nvf4<NQ>(d, v_desc + 2, p_desc + 2, c + 4, tmem + C::kSfP + 4, 1);
            mma_commit(&sm.v_empty[sl]);   // the V slot goes back once this page's product has retired
            ++j;
          }
          mma_commit(&sm.o_full[set]);
        }
      }
      mma_commit(&sm.drain[1]);
      mbar_wait(&sm.drain[1], 0, sm, p.status);
    }
    __syncwarp();
  }

  // ---- teardown ----
  tc_fence_before();
  __syncthreads();
  if (is_producer && lane == 0 && sm.abort_flag) {
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(sm.tmem_base), "r"(C::kAlloc)
                 : "memory");
  }
  // The CTA that leaves last counts the launch: the next one tags its scratch words one higher.
  // (Thread 0 has passed griddepcontrol.wait, so under a programmatic launch the previous
  // launch's own count is complete.)
  if (tid == 0) {
    int* launches = p.tile_counters;
    int* left = p.tile_counters + 1;
    if (atomicAdd(left, 1) == (int)gridDim.x - 1) {
      *left = 0;
      *launches = (*reinterpret_cast<volatile int*>(launches) + 1) & 0x3fffffff;
    }
  }
}

template <int G>
static cudaError_t launch_g(const DecodeParams& p, const CUtensorMap& km, const CUtensorMap& vm, int ctas,
                            cudaStream_t stream) {
  const size_t smem = sizeof(Smem<G>) + 1024;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    e = cudaFuncSetAttribute(decode_persistent_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, decode_persistent_kernel<G>, km, vm, p);
}

}  // namespace sm100p

int decode_persistent_ctas() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!cached[dev]) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = 2 * sms;
  }
  return cached[dev];
}

bool decode_persistent_supports(const DecodeParams& p) {
  if (p.heads_kv < 1 || p.heads_q % p.heads_kv) return false;
  const int g = p.heads_q / p.heads_kv;
  if (!(g == 1 || g == 2 || g == 4 || g == 8)) return false;
  const int ctas = decode_persistent_ctas();
  if (ctas < 1) return false;
  // pieces per CTA stay below the table's size whatever the lengths are
  const int groups = ctas / p.heads_kv;
  return groups >= 1 && p.rows / groups + 3 <= sm100p::kMaxSeg && p.rows <= 32768;
}

size_t decode_persistent_workspace_bytes(int rows, int heads_q, int heads_kv) {
  const int ctas = decode_persistent_ctas();
  if (ctas < 1 || heads_kv < 1 || rows < 1) return 0;
  const size_t g = (size_t)(heads_q / heads_kv);
  return 256 + (size_t)ctas * g * (kHeadDim + 1) * 2 * sizeof(uint32_t);
}

// workspace: [launch counter, CTAs that have left: two ints, zero-filled once, padded to 256 bytes]
//            [one scratch slot per CTA: G x 129 words {value, tag}]
cudaError_t launch_decode_persistent(const DecodeParams& p0, void* workspace, cudaStream_t stream) {
  if (p0.rows == 0) return cudaSuccess;
  if (!decode_persistent_supports(p0)) return cudaErrorNotSupported;
  if (p0.num_pages < 1 || p0.num_pages > 0x7FFFFFFF) return cudaErrorInvalidValue;
  const int ctas = decode_persistent_ctas();
  const int g = p0.heads_q / p0.heads_kv;
  DecodeParams p = p0;
  p.tile_counters = static_cast<int*>(workspace);
  p.o_partial = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256);
  p.lse_partial = nullptr;
  p.emit_partial = 0;
  p.num_splits = 1;
  // no more CTAs than shares of kMinShare units the longest possible step could fill
  const int64_t max_units = (int64_t)p.rows * (p.max_pages + sm100p::tail_units(kPage) + 1);
  int64_t want = (max_units + sm100p::kMinShare - 1) / sm100p::kMinShare;   // groups the longest step could fill
  const int groups = ctas / p.heads_kv;
  want = want < 1 ? 1 : (want < groups ? want : groups);
  const int grid = (int)want * p.heads_kv;
  CUtensorMap km, vm;
  cudaError_t e = sm100::make_map(0, p.k_packed, p.k_pitch, p.num_pages, p.heads_kv, &km);
  if (e != cudaSuccess) return e;
  e = sm100::make_map(1, p.v_packed, p.v_pitch, p.num_pages, p.heads_kv, &vm);
  if (e != cudaSuccess) return e;
  switch (g) {
    case 1: return sm100p::launch_g<1>(p, km, vm, grid, stream);
    case 2: return sm100p::launch_g<2>(p, km, vm, grid, stream);
    case 4: return sm100p::launch_g<4>(p, km, vm, grid, stream);
    case 8: return sm100p::launch_g<8>(p, km, vm, grid, stream);
    default: return cudaErrorNotSupported;
  }
}

}  // namespace nvfp4
