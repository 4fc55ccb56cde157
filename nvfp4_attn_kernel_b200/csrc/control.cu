// Per-step bookkeeping of the BF16 tail slots, resolved on the device by one CTA:
// row -> slot matching keyed on the row's first physical block, least-recently-seen
// reclamation, the FP4/tail split of every row, the promotion table and sticky error flags.
// Thread i plays row i and slot i; all tables live in shared memory (at most 128 slots).
// With four warps on an SM nothing hides latency, so the launch is laid out for few dependent
// steps: every global load sits in straight-line code (all in flight at once, the one block id
// a page-filling row needs included, fetched as soon as the row's length is there); the searches
// over slots and rows read the tables four entries per load, unrolled; ranks among the rows are
// ballots; the least-recently-seen ranking - the one quadratic step with 64-bit compares - runs
// only in a step where some row needs a new slot; owners and allocations are scatters.
// Also the page work table that tells the page quantiser which full pages a prefill step brings.
#include <climits>

#include "nvfp4_common.cuh"
#include "nvfp4_kernels.h"
#include "worklist.cuh"

namespace nvfp4 {

constexpr int kMaxSlots = 128;
constexpr int kFreeKey = -1, kNullBlock = 0, kInactive = -1;
constexpr int kErrContinuationPrefill = 1, kErrSlotLost = 2, kErrStaleHistory = 4, kErrNoFreeSlot = 8,
              kErrDuplicateKey = 16, kErrPromotionColumn = 32, kErrWorkListFull = 64;

__global__ void __launch_bounds__(kMaxSlots) control_kernel(const ControlArgs a) {
  __shared__ __align__(16) int key[kMaxSlots], live[kMaxSlots], slot_key[kMaxSlots], is_free[kMaxSlots];
  __shared__ __align__(16) long long slot_last_seen[kMaxSlots];
  __shared__ int seq[kMaxSlots], q_begin[kMaxSlots], q_end[kMaxSlots], slot_last_seq[kMaxSlots];
  __shared__ int claimed[kMaxSlots], slot_of[kMaxSlots], slot_by_rank[kMaxSlots], owner[kMaxSlots];
  __shared__ unsigned need_bits[kMaxSlots / 32];
  __shared__ int errors;
  __shared__ long long step_now;
  __shared__ int class_total[kSizeClasses], class_cursor[kSizeClasses], list_used;
  const int i = threadIdx.x, warp = i >> 5, lane = i & 31;
  const int n = a.num_slots;
  const bool in_batch = i < a.num_reqs, is_slot = i < n;
  // all loads of the launch but one, in flight together
  const int my_key = in_batch ? a.block_table[(int64_t)i * a.block_table_stride] : kFreeKey;
  const int my_seq = in_batch ? a.seq_lens[i] : 0;
  const int my_begin = in_batch ? a.query_start_loc[i] : 0;
  const int my_end = in_batch ? a.query_start_loc[i + 1] : 0;
  const int my_slot_key = is_slot ? a.slot_keys[i] : kFreeKey;
  const int my_slot_seq = is_slot ? a.slot_last_seq[i] : -1;
  const long long my_slot_seen = is_slot ? a.slot_last_seen[i] : -1;
  const long long step_before = i == 0 ? *a.step : 0;
  const int query_len = my_end - my_begin;
  const int computed = my_seq - query_len;
  // a row is a request only with both a length and a real block: padding rows keep a stale
  // block under a zero length, rows of a dummy batch a length over the null block
  const bool alive = in_batch && my_seq > 0 && my_key != kNullBlock;
  const int fp4 = alive ? ((my_seq - 1) / kPage) * kPage : 0;
  // where the flush would read and write if this step fills the row's tail page; the block id is
  // fetched now and needed only at the end
  const int column = fp4 / kPage;
  const bool crossing = alive && (my_seq % kPage == 0);
  const bool in_bounds = column < a.block_table_columns;
  const int promotion_page =
      (is_slot && crossing && in_bounds) ? a.block_table[(int64_t)i * a.block_table_stride + column] : kInactive;
  key[i] = my_key;
  seq[i] = my_seq;
  q_begin[i] = my_begin;
  q_end[i] = my_end;
  live[i] = alive;
  slot_key[i] = my_slot_key;
  slot_last_seq[i] = my_slot_seq;
  slot_last_seen[i] = my_slot_seen;
  claimed[i] = 0;
  slot_by_rank[i] = -1;
  owner[i] = INT_MAX;
  if (i < kSizeClasses) class_total[i] = 0;
  if (i == 0) {
    errors = 0;
    step_now = step_before + 1;
    *a.step = step_before + 1;
  }
  __syncthreads();

  // lowest slot whose key is this row's key (slots past n hold the free key and do not count);
  // and whether another live row has this row's key
  int m = kMaxSlots, dup = 0;
  if (alive) {
#pragma unroll 8
    for (int s4 = kMaxSlots / 4 - 1; s4 >= 0; --s4) {
      const int4 k = reinterpret_cast<const int4*>(slot_key)[s4];
      if (k.w == my_key) m = 4 * s4 + 3;
      if (k.z == my_key) m = 4 * s4 + 2;
      if (k.y == my_key) m = 4 * s4 + 1;
      if (k.x == my_key) m = 4 * s4;
    }
#pragma unroll 8
    for (int r4 = 0; r4 < kMaxSlots / 4; ++r4) {
      const int4 k = reinterpret_cast<const int4*>(key)[r4];
      const int4 v = reinterpret_cast<const int4*>(live)[r4];
      dup |= (v.x && k.x == my_key && 4 * r4 != i) | (v.y && k.y == my_key && 4 * r4 + 1 != i) |
             (v.z && k.z == my_key && 4 * r4 + 2 != i) | (v.w && k.w == my_key && 4 * r4 + 3 != i);
    }
  }
  if (m >= n) m = n;
  const bool has_match = m < n;
  if (has_match) claimed[m] = 1;   // benign race: every writer stores 1
  // rows without a slot take the unclaimed slots, least recently seen first
  const bool need = alive && !has_match;
  const unsigned need_word = __ballot_sync(0xffffffffu, need);
  if (lane == 0) need_bits[warp] = need_word;
  __syncthreads();
  const bool free_slot = is_slot && !claimed[i];
  is_free[i] = free_slot;
  int need_rank = __popc(need_word & ((1u << lane) - 1u)), need_total = 0;
#pragma unroll
  for (int w = 0; w < kMaxSlots / 32; ++w) {
    const int c = __popc(need_bits[w]);
    need_total += c;
    if (w < warp) need_rank += c;
  }
  __syncthreads();
  if (need_total > 0) {   // the same for every thread
    // rank of this slot among the free ones, ordered by (last seen, index)
    int fr = 0;
#pragma unroll 8
    for (int s2 = 0; s2 < kMaxSlots / 2; ++s2) {
      const longlong2 seen = reinterpret_cast<const longlong2*>(slot_last_seen)[s2];
      const int2 f = reinterpret_cast<const int2*>(is_free)[s2];
      fr += f.x && (seen.x < my_slot_seen || (seen.x == my_slot_seen && 2 * s2 < i));
      fr += f.y && (seen.y < my_slot_seen || (seen.y == my_slot_seen && 2 * s2 + 1 < i));
    }
    if (free_slot) slot_by_rank[fr] = i;   // the free slots' ranks are 0, 1, 2, ..., once each
    __syncthreads();
  }
  const int by_rank = need ? slot_by_rank[need_rank] : -1;
  const int got = by_rank >= 0;
  const int allocated = got ? by_rank : 0;
  const int slot = alive ? (has_match ? m : allocated) : kInactive;

  int e = 0;
  if (alive && query_len > 1 && computed > 0) e |= kErrContinuationPrefill;
  if (need && computed > 0) e |= kErrSlotLost;
  if (has_match && slot_last_seq[m] != computed && computed > 0) e |= kErrStaleHistory;
  if (need && !got) e |= kErrNoFreeSlot;
  if (alive && dup) e |= kErrDuplicateKey;
  if (is_slot && crossing && !in_bounds) e |= kErrPromotionColumn;
  slot_of[i] = slot;
  if (alive) atomicMin(&owner[slot], i);   // slot state follows the lowest row that landed on it
  if (e) atomicOr(&errors, e);
  __syncthreads();

  if (is_slot) {
    const int r = owner[i];   // unclaimed slots keep their state
    if (r != INT_MAX) {
      a.slot_keys[i] = key[r];
      a.slot_last_seq[i] = seq[r];
      a.slot_last_seen[i] = step_now;
    }
    a.row_to_slot[i] = slot;
    a.seqused_fp4[i] = fp4;
    a.seqused_residual[i] = alive ? my_seq - fp4 : 0;
    a.promotion_source_tokens[i] = alive ? slot * kPage : 0;
    a.promotion_pages[i] = promotion_page;
  }
  if (i == 0 && errors) atomicOr(a.error_code, errors);

  // The balanced split's list of pieces for the step's decode rows, from the lengths just
  // computed (a live row always holds a tail: 1 to 128 tokens).  Same list as the stand-alone
  // builder's; the decode launches of the step's layers then all reuse it.
  if (a.work != nullptr) {   // the same for every thread
    int count = 0, size_class = 0;
    const int tail = alive ? 1 : 0;
    const bool listed = i < a.work_rows;
    if (listed) {
      balanced_pieces_of_row(fp4, tail, a.work_max_pages, a.work_target_pages, count, size_class);
      atomicAdd(&class_total[size_class], count + tail);
    }
    __syncthreads();
    if (i == 0) {
      int at = 0;
      for (int c = 0; c < kSizeClasses; ++c) { class_cursor[c] = at; at += class_total[c]; }
      list_used = at;
    }
    __syncthreads();
    if (listed) {
      const int first = atomicAdd(&class_cursor[size_class], count + tail);
      a.work_row_offset[i] = first;
      a.work_row_count[i] = count + tail;
      if (!balanced_write_row(a.work, a.work_capacity, first, i, count, tail)) atomicOr(a.error_code, kErrWorkListFull);
    }
    for (int w = list_used + i; w < a.work_capacity; w += kMaxSlots) a.work[w] = make_int4(-1, 0, 0, 0);
    for (int w = i; w < a.work_counter_words; w += kMaxSlots) a.work_counters[w] = 0;
  }

  // a token belongs to the row whose [q_begin, q_end) holds it (the rows' ranges ascend)
  for (int t = i; t < a.num_actual_tokens; t += kMaxSlots) {
    int lo = 0, hi = a.num_reqs;   // first row whose q_end exceeds t
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (q_end[mid] > t) hi = mid; else lo = mid + 1;
    }
    a.token_to_slot[t] = (lo < a.num_reqs && live[lo] && t >= q_begin[lo]) ? slot_of[lo] : 0;
  }
}

// One block per prefill row: source token and destination block of each of its full pages.
__global__ void work_table_kernel(const int32_t* __restrict__ query_start_loc,
                                  const int32_t* __restrict__ seqused_fp4,
                                  const int32_t* __restrict__ row_to_slot,
                                  const int32_t* __restrict__ block_table, int64_t block_table_stride,
                                  int32_t* __restrict__ source_tokens, int32_t* __restrict__ destination_pages,
                                  int columns_per_row) {
  const int row = blockIdx.x;
  const int start = query_start_loc[row], end = query_start_loc[row + 1];
  const int slot = row_to_slot[row];
  const int full_pages = seqused_fp4[row] / kPage;
  // only a fresh prefill brings the tokens of its full pages with it
  const bool row_writes = (end - start > 1) && slot >= 0;
  for (int c = threadIdx.x; c < columns_per_row; c += blockDim.x) {
    const bool active = row_writes && c < full_pages;
    const int64_t out = (int64_t)row * columns_per_row + c;
    source_tokens[out] = start + c * kPage;
    destination_pages[out] = active ? block_table[(int64_t)row * block_table_stride + c] : -1;
  }
}

cudaError_t launch_control(const ControlArgs& a, cudaStream_t stream) {
  control_kernel<<<1, kMaxSlots, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_work_table(const int32_t* query_start_loc, const int32_t* seqused_fp4,
                              const int32_t* row_to_slot, const int32_t* block_table,
                              int64_t block_table_stride, int32_t* source_tokens,
                              int32_t* destination_pages, int num_reqs, int columns_per_row,
                              cudaStream_t stream) {
  if (num_reqs == 0 || columns_per_row == 0) return cudaSuccess;
  work_table_kernel<<<num_reqs, 128, 0, stream>>>(query_start_loc, seqused_fp4, row_to_slot, block_table,
                                                  block_table_stride, source_tokens, destination_pages,
                                                  columns_per_row);
  return cudaGetLastError();
}

}  // namespace nvfp4
