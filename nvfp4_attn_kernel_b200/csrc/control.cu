// Per-step bookkeeping of the BF16 tail slots, resolved on the device by one CTA:
// row -> slot matching keyed on the row's first physical block, least-recently-seen
// reclamation, the FP4/tail split of every row, the promotion table and sticky error flags.
// Thread i plays row i and slot i; all tables live in shared memory (at most 128 slots), so the
// quadratic matching is a few thousand shared-memory reads.  Also the page work table that tells
// the page quantiser which full pages a prefill step brings.
#include "nvfp4_common.cuh"
#include "nvfp4_kernels.h"

namespace nvfp4 {

constexpr int kMaxSlots = 128;
constexpr int kFreeKey = -1, kNullBlock = 0, kInactive = -1;
constexpr int kErrContinuationPrefill = 1, kErrSlotLost = 2, kErrStaleHistory = 4, kErrNoFreeSlot = 8,
              kErrDuplicateKey = 16, kErrPromotionColumn = 32;

__global__ void __launch_bounds__(kMaxSlots) control_kernel(const ControlArgs a) {
  __shared__ int key[kMaxSlots], seq[kMaxSlots], q_begin[kMaxSlots], q_end[kMaxSlots], live[kMaxSlots];
  __shared__ int slot_key[kMaxSlots], slot_last_seq[kMaxSlots], matched[kMaxSlots], claimed[kMaxSlots];
  __shared__ long long slot_last_seen[kMaxSlots];
  __shared__ int needs[kMaxSlots], slot_of[kMaxSlots], is_free[kMaxSlots], free_rank[kMaxSlots];
  __shared__ int errors;
  __shared__ long long step_now;
  const int i = threadIdx.x;
  const int n = a.num_slots;
  if (i == 0) {
    errors = 0;
    step_now = *a.step + 1;
    *a.step = step_now;
  }
  const bool in_batch = i < a.num_reqs, is_slot = i < n;
  key[i] = in_batch ? a.block_table[(int64_t)i * a.block_table_stride] : kFreeKey;
  seq[i] = in_batch ? a.seq_lens[i] : 0;
  q_begin[i] = in_batch ? a.query_start_loc[i] : 0;
  q_end[i] = in_batch ? a.query_start_loc[i + 1] : 0;
  // a row is a request only with both a length and a real block: padding rows keep a stale
  // block under a zero length, rows of a dummy batch a length over the null block
  live[i] = in_batch && seq[i] > 0 && key[i] != kNullBlock;
  slot_key[i] = is_slot ? a.slot_keys[i] : kFreeKey;
  slot_last_seq[i] = is_slot ? a.slot_last_seq[i] : -1;
  slot_last_seen[i] = is_slot ? a.slot_last_seen[i] : -1;
  claimed[i] = 0;
  __syncthreads();
  const int query_len = q_end[i] - q_begin[i];
  const int computed = seq[i] - query_len;

  // lowest slot whose key is this row's key
  int m = n;
  if (live[i])
    for (int s = n - 1; s >= 0; --s)
      if (slot_key[s] == key[i]) m = s;
  matched[i] = m;
  const bool has_match = m < n;
  if (has_match) claimed[m] = 1;   // benign race: every writer stores 1
  __syncthreads();

  // rows without a slot take the unclaimed slots, least recently seen first
  needs[i] = live[i] && !has_match;
  is_free[i] = is_slot && !claimed[i];
  __syncthreads();
  int need_rank = 0;
  for (int r = 0; r < i; ++r) need_rank += needs[r];
  int fr = 0;
  if (is_slot)
    for (int s = 0; s < n; ++s)
      if (is_free[s] && (slot_last_seen[s] < slot_last_seen[i] ||
                         (slot_last_seen[s] == slot_last_seen[i] && s < i)))
        ++fr;
  free_rank[i] = fr;
  __syncthreads();
  int allocated = 0, got = 0;
  if (needs[i])
    for (int s = 0; s < n; ++s)
      if (is_free[s] && free_rank[s] == need_rank) { allocated = s; got = 1; }
  const int slot = live[i] ? (has_match ? m : allocated) : kInactive;
  slot_of[i] = slot;

  int e = 0;
  if (live[i] && query_len > 1 && computed > 0) e |= kErrContinuationPrefill;
  if (needs[i] && computed > 0) e |= kErrSlotLost;
  if (has_match && slot_last_seq[m] != computed && computed > 0) e |= kErrStaleHistory;
  if (needs[i] && !got) e |= kErrNoFreeSlot;
  if (live[i])
    for (int r = 0; r < a.num_reqs; ++r)
      if (r != i && live[r] && key[r] == key[i]) e |= kErrDuplicateKey;
  __syncthreads();

  // slot state follows its owner (the lowest row that landed on it); unclaimed slots keep theirs
  if (is_slot) {
    int owner = -1;
    for (int r = a.num_reqs - 1; r >= 0; --r)
      if (live[r] && slot_of[r] == i) owner = r;
    if (owner >= 0) {
      a.slot_keys[i] = key[owner];
      a.slot_last_seq[i] = seq[owner];
      a.slot_last_seen[i] = step_now;
    }
    a.row_to_slot[i] = slot;
    const int fp4 = live[i] ? ((seq[i] - 1) / kPage) * kPage : 0;
    a.seqused_fp4[i] = fp4;
    a.seqused_residual[i] = live[i] ? seq[i] - fp4 : 0;
    // where the flush would read and write if this step fills the row's tail page
    const int column = fp4 / kPage;
    const bool crossing = live[i] && (seq[i] % kPage == 0);
    const bool in_bounds = column < a.block_table_columns;
    if (crossing && !in_bounds) e |= kErrPromotionColumn;
    a.promotion_source_tokens[i] = live[i] ? slot * kPage : 0;
    a.promotion_pages[i] =
        (crossing && in_bounds) ? a.block_table[(int64_t)i * a.block_table_stride + column] : kInactive;
  }
  if (e) atomicOr(&errors, e);
  __syncthreads();
  if (i == 0 && errors) atomicOr(a.error_code, errors);

  for (int t = i; t < a.num_actual_tokens; t += blockDim.x) {
    int v = 0;
    for (int r = 0; r < a.num_reqs; ++r)
      if (live[r] && t >= q_begin[r] && t < q_end[r]) v += slot_of[r];
    a.token_to_slot[t] = v;
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
