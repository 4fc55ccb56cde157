// LSE merge of split-KV partials: lse = log sum_s exp(lse_s), O = sum_s exp(lse_s - lse) O_s.
// One CTA of 128 threads (one per channel) per (query head, row); splits are folded in
// index order, so the result is bitwise reproducible.  The partials may sit at a uniform
// split stride or behind one pointer per split (buffers of peer GPUs mapped into this
// process are read with plain loads).
#include "decode_common.cuh"
#include "worklist.cuh"

namespace nvfp4 {

template <bool kOutF32>
__global__ void __launch_bounds__(128)
lse_merge_kernel(const float* __restrict__ o_parts, int64_t o_split_stride,
                 const float* __restrict__ lse_parts, int64_t lse_split_stride,
                 const float* const* __restrict__ o_ptrs, const float* const* __restrict__ lse_ptrs,
                 int num_splits, int rows, int heads_q, void* __restrict__ out,
                 const int32_t* __restrict__ out_indices, float* __restrict__ lse_out) {
  const int head = blockIdx.x, row = blockIdx.y, d = threadIdx.x;
  const int64_t idx = (int64_t)row * heads_q + head;
  // the first kAhead splits' LSEs and outputs are fetched side by side before anything is
  // computed (one round trip instead of two); the arithmetic and its order do not change
  constexpr int kAhead = 8;
  float ls_ahead[kAhead], o_ahead[kAhead];
  const bool ahead = lse_ptrs == nullptr && o_ptrs == nullptr;
#pragma unroll
  for (int s = 0; s < kAhead; ++s) {
    const bool live = ahead && s < num_splits;
    ls_ahead[s] = live ? lse_parts[s * lse_split_stride + idx] : -INFINITY;
    o_ahead[s] = live ? o_parts[s * o_split_stride + idx * kHeadDim + d] : 0.f;
  }
  const int from = ahead ? (num_splits < kAhead ? num_splits : kAhead) : 0;
  float mx = -INFINITY;
#pragma unroll
  for (int s = 0; s < kAhead; ++s) mx = fmaxf(mx, ls_ahead[s]);
  for (int s = from; s < num_splits; ++s) {
    const float* lp = lse_ptrs ? lse_ptrs[s] : lse_parts + s * lse_split_stride;
    mx = fmaxf(mx, lp[idx]);
  }
  float acc = 0.f, tot = 0.f;
  if (mx != -INFINITY) {
#pragma unroll
    for (int s = 0; s < kAhead; ++s) {
      if (s >= from || ls_ahead[s] == -INFINITY) continue;  // an empty split weighs nothing, whatever its O holds
      const float wgt = expf(ls_ahead[s] - mx);
      tot += wgt;
      acc = fmaf(wgt, o_ahead[s], acc);
    }
    for (int s = from; s < num_splits; ++s) {
      const float* lp = lse_ptrs ? lse_ptrs[s] : lse_parts + s * lse_split_stride;
      const float* op = o_ptrs ? o_ptrs[s] : o_parts + s * o_split_stride;
      const float ls = lp[idx];
      if (ls == -INFINITY) continue;
      const float wgt = expf(ls - mx);
      tot += wgt;
      acc = fmaf(wgt, op[idx * kHeadDim + d], acc);
    }
  }
  const float val = tot > 0.f ? __fdiv_rn(acc, tot) : 0.f;
  if (out) {
    const int64_t orow = out_indices ? (int64_t)out_indices[row] : (int64_t)row;
    const int64_t at = (orow * heads_q + head) * kHeadDim + d;
    if (kOutF32) static_cast<float*>(out)[at] = val;
    else static_cast<uint16_t*>(out)[at] = __bfloat16_as_ushort(__float2bfloat16_rn(val));
  }
  if (lse_out && d == 0) lse_out[idx] = tot > 0.f ? mx + logf(tot) : -INFINITY;
}

cudaError_t launch_lse_merge(const float* o_parts, int64_t o_split_stride, const float* lse_parts,
                             int64_t lse_split_stride, const float* const* o_ptrs,
                             const float* const* lse_ptrs, int num_splits, int rows, int heads_q,
                             void* out, int out_is_f32, const int32_t* out_indices,
                             float* lse_out, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  dim3 grid(heads_q, rows);
  if (out_is_f32)
    lse_merge_kernel<true><<<grid, 128, 0, stream>>>(o_parts, o_split_stride, lse_parts,
                                                     lse_split_stride, o_ptrs, lse_ptrs, num_splits,
                                                     rows, heads_q, out, out_indices, lse_out);
  else
    lse_merge_kernel<false><<<grid, 128, 0, stream>>>(o_parts, o_split_stride, lse_parts,
                                                      lse_split_stride, o_ptrs, lse_ptrs, num_splits,
                                                      rows, heads_q, out, out_indices, lse_out);
  return cudaGetLastError();
}

}  // namespace nvfp4

// ---------------------------------------------------------------------------
// Cross-GPU merge for the KV page-range split: every rank has written its partial
// (normalised O, LSE) into a buffer that all ranks can address.  One launch per
// rank: announce "my partial of this epoch is written" in every peer's flag array,
// wait (bounded) until every peer has announced the same, then merge with plain loads
// from the peers' buffers.  The kernels of the ranks run on different GPUs.
// ---------------------------------------------------------------------------
namespace nvfp4 {



template <bool kOutF32>
__global__ void __launch_bounds__(128)
peer_merge_kernel(const float* const* __restrict__ o_ptrs, const float* const* __restrict__ lse_ptrs,
                  int* const* __restrict__ flag_ptrs, int rank, int world, int epoch_arg,
                  int* __restrict__ epoch_state, int rows, int heads_q, void* __restrict__ out,
                  uint32_t* __restrict__ status) {
  __shared__ int ready;
  const int head = blockIdx.x, row = blockIdx.y, d = threadIdx.x;
  // With a device-resident epoch (graph replay) every block reads it before any block can
  // advance it: the block that finishes last does that.
  const int epoch = epoch_state ? *reinterpret_cast<volatile int*>(epoch_state) + 1 : epoch_arg;
  if (blockIdx.x == 0 && blockIdx.y == 0 && d < world) {
    __threadfence_system();
    st_release_sys(flag_ptrs[d] + rank, epoch);
  }
  if (d == 0) {
    const int* mine = flag_ptrs[rank];
    unsigned long long t0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    int ok = 1;
    for (int w = 0; w < world && ok; ++w) {
      // epochs only grow; a peer that is already a step ahead has certainly written this one
      while (ld_acquire_sys(mine + w) - epoch < 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        if (t - t0 > kPeerWaitNs) { ok = 0; break; }
        __nanosleep(64);
      }
    }
    if (!ok) set_status(status, NVFP4_STATUS_WAIT_TIMEOUT);
    ready = ok;
  }
  __syncthreads();
  if (epoch_state && d == 0) {
    const int blocks = gridDim.x * gridDim.y;
    if (atomicAdd(epoch_state + 1, 1) == blocks - 1) {
      epoch_state[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(epoch_state) = epoch;
    }
  }
  if (!ready) return;  // the output is left untouched and the status word says why
  const int64_t idx = (int64_t)row * heads_q + head;
  float mx = -INFINITY;
  for (int s = 0; s < world; ++s) mx = fmaxf(mx, ld_relaxed_sys(lse_ptrs[s] + idx));
  float acc = 0.f, tot = 0.f;
  if (mx != -INFINITY) {
    for (int s = 0; s < world; ++s) {
      const float ls = ld_relaxed_sys(lse_ptrs[s] + idx);
      if (ls == -INFINITY) continue;
      const float wgt = expf(ls - mx);
      tot += wgt;
      acc = fmaf(wgt, ld_relaxed_sys(o_ptrs[s] + idx * kHeadDim + d), acc);
    }
  }
  const float val = tot > 0.f ? __fdiv_rn(acc, tot) : 0.f;
  const int64_t at = idx * kHeadDim + d;
  if (kOutF32) static_cast<float*>(out)[at] = val;
  else static_cast<uint16_t*>(out)[at] = __bfloat16_as_ushort(__float2bfloat16_rn(val));
}

cudaError_t launch_peer_merge(const float* const* o_ptrs, const float* const* lse_ptrs,
                              int* const* flag_ptrs, int rank, int world, int epoch,
                              int* epoch_state, int rows, int heads_q, void* out, int out_is_f32,
                              uint32_t* status, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  dim3 grid(heads_q, rows);
  if (out_is_f32)
    peer_merge_kernel<true><<<grid, 128, 0, stream>>>(o_ptrs, lse_ptrs, flag_ptrs, rank, world, epoch,
                                                      epoch_state, rows, heads_q, out, status);
  else
    peer_merge_kernel<false><<<grid, 128, 0, stream>>>(o_ptrs, lse_ptrs, flag_ptrs, rank, world, epoch,
                                                       epoch_state, rows, heads_q, out, status);
  return cudaGetLastError();
}

}  // namespace nvfp4

// ---------------------------------------------------------------------------
// Push exchange for the KV page-range split, ONE launch per rank after the decode:
// the CTA of (query head, row) folds this rank's local split partials, stores the result
// into the matching slot of every peer's inbox (posted remote stores, nothing is loaded over
// NVLink), announces it per (head, row), waits (bounded) for the peers' announcements of the
// same (head, row) only, and merges out of its own memory.  CTAs of different (head, row) never
// wait for one another, so a late rank delays only the pairs it has not pushed yet.
//   inbox of a rank : float [2 copies][world sources][rows * heads_q][kInboxStride]
//                     (128 channels of normalised O, then the LSE); copies alternate by epoch
//   flags of a rank : int   [world sources][rows * heads_q], the epoch of the latest push
// ---------------------------------------------------------------------------
namespace nvfp4 {



template <bool kOutF32>
__global__ void __launch_bounds__(128)
push_merge_kernel(const float* __restrict__ o_local, int64_t o_split_stride,
                  const float* __restrict__ lse_local, int64_t lse_split_stride, int local_splits,
                  float* const* __restrict__ inbox_ptrs, int* const* __restrict__ flag_ptrs, int rank,
                  int world, int epoch_arg, int* __restrict__ epoch_state, int rows, int heads_q,
                  void* __restrict__ out, uint32_t* __restrict__ status) {
  __shared__ int ready;
  const int head = blockIdx.x, row = blockIdx.y, d = threadIdx.x;
  const int64_t idx = (int64_t)row * heads_q + head;
  const int64_t pairs = (int64_t)rows * heads_q;
  // With a device-resident epoch (graph replay) every block reads it before any block can
  // advance it: the block that finishes last does that.
  const int epoch = epoch_state ? *reinterpret_cast<volatile int*>(epoch_state) + 1 : epoch_arg;
  if (d == 0) ready = 1;

  // fold this rank's local splits (index order, the arithmetic of lse_merge_kernel)
  float mx = -INFINITY;
  for (int s = 0; s < local_splits; ++s) mx = fmaxf(mx, lse_local[s * lse_split_stride + idx]);
  float acc = 0.f, tot = 0.f;
  if (mx != -INFINITY) {
    for (int s = 0; s < local_splits; ++s) {
      const float ls = lse_local[s * lse_split_stride + idx];
      if (ls == -INFINITY) continue;
      const float wgt = expf(ls - mx);
      tot += wgt;
      acc = fmaf(wgt, o_local[s * o_split_stride + idx * kHeadDim + d], acc);
    }
  }
  const float my_o = tot > 0.f ? __fdiv_rn(acc, tot) : 0.f;
  const float my_lse = tot > 0.f ? mx + logf(tot) : -INFINITY;

  // push to every peer's inbox, then announce
  const int64_t copy_elems = (int64_t)world * pairs * kInboxStride;
  const int64_t slot = ((epoch & 1) * copy_elems) + ((int64_t)rank * pairs + idx) * kInboxStride;
  for (int w = 0; w < world; ++w) {
    if (w == rank) continue;
    float* dst = inbox_ptrs[w] + slot;
    st_relaxed_sys(dst + d, my_o);
    if (d == 0) st_relaxed_sys(dst + kHeadDim, my_lse);
  }
  __threadfence_system();
  __syncthreads();
  if (d < world && d != rank) st_release_sys(flag_ptrs[d] + (int64_t)rank * pairs + idx, epoch);

  // wait for the peers' pushes of this (head, row): thread w watches source w
  if (d < world && d != rank) {
    const int* flag = flag_ptrs[rank] + (int64_t)d * pairs + idx;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    // epochs only grow; a peer that is already a step ahead has certainly pushed this one
    while (ld_acquire_sys(flag) - epoch < 0) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
      if (t - t0 > kPeerWaitNs) {
        set_status(status, NVFP4_STATUS_WAIT_TIMEOUT);
        ready = 0;
        break;
      }
      __nanosleep(32);
    }
  }
  __syncthreads();
  if (epoch_state && d == 0) {
    const int blocks = gridDim.x * gridDim.y;
    if (atomicAdd(epoch_state + 1, 1) == blocks - 1) {
      epoch_state[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(epoch_state) = epoch;
    }
  }
  if (!ready) return;  // the output is left untouched and the status word says why

  // merge in source order (identical on every rank), own partial out of registers
  const float* mine = inbox_ptrs[rank] + (epoch & 1) * copy_elems;
  float gm = -INFINITY;
  for (int s = 0; s < world; ++s)
    gm = fmaxf(gm, s == rank ? my_lse : ld_relaxed_sys(mine + ((int64_t)s * pairs + idx) * kInboxStride + kHeadDim));
  float a2 = 0.f, t2 = 0.f;
  if (gm != -INFINITY) {
    for (int s = 0; s < world; ++s) {
      const float* src = mine + ((int64_t)s * pairs + idx) * kInboxStride;
      const float ls = s == rank ? my_lse : ld_relaxed_sys(src + kHeadDim);
      if (ls == -INFINITY) continue;
      const float wgt = expf(ls - gm);
      t2 += wgt;
      a2 = fmaf(wgt, s == rank ? my_o : ld_relaxed_sys(src + d), a2);
    }
  }
  const float val = t2 > 0.f ? __fdiv_rn(a2, t2) : 0.f;
  const int64_t at = idx * kHeadDim + d;
  if (kOutF32) static_cast<float*>(out)[at] = val;
  else static_cast<uint16_t*>(out)[at] = __bfloat16_as_ushort(__float2bfloat16_rn(val));
}

cudaError_t launch_push_merge(const float* o_local, int64_t o_split_stride, const float* lse_local,
                              int64_t lse_split_stride, int local_splits, float* const* inbox_ptrs,
                              int* const* flag_ptrs, int rank, int world, int epoch, int* epoch_state,
                              int rows, int heads_q, void* out, int out_is_f32, uint32_t* status,
                              cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  dim3 grid(heads_q, rows);
  if (out_is_f32)
    push_merge_kernel<true><<<grid, 128, 0, stream>>>(o_local, o_split_stride, lse_local, lse_split_stride,
                                                      local_splits, inbox_ptrs, flag_ptrs, rank, world, epoch,
                                                      epoch_state, rows, heads_q, out, status);
  else
    push_merge_kernel<false><<<grid, 128, 0, stream>>>(o_local, o_split_stride, lse_local, lse_split_stride,
                                                       local_splits, inbox_ptrs, flag_ptrs, rank, world, epoch,
                                                       epoch_state, rows, heads_q, out, status);
  return cudaGetLastError();
}

}  // namespace nvfp4

// ---------------------------------------------------------------------------
// Balanced split: every row gets its own split count, ceil(pages / target_pages) (at least
// one), so that each CTA walks about target_pages pages however ragged the batch is.
// ---------------------------------------------------------------------------
namespace nvfp4 {

// One CTA.  A row's FP4 pages are cut into ceil(pages / target_pages) pieces; a row that holds a
// BF16 tail gets one more piece for the tail alone (entry.w = 1), which the decode kernel serves
// with a path of its own that stages the tail in shared memory - so the tail is never walked in
// front of a piece's page stream.  A row with neither pages nor a tail keeps one (empty) piece.
// A row's pieces sit side by side, the tail piece first.  The rows are listed by the length of
// their pieces, longest first (sixteen size classes; within a class in no particular order - a
// row's result does not depend on where its pieces sit),
// because the CTAs of the decode grid start in list order and the last ones to start should be
// the short ones.  Entries past the end get row -1.
__global__ void __launch_bounds__(1024)
balanced_worklist_kernel(const int32_t* __restrict__ seqused_fp4, const int32_t* __restrict__ seqused_tail,
                         int rows, int max_pages, int target_pages, int4* __restrict__ work, int capacity,
                         int32_t* __restrict__ row_offset, int32_t* __restrict__ row_count,
                         int32_t* __restrict__ counters, int counter_words, uint32_t* __restrict__ status) {
  __shared__ int class_total[kSizeClasses], class_cursor[kSizeClasses];
  __shared__ int used;
  const int tid = threadIdx.x;
  if (tid < kSizeClasses) class_total[tid] = 0;
  __syncthreads();
  for (int row = tid; row < rows; row += 1024) {
    int count, size_class;
    const int tail = seqused_tail != nullptr && seqused_tail[row] > 0 ? 1 : 0;
    balanced_pieces_of_row(seqused_fp4[row], tail, max_pages, target_pages, count, size_class);
    // a row's partials sit side by side: its tail piece is counted with its page pieces
    atomicAdd(&class_total[size_class], count + tail);
  }
  __syncthreads();
  if (tid == 0) {
    int at = 0;
    for (int c = 0; c < kSizeClasses; ++c) { class_cursor[c] = at; at += class_total[c]; }
    used = at;
  }
  __syncthreads();
  for (int row = tid; row < rows; row += 1024) {
    int count, size_class;
    const int tail = seqused_tail != nullptr && seqused_tail[row] > 0 ? 1 : 0;
    balanced_pieces_of_row(seqused_fp4[row], tail, max_pages, target_pages, count, size_class);
    const int first = atomicAdd(&class_cursor[size_class], count + tail);
    row_offset[row] = first;
    row_count[row] = count + tail;
    if (!balanced_write_row(work, capacity, first, row, count, tail)) set_status(status, NVFP4_STATUS_BAD_LENGTH);
  }
  for (int w = used + tid; w < capacity; w += 1024) work[w] = make_int4(-1, 0, 0, 0);
  if (counters != nullptr)
    for (int w = tid; w < counter_words; w += 1024) counters[w] = 0;
}

// LSE merge where row r's partials are slots [row_offset[r], row_offset[r] + row_count[r]).
// The launch is a chain of round trips to memory (the row's range, the pieces' LSEs, their
// outputs), so the first kMergeAhead pieces' LSEs AND outputs are fetched side by side before
// anything is computed; the arithmetic and its order are those of lse_merge_kernel.
constexpr int kMergeAhead = 8;
__global__ void __launch_bounds__(128)
lse_merge_ranges_kernel(const float* __restrict__ o_parts, const float* __restrict__ lse_parts,
                        const int32_t* __restrict__ row_offset, const int32_t* __restrict__ row_count,
                        int heads_q, uint16_t* __restrict__ out) {
  const int head = blockIdx.x, row = blockIdx.y, d = threadIdx.x;
  const int first = row_offset[row], count = row_count[row];
  float ls_ahead[kMergeAhead], o_ahead[kMergeAhead];
#pragma unroll
  for (int s = 0; s < kMergeAhead; ++s) {
    const int64_t idx = (int64_t)(first + (s < count ? s : 0)) * heads_q + head;
    ls_ahead[s] = s < count ? lse_parts[idx] : -INFINITY;
    o_ahead[s] = s < count ? o_parts[idx * kHeadDim + d] : 0.f;
  }
  float mx = -INFINITY;
#pragma unroll
  for (int s = 0; s < kMergeAhead; ++s) mx = fmaxf(mx, ls_ahead[s]);
  for (int s = kMergeAhead; s < count; ++s) mx = fmaxf(mx, lse_parts[(int64_t)(first + s) * heads_q + head]);
  float acc = 0.f, tot = 0.f;
  if (mx != -INFINITY) {
#pragma unroll
    for (int s = 0; s < kMergeAhead; ++s) {
      if (s >= count || ls_ahead[s] == -INFINITY) continue;
      const float wgt = expf(ls_ahead[s] - mx);
      tot += wgt;
      acc = fmaf(wgt, o_ahead[s], acc);
    }
    for (int s = kMergeAhead; s < count; ++s) {
      const int64_t idx = (int64_t)(first + s) * heads_q + head;
      const float ls = lse_parts[idx];
      if (ls == -INFINITY) continue;
      const float wgt = expf(ls - mx);
      tot += wgt;
      acc = fmaf(wgt, o_parts[idx * kHeadDim + d], acc);
    }
  }
  const float val = tot > 0.f ? __fdiv_rn(acc, tot) : 0.f;
  out[((int64_t)row * heads_q + head) * kHeadDim + d] = __bfloat16_as_ushort(__float2bfloat16_rn(val));
}

cudaError_t launch_balanced_worklist(const int32_t* seqused_fp4, const int32_t* seqused_tail, int rows,
                                     int max_pages, int target_pages, int4* work, int capacity,
                                     int32_t* row_offset, int32_t* row_count, int32_t* counters,
                                     int counter_words, uint32_t* status, cudaStream_t stream) {
  balanced_worklist_kernel<<<1, 1024, 0, stream>>>(seqused_fp4, seqused_tail, rows, max_pages, target_pages, work,
                                                   capacity, row_offset, row_count, counters, counter_words,
                                                   status);
  return cudaGetLastError();
}

cudaError_t launch_lse_merge_ranges(const float* o_parts, const float* lse_parts, const int32_t* row_offset,
                                    const int32_t* row_count, int rows, int heads_q, void* out,
                                    cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  dim3 grid(heads_q, rows);
  lse_merge_ranges_kernel<<<grid, 128, 0, stream>>>(o_parts, lse_parts, row_offset, row_count, heads_q,
                                                    static_cast<uint16_t*>(out));
  return cudaGetLastError();
}

}  // namespace nvfp4
