// Piece arithmetic of the balanced split, shared by the stand-alone list builder and the slot
// control step (which can build the list of its own step in the same launch).
#pragma once

namespace nvfp4 {

// The rows are listed by the length of their pieces, longest first, in sixteen size classes.
constexpr int kSizeClasses = 16;

// A row of `fp4_tokens` quantised tokens (a multiple of 128; out-of-range values are clamped here
// and reported by the decode kernel) that holds a BF16 tail or not: how many page pieces it
// gets (one empty piece if it has neither pages nor a tail) and the size class of its longest.
__device__ __forceinline__ void balanced_pieces_of_row(int fp4_tokens, int has_tail, int max_pages,
                                                       int target_pages, int& count, int& size_class) {
  int n = fp4_tokens >> 7;
  if (fp4_tokens < 0 || n > max_pages) n = fp4_tokens < 0 ? 0 : max_pages;
  count = n > 0 ? (n + target_pages - 1) / target_pages : 1 - has_tail;
  const int piece = count > 0 ? (n + count - 1) / count : 0;   // pages of the row's longest piece
  size_class = kSizeClasses - 1 - min(kSizeClasses - 1, piece * kSizeClasses / (target_pages + 1));
}

// The entries of one row, starting at list index `first`: the tail piece first (it is the
// quickest to finish), then the page pieces.
__device__ __forceinline__ bool balanced_write_row(int4* work, int capacity, int first, int row, int count,
                                                   int tail) {
  bool fits = true;
  for (int s = 0; s < count + tail; ++s) {
    const int4 entry = s < tail ? make_int4(row, 0, 1, 1) : make_int4(row, s - tail, count, 0);
    if (first + s < capacity) work[first + s] = entry;
    else fits = false;   // cannot happen with the documented capacity
  }
  return fits;
}

}  // namespace nvfp4
