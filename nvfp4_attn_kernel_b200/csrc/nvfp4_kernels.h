// Internal launcher declarations shared by the .cu translation units and the C ABI.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace nvfp4 {

cudaError_t launch_quantize_q(const void* q, int64_t row_stride, int64_t head_stride,
                              const int32_t* row_indices, void* q_fp4, void* q_sf, void* q_padded,
                              int rows, int heads_q, int heads_kv, cudaStream_t stream);

cudaError_t launch_quantize_k(const void* tokens, int64_t token_stride, const void* key_shift,
                              void* packed, int64_t packed_pitch, void* sf, int64_t sf_pitch,
                              const int32_t* src_tokens, const int32_t* dst_pages,
                              const int64_t* packed_bases, const int64_t* sf_bases, int work,
                              int layers, int64_t src_layer_stride, int heads_kv,
                              cudaStream_t stream);

cudaError_t launch_quantize_v(const void* tokens, int64_t token_stride, void* packed,
                              int64_t packed_pitch, void* sf, int64_t sf_pitch,
                              const int32_t* src_tokens, const int32_t* dst_pages,
                              const int64_t* packed_bases, const int64_t* sf_bases, int work,
                              int layers, int64_t src_layer_stride, int heads_kv,
                              cudaStream_t stream);

cudaError_t launch_tail_append(const void* key, const void* value, int64_t key_token_stride,
                               int64_t value_token_stride, const void* key_shift, void* tail_key,
                               void* tail_value, int64_t tail_slot_stride,
                               const int32_t* query_start_loc, const int32_t* seq_lens,
                               const int32_t* seqused_fp4, const int32_t* row_to_slot,
                               int num_tokens, int num_reqs, int heads_kv, cudaStream_t stream);

cudaError_t launch_write_kv(const void* key, const void* value, int64_t key_token_stride,
                            int64_t value_token_stride, const void* key_shift, void* k_packed,
                            int64_t k_pitch, void* k_sf, int64_t k_sf_pitch, void* v_packed,
                            int64_t v_pitch, void* v_sf, int64_t v_sf_pitch, const int32_t* src_tokens,
                            const int32_t* dst_pages, int work, void* tail_key, void* tail_value,
                            int64_t tail_slot_stride, const int32_t* query_start_loc,
                            const int32_t* seq_lens, const int32_t* seqused_fp4,
                            const int32_t* row_to_slot, int num_tokens, int num_reqs, int heads_kv,
                            cudaStream_t stream);

cudaError_t launch_tail_reset(void* tail_key, void* tail_value, int64_t layer_stride,
                              int64_t slot_stride, int layers, const int32_t* query_start_loc,
                              const int32_t* seq_lens, const int32_t* row_to_slot, int num_reqs,
                              int heads_kv, cudaStream_t stream);

cudaError_t launch_tail_flush(const void* tail_key, const void* tail_value,
                              int64_t src_layer_stride, const int32_t* src_tokens,
                              const int32_t* dst_pages, const int64_t* bases, int64_t k_pitch,
                              int64_t k_sf_pitch, int64_t v_pitch, int64_t v_sf_pitch, int work,
                              int layers, int heads_kv, cudaStream_t stream);

// Everything a decode kernel needs, by value.
struct DecodeParams {
  const uint8_t* q_fp4;
  const uint8_t* q_sf;
  const uint16_t* q_bf16;  // nullable
  int64_t q_row_stride, q_head_stride;
  const uint8_t* k_packed; int64_t k_pitch;
  const uint8_t* k_sf; int64_t k_sf_pitch;
  const uint8_t* v_packed; int64_t v_pitch;
  const uint8_t* v_sf; int64_t v_sf_pitch;
  int64_t num_pages;
  const int32_t* page_table; int64_t page_table_row_stride; int max_pages;
  const int32_t* seqused_fp4;
  const uint16_t* tail_key; const uint16_t* tail_value; int64_t tail_pages;
  const int32_t* tail_ids; const int32_t* seqused_tail;
  uint16_t* out; const int32_t* out_indices;  // bf16 out (only when num_splits == 1)
  float* o_partial; float* lse_partial;       // partial outputs (when emit_partial)
  int rows, heads_q, heads_kv;
  float scale_log2;  // softmax_scale * log2(e)
  int num_splits;
  int emit_partial;  // 1: write (O normalised fp32, LSE) per split; 0: write bf16 out
  uint32_t* status;
  // Cross-GPU page-range exchange done by the decode kernel itself (xchg_inbox null: off).
  // The CTA that completes a (row, KV head) tile last folds its splits, pushes the result into
  // every peer's inbox, waits for the peers' pushes of the same tile and writes the merged rows.
  float* const* xchg_inbox;   // device array [world]: each rank's inbox, see nvfp4_push_merge
  int* const* xchg_flags;     // device array [world]: each rank's flags
  int* xchg_epoch_state;      // two device ints, zero-filled once: the epoch, finished tiles
  int* xchg_counters;         // device ints [rows * heads_kv], zero-filled once: arrivals per tile
  void* xchg_out;             // [rows][heads_q][128] bf16 or fp32
  int xchg_out_f32, xchg_rank, xchg_world;
  int pdl;                    // 1: launched with programmatic stream serialization (tensor-core kernel)
  // The step's own K/V token of every row (decode rows bring exactly one), null: the tail was
  // appended beforehand.  The CTA that owns a row's tail stores the token at tail position
  // seqused_tail - 1 (key shifted) and uses it from the source.
  const uint16_t* append_key; const uint16_t* append_value;   // bf16 [rows][heads_kv][128], token strides below
  int64_t append_key_stride, append_value_stride;             // elements
  const uint16_t* key_shift;                                   // nullable bf16 [heads_kv][128]
  // Work list of the balanced split (null: the grid is (splits, heads_kv, rows)).  Entry w =
  // {row, split, splits of that row, unused}, row -1 = no work; the grid is (entries, heads_kv)
  // and entry w stores its partial in slot w.
  const int4* work_list;
  int work_capacity;
  // With a work list the row's pieces can be merged inside the launch (list_counters non-null):
  // the piece of a (row, KV head) that arrives last - arrival counters, [rows][heads_kv] ints that
  // the list builder zeroes and the last arrival leaves at zero - folds the row's partials, slots
  // list_row_offset[row] .. + list_row_count[row], into `out` with the arithmetic of the merge launch.
  const int32_t* list_row_offset; const int32_t* list_row_count; int* list_counters;
  // Persistent kernel: launch counter and leaving CTAs of the scratch slots.
  int* tile_counters;
  int wide_hint;              // 1: the caller expects at most one busy CTA per SM
};

// CUDA-core kernel: any G = Hq/Hkv in {1,2,4,8,16,32}.
cudaError_t launch_decode_generic(const DecodeParams& p, cudaStream_t stream);

// tcgen05 kernel: G in {1, 2, 4, 8, 16, 32}.  Returns cudaErrorNotSupported when the shape is outside it.
cudaError_t launch_decode_sm100(const DecodeParams& p, cudaStream_t stream);
bool decode_sm100_supports(const DecodeParams& p);

// Persistent tcgen05 kernel (one launch, equal shares of page tiles per resident CTA, pieces of a
// tile merged by the piece that arrives last): G in {1, 2, 4, 8}, final BF16 output only.
// workspace: decode_persistent_workspace_bytes() bytes whose first rows * heads_kv ints were
// zero-filled once.
cudaError_t launch_decode_persistent(const DecodeParams& p, void* workspace, cudaStream_t stream);
bool decode_persistent_supports(const DecodeParams& p);
size_t decode_persistent_workspace_bytes(int rows, int heads_q, int heads_kv);
int decode_persistent_ctas();

cudaError_t launch_lse_merge(const float* o_parts, int64_t o_split_stride, const float* lse_parts,
                             int64_t lse_split_stride, const float* const* o_ptrs,
                             const float* const* lse_ptrs, int num_splits, int rows, int heads_q,
                             void* out, int out_is_f32, const int32_t* out_indices,
                             float* lse_out, cudaStream_t stream);

// Slot control plane (one CTA) and the page work table.
struct ControlArgs {
  const int32_t* block_table; int64_t block_table_stride; int block_table_columns;
  const int32_t* seq_lens; const int32_t* query_start_loc;
  int32_t* slot_keys; int32_t* slot_last_seq; int64_t* slot_last_seen; int64_t* step;
  int32_t* row_to_slot; int32_t* token_to_slot; int32_t* seqused_fp4; int32_t* seqused_residual;
  int32_t* promotion_source_tokens; int32_t* promotion_pages; int32_t* error_code;
  int num_reqs, num_actual_tokens, num_slots;
  // optional (work null: off): the balanced split's list of pieces for the first work_rows rows
  // of this step, built from the lengths this launch computes (see launch_balanced_worklist)
  int4* work; int32_t* work_row_offset; int32_t* work_row_count; int32_t* work_counters; int work_counter_words;
  int work_rows, work_capacity, work_max_pages, work_target_pages;
};

cudaError_t launch_control(const ControlArgs& a, cudaStream_t stream);
cudaError_t launch_work_table(const int32_t* query_start_loc, const int32_t* seqused_fp4,
                              const int32_t* row_to_slot, const int32_t* block_table,
                              int64_t block_table_stride, int32_t* source_tokens,
                              int32_t* destination_pages, int num_reqs, int columns_per_row,
                              cudaStream_t stream);

// Balanced split: row r gets ceil(pages / target_pages) pieces of pages plus, when seqused_tail
// (nullable) says it holds a BF16 tail, one piece for the tail alone; at least one piece.
// work [capacity] entries (row, piece, page pieces of the row, 1 for the tail piece), row_offset /
// row_count [rows]: first partial slot and piece count of a row.
// counters (nullable): `counter_words` ints zeroed for the in-launch merge of the pieces.
cudaError_t launch_balanced_worklist(const int32_t* seqused_fp4, const int32_t* seqused_tail, int rows,
                                     int max_pages, int target_pages, int4* work, int capacity,
                                     int32_t* row_offset, int32_t* row_count, int32_t* counters,
                                     int counter_words, uint32_t* status, cudaStream_t stream);
cudaError_t launch_lse_merge_ranges(const float* o_parts, const float* lse_parts, const int32_t* row_offset,
                                    const int32_t* row_count, int rows, int heads_q, void* out,
                                    cudaStream_t stream);

cudaError_t launch_peer_merge(const float* const* o_ptrs, const float* const* lse_ptrs,
                              int* const* flag_ptrs, int rank, int world, int epoch,
                              int* epoch_state, int rows, int heads_q, void* out, int out_is_f32,
                              uint32_t* status, cudaStream_t stream);

cudaError_t launch_push_merge(const float* o_local, int64_t o_split_stride, const float* lse_local,
                              int64_t lse_split_stride, int local_splits, float* const* inbox_ptrs,
                              int* const* flag_ptrs, int rank, int world, int epoch, int* epoch_state,
                              int rows, int heads_q, void* out, int out_is_f32, uint32_t* status,
                              cudaStream_t stream);

// sum[c] += the fp64 sum over tokens of key[t][c] (c over heads_kv * 128 channels).
cudaError_t launch_key_sum(const void* key, int64_t token_stride, int tokens, int heads_kv, double* sum,
                           cudaStream_t stream);

}  // namespace nvfp4
