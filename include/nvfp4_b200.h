/*
 * nvfp4_b200 — C ABI of the B200 (sm_100a) paged NVFP4/BF16 hybrid decode-attention path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t).  Nothing here allocates device
 * memory unless stated, nothing synchronises the stream, and every call is
 * safe to record into a CUDA graph unless stated.  All functions return 0 on
 * success and a non-zero code on failure; nvfp4_last_error() then holds a
 * human-readable message for the calling thread.
 *
 * Formats (identical to the reference project, so buffers are interchangeable):
 *   E2M1  : 4-bit float, two per byte, even element in the LOW nibble.
 *   scale : E4M3 byte per 16 elements, value = e2m1 * e4m3, no second-level scale.
 *   K page: packed [page][128 tok][Hkv][64 B]; scales, per page and head, one
 *           1024-byte block: byte (g/4)*512 + (tok%32)*16 + (tok/32)*4 + g%4
 *           for 16-channel group g of token tok.
 *   V page: packed [page][Hkv][128 ch][64 B] (byte j of a channel row = tokens
 *           2j, 2j+1); groups run along TOKENS; scale block as for K with the
 *           channel in place of the token and the 16-token group in place of g.
 *   Q     : packed [rows][1][Hq][64 B]; scales [rows][Hq*1024 B], head h of KV
 *           head kv=h/G, slot r=h%G: byte kv*1024 + (g/4)*512 + (r%32)*16 +
 *           (r/32)*4 + g%4; the unwritten slots must be zero.
 * Page pitches are free (>= dense size, 16-byte aligned; scale pitches 16-byte
 * aligned), so the four regions may be carved out of one vLLM block.
 *
 * Citations "ref:" name the file:line of the reference project interface that
 * the entry point stands in for.
 */
#ifndef NVFP4_B200_H_
#define NVFP4_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NVFP4_PAGE_SIZE 128
#define NVFP4_HEAD_DIM 128

/* error codes */
#define NVFP4_OK 0
#define NVFP4_ERR_INVALID 1     /* bad argument (message says which) */
#define NVFP4_ERR_CUDA 2        /* a CUDA runtime/driver call failed */
#define NVFP4_ERR_UNSUPPORTED 3 /* shape or device outside what the kernels cover */

/* bits of the sticky device status word (nvfp4_decode_args.status) */
#define NVFP4_STATUS_BAD_PAGE_ID 1u   /* a consumed page-table entry was outside [0, num_pages) */
#define NVFP4_STATUS_BAD_TAIL_ID 2u   /* tail length > 0 with a tail id outside [0, tail_pages) */
#define NVFP4_STATUS_WAIT_TIMEOUT 4u  /* a bounded device-side wait gave up */
#define NVFP4_STATUS_BAD_LENGTH 8u    /* seqused_fp4 not a multiple of 128 / beyond the table, tail length > 128 */

/* decode implementations */
#define NVFP4_IMPL_AUTO 0
#define NVFP4_IMPL_GENERIC 1 /* CUDA-core kernel, any G = Hq/Hkv in {1,2,4,8,16,32} */
#define NVFP4_IMPL_SM100 2   /* tcgen05 block-scaled MMA kernel, G in {1, 2, 4, 8, 16, 32} */

const char* nvfp4_last_error(void);
int nvfp4_version(void);

/* 1 if the CUDA device can run the kernels (compute capability 10.x), 0 if not,
 * negative on a CUDA error. */
int nvfp4_device_supported(int device);

/*
 * Q quantiser.  ref: quantize_query, src/nvfp4_decode_kernel/_quantize.py:14-117 and
 * quantize_decode_q_to_padded_fp4, quantize_q_kernel.py:304-505.
 *   q_bf16      [src_rows][Hq][128] bf16, strides in ELEMENTS, last stride 1
 *   row_indices nullable int32[rows]: compact row i reads source row row_indices[i]
 *   q_fp4       out, [rows][1][Hq][64] bytes, every byte rewritten
 *   q_sf        out, [rows][Hq*1024] bytes; only the G=Hq/Hkv live slots of each
 *               KV head are written (the caller zeroes the buffer once)
 *   q_padded    nullable out, bf16 [>=rows][128][Hq][128]; only [row][0][h][:] is written
 */
int nvfp4_quantize_q(const void* q_bf16, int64_t q_row_stride, int64_t q_head_stride,
                     const int32_t* row_indices, void* q_fp4, void* q_sf, void* q_padded,
                     int rows, int heads_q, int heads_kv, void* stream);

/*
 * K / V page quantiser, dense or indexed, optional per-layer destinations and an
 * optional fused per-channel key shift.
 * ref: quantize_key_pages / quantize_value_pages / quantize_key_tokens_into /
 * quantize_value_tokens_into, quantize_kv_kernel.py:661-822; shift: nvfp4_vllm/impl.py:145-152.
 *   which          0 = K, 1 = V
 *   tokens_bf16    flat [tokens][Hkv][128] bf16, dense inside a token; token_stride in elements
 *   key_shift_bf16 nullable bf16 [layers][Hkv][128] (K only): k <- bf16(k - shift) before quantising
 *   packed/sf      destination regions with page pitches in BYTES
 *   src_tokens     nullable int32[work]: first token of work item w (default w*128)
 *   dst_pages      nullable int32[work]: destination page of w (default w); negative = skip
 *   packed_bases / sf_bases  nullable int64[layers]: per-layer destination base addresses
 *                  (then packed/sf only fix the layout and may be NULL)
 *   src_layer_stride tokens between consecutive layers of the source
 */
int nvfp4_quantize_kv_pages(int which, const void* tokens_bf16, int64_t token_stride,
                            const void* key_shift_bf16, void* packed, int64_t packed_pitch,
                            void* sf, int64_t sf_pitch, const int32_t* src_tokens,
                            const int32_t* dst_pages, const int64_t* packed_bases,
                            const int64_t* sf_bases, int work, int layers,
                            int64_t src_layer_stride, int heads_kv, void* stream);

/*
 * BF16 tail append for one layer (with the key shift fused).
 * ref: write_kv / _tail_write_kernel, src/nvfp4_vllm/write.py:79-130,280-337.
 * Token t of row r lands at tail[slot(r)][seq_len[r] + t - row_end[r] - seqused_fp4[r]]
 * when slot(r) >= 0 and that offset is >= 0.
 *   key/value      [tokens][Hkv][128] bf16, token strides in elements
 *   tail_key/value this layer's [slots][128][Hkv][128] bf16; tail_slot_stride in elements
 */
int nvfp4_tail_append(const void* key, const void* value, int64_t key_token_stride,
                      int64_t value_token_stride, const void* key_shift_bf16, void* tail_key,
                      void* tail_value, int64_t tail_slot_stride,
                      const int32_t* query_start_loc, const int32_t* seq_lens,
                      const int32_t* seqused_fp4, const int32_t* row_to_slot, int num_tokens,
                      int num_reqs, int heads_kv, void* stream);

/*
 * Calibration of the key shift: sum[h][d] += the sum over the step's tokens of key[t][h][d],
 * accumulated in fp64, in one launch.
 * ref: the accumulation in NVFP4Impl.do_kv_cache_update, src/nvfp4_vllm/impl.py:137-144
 * (key[:num_actual_tokens].double().sum(dim=0) added to key_shift_sum[layer]).
 *   key  [tokens][Hkv][128] bf16, token stride in elements (multiple of 8), 16-byte aligned
 *   sum  [Hkv][128] fp64 accumulator of this layer (device)
 * The addends are BF16 numbers, so the fp64 partial sums are exact for any realistic spread of
 * magnitudes and the result does not depend on the order of the additions.
 */
int nvfp4_key_sum_accumulate(const void* key, int64_t key_token_stride, int num_tokens, int heads_kv,
                             double* sum, void* stream);

/*
 * One layer's K/V of a step in ONE launch: every full page of this step's prompts quantised
 * into its block (work table: src_tokens / dst_pages, -1 = skip; key shift fused) and every other
 * token copied to its row's tail slot (key shift fused).  Replaces the three launches of
 * write_kv, src/nvfp4_vllm/write.py:280-337 (two page quantisers + the tail copy) and the
 * torch.sub of impl.py:152.  Arguments as in nvfp4_quantize_kv_pages and nvfp4_tail_append;
 * work = 0 (a step without a full page) needs no page regions.
 */
int nvfp4_write_kv(const void* key, const void* value, int64_t key_token_stride, int64_t value_token_stride,
                   const void* key_shift_bf16, void* k_packed, int64_t k_pitch, void* k_sf, int64_t k_sf_pitch,
                   void* v_packed, int64_t v_pitch, void* v_sf, int64_t v_sf_pitch, const int32_t* src_tokens,
                   const int32_t* dst_pages, int work, void* tail_key, void* tail_value,
                   int64_t tail_slot_stride, const int32_t* query_start_loc, const int32_t* seq_lens,
                   const int32_t* seqused_fp4, const int32_t* row_to_slot, int num_tokens, int num_reqs,
                   int heads_kv, void* stream);

/*
 * Zero the tail page (all layers) of every row that starts a request this step
 * (seq_len <= query_len).  ref: reset_new_request_tails, write.py:133-215.
 */
int nvfp4_tail_reset(void* tail_key, void* tail_value, int64_t tail_layer_stride,
                     int64_t tail_slot_stride, int layers, const int32_t* query_start_loc,
                     const int32_t* seq_lens, const int32_t* row_to_slot, int num_reqs,
                     int heads_kv, void* stream);

/*
 * Tail flush (promotion): quantise every filled tail page of every layer into
 * its block, K and V in ONE launch.  ref: promote.launch, src/nvfp4_vllm/promote.py:33-62.
 *   tail_key/value [layers][slots][128][Hkv][128] bf16 seen as flat tokens
 *   src_tokens     int32[work] first tail token of item w (slot*128), dst_pages int32[work] (-1 = skip)
 *   bases          int64[4][layers]: K packed, K scales, V packed, V scales base addresses
 */
int nvfp4_tail_flush(const void* tail_key, const void* tail_value, int64_t src_layer_stride,
                     const int32_t* src_tokens, const int32_t* dst_pages, const int64_t* bases,
                     int64_t k_pitch, int64_t k_sf_pitch, int64_t v_pitch, int64_t v_sf_pitch,
                     int work, int layers, int heads_kv, void* stream);

/*
 * Split-KV paged decode.  ref: fp4_decode, src/nvfp4_decode_kernel/interface.py:17-182;
 * decode_fp4 / decode_fp4_split, _decode.py:532-1171.
 */
typedef struct nvfp4_decode_args {
  /* query */
  const void* q_fp4;          /* [rows][1][Hq][64] */
  const void* q_sf;           /* [rows][Hq*1024] */
  const void* q_bf16;         /* nullable: bf16 query used against the BF16 tail.  With q_fp4 and q_sf
                                 both NULL it is required, and the decode kernel quantises the rows
                                 itself with the arithmetic of nvfp4_quantize_q (bit-identical result,
                                 one launch instead of two): row r, head h at
                                 q_bf16 + r*row_stride + h*head_stride, 128 contiguous channels */
  int64_t q_bf16_row_stride;  /* elements */
  int64_t q_bf16_head_stride; /* elements */
  /* NVFP4 pages */
  const void* k_packed;
  int64_t k_pitch; /* bytes per page */
  const void* k_sf;
  int64_t k_sf_pitch;
  const void* v_packed;
  int64_t v_pitch;
  const void* v_sf;
  int64_t v_sf_pitch;
  int64_t num_pages;
  const int32_t* page_table;     /* [rows][max_pages], row stride in elements */
  int64_t page_table_row_stride;
  int32_t max_pages;
  const int32_t* seqused_fp4;    /* [rows], multiples of 128 */
  /* BF16 tail (all four NULL/0 when the call has no tail) */
  const void* tail_key;          /* [tail_pages][128][Hkv][128] bf16 */
  const void* tail_value;
  int64_t tail_pages;
  const int32_t* tail_ids;       /* [rows] */
  const int32_t* seqused_tail;   /* [rows] in [0,128] */
  /* outputs */
  void* out;                     /* nullable bf16 [>=rows][Hq][128] */
  const int32_t* out_indices;    /* nullable int32[rows] */
  float* o_partial;              /* nullable fp32 [S][rows][Hq][128]: normalised partial O */
  float* lse_partial;            /* nullable fp32 [S][rows][Hq]: natural-log LSE, -inf if empty */
  /* shape */
  int32_t rows;
  int32_t heads_q;
  int32_t heads_kv;
  float softmax_scale;
  int32_t num_splits;            /* >= 1; split s owns pages [s*ceil(n/S), min((s+1)*ceil(n/S), n)), the tail belongs to split 0 */
  int32_t impl;                  /* NVFP4_IMPL_* */
  /* scratch for num_splits > 1 when o_partial/lse_partial are NULL */
  void* workspace;
  size_t workspace_bytes;
  uint32_t* status;              /* nullable sticky device status word */
  uint32_t flags;                /* NVFP4_DECODE_* bits, 0 for the plain call */
  /* Fused tail append for one-token rows (all NULL/0: the tail was appended beforehand, as the
   * reference does with write_kv, src/nvfp4_vllm/write.py:280-337).  With append_key and
   * append_value given, row r's own token (token r of both, bf16 [rows][Hkv][128] at the token
   * strides) is stored at position seqused_tail[r] - 1 of tail page tail_ids[r] by the CTA that
   * owns the row's tail (key_shift, nullable bf16 [Hkv][128], subtracted from the key with one
   * BF16 subtract) and meets the query from the source.  seqused_tail counts the token; the tail
   * buffers are written; rows with seqused_tail 0 or a refused tail id append nothing.  The bytes
   * of the tail and of the output equal nvfp4_tail_append followed by the plain call. */
  const void* append_key;
  const void* append_value;
  int64_t append_key_token_stride;   /* elements */
  int64_t append_value_token_stride; /* elements */
  const void* key_shift;
} nvfp4_decode_args;

/*
 * NVFP4_DECODE_PROGRAMMATIC_LAUNCH (tensor-core kernel, no counterpart in the reference): the
 * launch carries the programmatic-stream-serialization attribute, so its CTAs may start while the
 * previous kernel in the stream is still draining.  Page tiles, scale blocks, the page table and
 * the lengths are then read BEFORE that kernel has completed: they must not be written by it
 * (in a decode step they are not: sealed pages and the step's metadata were written earlier).
 * The query, the BF16 tail and every output are touched only after the previous kernel has
 * completed and its writes are visible (griddepcontrol.wait); only then are this launch's own
 * dependents released, so the rule holds along a chain of such launches.
 */
#define NVFP4_DECODE_PROGRAMMATIC_LAUNCH 1u

/*
 * NVFP4_DECODE_REUSE_WORK_LIST (nvfp4_decode_balanced only): the workspace still holds the list
 * of pieces that an earlier nvfp4_decode_balanced call on this stream built from the same
 * seqused_fp4 values, rows, max_pages and target_pages; the list launch is skipped.  Meant for
 * the layers of one model step, whose lengths are the same: the first layer builds the list, the
 * others reuse it (their partial results overwrite the earlier layer's in the same workspace).
 * The list is trusted like trusted metadata: over a workspace that holds no such list the kernel
 * would follow whatever row numbers the bytes spell.
 */
#define NVFP4_DECODE_REUSE_WORK_LIST 2u

/*
 * NVFP4_DECODE_PERSISTENT (tensor-core kernel, 1, 2, 4 or 8 query heads per KV head; the launch
 * shape of the reference's persistent scheduler, src/nvfp4_decode_kernel/_fa4/tile_scheduler.py:202-211,
 * with page-granular shares in place of whole tiles): ONE launch of two CTAs per SM.  The step's
 * page tiles (and BF16 tails, weighted) are cut into equal shares, one per CTA, from the
 * device-resident lengths; a CTA sets up once and walks the pieces of its share back to back.  A
 * (row, KV head) tile that falls into several shares is merged by the piece that finishes last, in
 * a fixed order, so identical calls give identical bits.  Requires num_splits = 1, out != NULL, no
 * partial buffers; out_indices, the fused tail append and NVFP4_DECODE_PROGRAMMATIC_LAUNCH are
 * honoured.  workspace / workspace_bytes: at least nvfp4_decode_persistent_workspace_bytes(rows,
 * heads_q, heads_kv) bytes (computed for the current device), 16-byte aligned, ZERO-FILLED ONCE
 * before the first call; the kernel leaves it ready for the next call.  Calls that share a
 * workspace must not overlap on the device.  The result agrees with the plain call within the
 * re-association of the merge (a tile cut into pieces is folded as split partials are).
 */
#define NVFP4_DECODE_PERSISTENT 4u
size_t nvfp4_decode_persistent_workspace_bytes(int rows, int heads_q, int heads_kv);
/* 1 if NVFP4_DECODE_PERSISTENT takes this shape on the current device, else 0. */
int nvfp4_decode_persistent_supported(int rows, int heads_q, int heads_kv);

/*
 * NVFP4_DECODE_WIDE_FORM (tensor-core kernel; a hint, no counterpart in the reference): the caller
 * expects at most one busy CTA per SM - rows x KV heads x pieces at or below the SM count.  Such a
 * launch is bound by a CTA's own page period, not by HBM, and runs on the kernel's wide form: one
 * CTA per SM with two sets of producers, issuers and score warps and deeper rings.  Without the
 * flag the library chooses from what it can see (the grid of nvfp4_decode; for
 * nvfp4_decode_balanced the capacity of the list, an upper bound that is often far above the
 * pieces a step really has - a caller that knows the lengths on the host should say).  The
 * results are the same bits either way except for the row sum's association (see the kernel).
 */
#define NVFP4_DECODE_WIDE_FORM 8u
/* nvfp4_decode_balanced only: merge the pieces inside the decode launch (see there). */
#define NVFP4_DECODE_MERGE_IN_LAUNCH 16u
/* nvfp4_decode_host_io only: no copy operations, the kernel reads and writes the pinned host buffers (see there). */
#define NVFP4_DECODE_HOST_IO_DIRECT 32u

/*
 * With out != NULL the merged bf16 result is written (for num_splits > 1 the
 * partials go through o_partial/lse_partial if given, else through workspace).
 * With out == NULL the call only emits the partials (used by the cross-GPU
 * page-range split, where the merge happens after the exchange).
 */
int nvfp4_decode(const nvfp4_decode_args* args, void* stream);

size_t nvfp4_decode_workspace_bytes(int rows, int heads_q, int num_splits);

/* 1 if this build of the library carries the given NVFP4_IMPL_* decode kernel for a
 * group size heads_q / heads_kv, else 0. */
int nvfp4_decode_impl_available(int impl, int heads_q, int heads_kv);

/*
 * LSE merge of split partials.  ref: flash_attn_combine,
 * src/nvfp4_decode_kernel/split_k_combine.py:694-768.
 *   o_parts   fp32 [S][rows][Hq][128] with split stride o_split_stride (elements)
 *   lse_parts fp32 [S][rows][Hq] with split stride lse_split_stride (elements)
 *   out       [>=rows][Hq][128], bf16 (out_is_f32 = 0) or fp32 (1); out_indices nullable;
 *             lse_out nullable fp32 [rows][Hq]
 */
int nvfp4_lse_merge(const float* o_parts, int64_t o_split_stride, const float* lse_parts,
                    int64_t lse_split_stride, int num_splits, int rows, int heads_q, void* out,
                    int out_is_f32, const int32_t* out_indices, float* lse_out, void* stream);

/*
 * Same merge with one base pointer per split (partials that live in different
 * allocations, e.g. peer GPUs' buffers mapped into this process).
 *   o_part_ptrs / lse_part_ptrs: DEVICE arrays of num_splits pointers.
 */
int nvfp4_lse_merge_ptrs(const float* const* o_part_ptrs, const float* const* lse_part_ptrs,
                         int num_splits, int rows, int heads_q, void* out, int out_is_f32,
                         const int32_t* out_indices, float* lse_out, void* stream);

/*
 * Slot control plane: one step of the BF16 tail-slot table, entirely on the device (one CTA).
 * ref: _control_kernel / ControlPlane.prepare, src/nvfp4_vllm/control.py:114-334,447-511.
 * A row is a request iff seq_len > 0 and block_table[row][0] != 0 (the null block).  Rows keep
 * the slot keyed on their first block; new rows take the unclaimed slot that was seen longest
 * ago.  Outputs (all of width num_slots): row_to_slot (-1 = none), seqused_fp4 =
 * ((seq-1)/128)*128, seqused_residual = seq - seqused_fp4, promotion_source_tokens = slot*128,
 * promotion_pages = block_table[row][seq/128 - 1] when seq is a multiple of 128, else -1;
 * token_to_slot has num_actual_tokens entries.  error_code is a sticky OR of:
 * 1 prompt split across steps, 2 row with history matched no slot, 4 matched slot's length does
 * not continue, 8 no free slot, 16 two live rows share a block, 32 promotion column out of range.
 * slot_keys start at -1, slot_last_seq at -1, slot_last_seen (int64) at -1, step (int64) at 0.
 */
int nvfp4_control_step(const int32_t* block_table, int64_t block_table_stride, int block_table_columns,
                       const int32_t* seq_lens, const int32_t* query_start_loc, int32_t* slot_keys,
                       int32_t* slot_last_seq, int64_t* slot_last_seen, int64_t* step, int32_t* row_to_slot,
                       int32_t* token_to_slot, int32_t* seqused_fp4, int32_t* seqused_residual,
                       int32_t* promotion_source_tokens, int32_t* promotion_pages, int32_t* error_code,
                       int num_reqs, int num_actual_tokens, int num_slots, void* stream);

/*
 * The same step that also builds, in the same launch, the balanced split's list of pieces
 * (nvfp4_decode_balanced) for the first decode_rows rows of the batch, from the lengths it has
 * just computed (every live row holds a tail, so every live row gets its tail piece).  No
 * counterpart in the reference project.  workspace / max_pages / target_pages / heads_q: exactly
 * what the step's nvfp4_decode_balanced calls will be given (rows = decode_rows); those calls
 * then all pass NVFP4_DECODE_REUSE_WORK_LIST.  error_code bit 64: the list did not fit its
 * capacity (cannot happen with nvfp4_decode_balanced_capacity).
 */
int nvfp4_control_step_balanced(const int32_t* block_table, int64_t block_table_stride, int block_table_columns,
                                const int32_t* seq_lens, const int32_t* query_start_loc, int32_t* slot_keys,
                                int32_t* slot_last_seq, int64_t* slot_last_seen, int64_t* step,
                                int32_t* row_to_slot, int32_t* token_to_slot, int32_t* seqused_fp4,
                                int32_t* seqused_residual, int32_t* promotion_source_tokens,
                                int32_t* promotion_pages, int32_t* error_code, int num_reqs,
                                int num_actual_tokens, int num_slots, int decode_rows, int max_pages,
                                int target_pages, int heads_q, void* workspace, size_t workspace_bytes,
                                void* stream);

/*
 * Page work table of a step: for row r and page column c < columns_per_row,
 * source_tokens[r*columns+c] = query_start_loc[r] + 128*c and destination_pages[...] =
 * block_table[r][c] if the row is a fresh prefill (more than one query token, owns a slot) and
 * c < seqused_fp4[r]/128, else -1.  ref: _work_table_kernel, src/nvfp4_vllm/write.py:30-76.
 */
int nvfp4_work_table(const int32_t* query_start_loc, const int32_t* seqused_fp4, const int32_t* row_to_slot,
                     const int32_t* block_table, int64_t block_table_stride, int32_t* source_tokens,
                     int32_t* destination_pages, int num_reqs, int columns_per_row, void* stream);

/*
 * Cross-GPU page-range split, push form: ONE launch per rank after the decode.  No counterpart
 * in the reference project (it has no multi-GPU code); the partial format and the merge are those
 * of its split path (fp4_decode_kernel.py:5186-5196, split_k_combine.py:694-768).
 * The CTA of (query head, row) folds this rank's local_splits partials
 *   o_local   fp32 [S][rows][Hq][128] (split stride in elements), lse_local fp32 [S][rows][Hq],
 * stores the result into its slot of every peer's inbox (remote stores only), announces it in the
 * peer's flag array, waits (bounded, 1 s; NVFP4_STATUS_WAIT_TIMEOUT and out untouched on expiry)
 * for the peers' pushes of the same (head, row), and merges in rank order out of its own inbox.
 *   inbox_ptrs DEVICE array [world] of each rank's inbox as this process addresses it:
 *              float [2][world][rows*Hq][132] (nvfp4_push_merge_inbox_floats), zero-filled once
 *   flag_ptrs  DEVICE array [world] of each rank's flags: int32 [world][rows*Hq], zero-filled once
 *   epoch      1, 2, 3, ... per call, the same on every rank; with epoch_state != NULL (two device
 *              ints, zero-filled once) the kernel keeps the count itself, for CUDA-graph replay
 * The ranks' kernels must run on different GPUs.
 */
int nvfp4_push_merge(const float* o_local, int64_t o_split_stride, const float* lse_local,
                     int64_t lse_split_stride, int local_splits, float* const* inbox_ptrs,
                     int32_t* const* flag_ptrs, int rank, int world, int epoch, int32_t* epoch_state,
                     int rows, int heads_q, void* out, int out_is_f32, uint32_t* status, void* stream);
size_t nvfp4_push_merge_inbox_floats(int world, int rows, int heads_q);

/*
 * Decode and cross-GPU page-range exchange in ONE launch per rank (tensor-core kernel only).
 * No counterpart in the reference project.  The decode runs in partial mode with
 * args->num_splits local splits (args->o_partial / lse_partial: this rank's scratch,
 * [S][rows][Hq][128] and [S][rows][Hq]; args->out must be NULL).  The CTA that stores the last
 * split partial of a (row, KV head) tile folds the tile's splits, pushes the result into every
 * peer's inbox, announces it, waits (bounded, 1 s) for the peers' pushes of that tile and writes
 * the merged rows to x->out: tiles that finish early are exchanged while others still stream.
 * Inbox, flags and epoch_state are those of nvfp4_push_merge (the two entry points produce the
 * same bits); tile_counters: device int32 [rows * heads_kv], zero-filled once.
 * heads_q / heads_kv <= 8 (16 and 32 heads per KV head take nvfp4_push_merge as a second launch),
 * world * (heads_q / heads_kv) <= 128.  The ranks' kernels must run on different GPUs.
 */
typedef struct nvfp4_exchange_args {
  float* const* inbox_ptrs;   /* DEVICE array [world] */
  int32_t* const* flag_ptrs;  /* DEVICE array [world] */
  int32_t* epoch_state;       /* two device ints, zero-filled once */
  int32_t* tile_counters;     /* device ints [rows * heads_kv], zero-filled once */
  void* out;                  /* [rows][Hq][128] bf16 (out_is_f32 = 0) or fp32 (1) */
  int32_t out_is_f32;
  int32_t rank;
  int32_t world;
} nvfp4_exchange_args;

int nvfp4_decode_exchange(const nvfp4_decode_args* args, const nvfp4_exchange_args* x, void* stream);

/*
 * Split-KV decode with a split count per row ("balanced split").  No counterpart in the
 * reference project, whose split count is one number for the whole batch
 * (src/nvfp4_decode_kernel/_decode.py:1018-1049): in a ragged batch that number follows the
 * longest row, so short rows are cut into pieces far smaller than a CTA's fixed cost is worth, or
 * the long rows into pieces too long.
 *
 * Row r is cut into ceil(pages_r / target_pages) pieces of pages, and a row that holds a BF16
 * tail gets one more piece for the tail alone (served out of shared memory, never walked in front
 * of a piece's page stream); a row with neither keeps one empty piece.  A page piece is computed
 * exactly as split s of num_splits = that count would be (without the tail), and the pieces of a
 * row are merged by their log-sum-exp.  Three launches on the stream: the work list (built on
 * the device from seqused_fp4 and seqused_tail, so the call needs no host knowledge of the lengths
 * and can be captured in a CUDA graph), the decode, and the merge of every row's pieces.
 *
 *  - args as for nvfp4_decode with num_splits = 1, out != NULL, o_partial = lse_partial =
 *    out_indices = NULL, no NVFP4_DECODE_PROGRAMMATIC_LAUNCH; tensor-core kernel only.
 *  - args.flags may carry NVFP4_DECODE_REUSE_WORK_LIST (no list launch: the list of an earlier
 *    call or of nvfp4_control_step_balanced is still in the workspace) and
 *    NVFP4_DECODE_MERGE_IN_LAUNCH (no merge launch: the piece of a (row, KV head) that finishes
 *    last merges the row's pieces inside the decode launch - same arithmetic, same order, the
 *    same bits whichever piece is last.  Measured slower than the merge launch on a B200: every
 *    piece pays a device-wide fence before it counts its arrival; kept as an option).
 *  - args.workspace must hold nvfp4_decode_balanced_workspace_bytes(rows, heads_q, max_pages,
 *    target_pages) bytes (args.max_pages is the bound on a row's page count that the list's
 *    capacity, nvfp4_decode_balanced_capacity, is derived from).
 */
int nvfp4_decode_balanced(const nvfp4_decode_args* args, int target_pages, void* stream);
int64_t nvfp4_decode_balanced_capacity(int rows, int max_pages, int target_pages);
size_t nvfp4_decode_balanced_workspace_bytes(int rows, int heads_q, int max_pages, int target_pages);

/*
 * Split-KV decode for callers that cannot allocate.  No counterpart in the reference project
 * (its split path allocates and fills its partial buffers on every call,
 * src/nvfp4_decode_kernel/_decode.py:1051-1065).
 *
 * Meant for an engine that has handed every free byte of HBM to its KV cache after a memory
 * profiling pass, or that must not take the device-wide synchronisation an allocation implies in
 * the middle of a decode step: the per-split partial results go into a fixed array of
 * NVFP4_STATIC_WORKSPACE_BYTES that is part of the library image (every GPU that loads the
 * library holds it until the process exits).  The call itself never allocates or frees.
 *
 *  - args as for nvfp4_decode with num_splits >= 2 and out != NULL; workspace, workspace_bytes,
 *    o_partial and lse_partial are ignored / must be NULL.
 *  - rows * heads_q * num_splits * 516 bytes must fit the array, otherwise NVFP4_ERR_INVALID with
 *    a message (nvfp4_decode_split_static_error()) that names both sizes.
 *  - Set-up: the first call on a device (with that device current) looks the array's address
 *    up before it checks anything else.  The CUDA runtime loads the module holding the array at
 *    that moment, which takes the array's bytes out of the device's free memory - once, by the
 *    module loader, not by an allocation call, and measured on a B200 as exactly
 *    NVFP4_STATIC_WORKSPACE_BYTES.  A caller that sizes its KV cache from the free memory makes
 *    that first call beforehand, and before any stream capture: nvfp4_decode_split_static(NULL,
 *    NULL) does the set-up and then returns NVFP4_ERR_INVALID ("null argument block").  Every
 *    later call on the device leaves both the allocator and the free-memory count untouched.
 *  - All calls on a device share the one array: two calls whose kernels may overlap on the GPU
 *    (different streams, no ordering) race on it.  Nothing in it needs clearing between calls -
 *    every slot that the merge reads is written by the decode kernel of the same call.
 */
#define NVFP4_STATIC_WORKSPACE_BYTES (8u << 20)
int nvfp4_decode_split_static(const nvfp4_decode_args* args, void* stream);
size_t nvfp4_static_workspace_bytes(void);
const char* nvfp4_decode_split_static_error(void);

/*
 * Merge for the cross-GPU KV page-range split (one process per GPU).  Each rank has written
 * its partial (normalised fp32 O [rows][Hq][128], fp32 LSE [rows][Hq]) into memory every rank
 * can address (peer-mapped / symmetric allocations).  The call announces "partial of `epoch`
 * written" in every peer's flag array (flag_ptrs[p][rank] = epoch), waits - at most one second,
 * then NVFP4_STATUS_WAIT_TIMEOUT is raised and `out` is left untouched - until every peer has
 * announced the same epoch, and merges by LSE weight with plain loads from the peers' buffers.
 * Epochs must grow by one per call on every rank; partial buffers should alternate between two
 * copies so that a fast rank cannot overwrite what a slow one still reads.  With epoch_state
 * (two zero-initialised int32 in device memory, private to the rank) the epoch is kept on the
 * device - the call uses epoch_state[0] + 1 and advances it - so that the launch can be
 * replayed from a CUDA graph; `epoch` is then ignored.
 * The reference has no multi-GPU path; the merge arithmetic is that of flash_attn_combine
 * (src/nvfp4_decode_kernel/split_k_combine.py:516-554).
 *   o_part_ptrs / lse_part_ptrs / flag_ptrs: DEVICE arrays of `world` pointers.
 */
int nvfp4_peer_merge(const float* const* o_part_ptrs, const float* const* lse_part_ptrs,
                     int32_t* const* flag_ptrs, int rank, int world, int epoch, int32_t* epoch_state,
                     int rows, int heads_q, void* out, int out_is_f32, uint32_t* status, void* stream);

/*
 * One decode step for a caller whose query and result live in HOST memory (no counterpart in the
 * reference, whose operator takes device tensors; it saves such a caller three trips through its
 * framework per step): copies q_host (pinned, q_bytes: the BF16 query exactly as args->q_bf16 with
 * its strides lays it out) to args->q_bf16 on `stream`, runs nvfp4_decode(args), copies
 * out_bytes of args->out to out_host (pinned) and waits for the stream.  Everything args points
 * to stays device memory, the KV pages stay resident.  Returns after the result is in out_host.
 * With NVFP4_DECODE_HOST_IO_DIRECT in args->flags there are no copy operations: pinned host memory
 * is mapped into the device's address space, so the decode kernel reads the query from q_host and
 * writes the rows to out_host over PCIe itself (every byte crosses once, as with the copies;
 * args->q_bf16 and args->out then only describe the layout).  One launch and the wait.
 */
int nvfp4_decode_host_io(const nvfp4_decode_args* args, const void* q_host, size_t q_bytes, void* out_host,
                         size_t out_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NVFP4_B200_H_ */
