// C ABI of the library: argument validation, error reporting, dispatch.
// No torch types, no allocation, no stream synchronisation.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/nvfp4_b200.h"
#include "nvfp4_kernels.h"

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(e == cudaErrorNotSupported ? NVFP4_ERR_UNSUPPORTED : NVFP4_ERR_CUDA, "%s: %s", what,
              cudaGetErrorString(e));
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool valid_group(int heads_q, int heads_kv) {
  if (heads_kv < 1 || heads_q < 1 || heads_q % heads_kv) return false;
  const int g = heads_q / heads_kv;
  return (g >= 1 && g <= 8) || g == 16 || g == 32;
}

}  // namespace

extern "C" {

const char* nvfp4_last_error(void) { return g_error; }

int nvfp4_version(void) { return 100; }

int nvfp4_device_supported(int device) {
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) {
    cuda_fail(e, "cudaGetDeviceProperties");
    return -1;
  }
  return prop.major == 10 ? 1 : 0;
}

int nvfp4_quantize_q(const void* q_bf16, int64_t q_row_stride, int64_t q_head_stride,
                     const int32_t* row_indices, void* q_fp4, void* q_sf, void* q_padded, int rows,
                     int heads_q, int heads_kv, void* stream) {
  if (rows < 0) return fail(NVFP4_ERR_INVALID, "rows must be non-negative, got %d", rows);
  if (rows == 0) return NVFP4_OK;
  if (!q_bf16 || !q_fp4 || !q_sf) return fail(NVFP4_ERR_INVALID, "q_bf16, q_fp4 and q_sf must be non-null");
  if (heads_kv < 1 || heads_q < 1 || heads_q % heads_kv)
    return fail(NVFP4_ERR_INVALID, "query heads must be divisible by heads_kv (%d, %d)", heads_q, heads_kv);
  if (heads_q / heads_kv > 128)
    return fail(NVFP4_ERR_INVALID, "at most 128 query heads per KV head fit one scale block");
  if (!aligned16(q_bf16) || !aligned16(q_fp4) || !aligned16(q_sf) || (q_padded && !aligned16(q_padded)) ||
      (q_row_stride % 8) || (q_head_stride % 8))
    return fail(NVFP4_ERR_INVALID, "query buffers and strides must keep 16-byte alignment");
  cudaError_t e = nvfp4::launch_quantize_q(q_bf16, q_row_stride, q_head_stride, row_indices, q_fp4,
                                           q_sf, q_padded, rows, heads_q, heads_kv,
                                           static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "quantize_q launch");
}

int nvfp4_quantize_kv_pages(int which, const void* tokens_bf16, int64_t token_stride,
                            const void* key_shift_bf16, void* packed, int64_t packed_pitch, void* sf,
                            int64_t sf_pitch, const int32_t* src_tokens, const int32_t* dst_pages,
                            const int64_t* packed_bases, const int64_t* sf_bases, int work,
                            int layers, int64_t src_layer_stride, int heads_kv, void* stream) {
  if (which != 0 && which != 1) return fail(NVFP4_ERR_INVALID, "which must be 0 (K) or 1 (V)");
  if (work < 0 || layers < 1) return fail(NVFP4_ERR_INVALID, "work must be >= 0 and layers >= 1");
  if (work == 0) return NVFP4_OK;
  if (heads_kv < 1 || heads_kv > 128) return fail(NVFP4_ERR_INVALID, "heads_kv out of range: %d", heads_kv);
  if (!tokens_bf16) return fail(NVFP4_ERR_INVALID, "tokens_bf16 must be non-null");
  if ((!packed_bases) != (!sf_bases))
    return fail(NVFP4_ERR_INVALID, "packed_bases and sf_bases must be given together");
  if (!packed_bases && (!packed || !sf))
    return fail(NVFP4_ERR_INVALID, "packed and sf must be non-null without a base table");
  if (layers > 1 && !packed_bases)
    return fail(NVFP4_ERR_INVALID, "layers > 1 needs per-layer destination bases");
  const int64_t dense_packed = (int64_t)128 * heads_kv * 64, dense_sf = (int64_t)heads_kv * 1024;
  if (packed_pitch < dense_packed || (packed_pitch % 16))
    return fail(NVFP4_ERR_INVALID, "packed page pitch must be >= %lld bytes and 16-byte aligned, got %lld",
                (long long)dense_packed, (long long)packed_pitch);
  if (sf_pitch < dense_sf || (sf_pitch % 16))
    return fail(NVFP4_ERR_INVALID, "scale page pitch must be >= %lld bytes and 16-byte aligned, got %lld",
                (long long)dense_sf, (long long)sf_pitch);
  if (token_stride < (int64_t)heads_kv * 128 || (token_stride % 8) || !aligned16(tokens_bf16))
    return fail(NVFP4_ERR_INVALID, "token source must be dense within a token and 16-byte aligned");
  if ((packed && !aligned16(packed)) || (sf && !aligned16(sf)) || (key_shift_bf16 && !aligned16(key_shift_bf16)))
    return fail(NVFP4_ERR_INVALID, "destination regions must be 16-byte aligned");
  if (which == 1 && key_shift_bf16) return fail(NVFP4_ERR_INVALID, "the key shift applies to K only");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e =
      which == 0 ? nvfp4::launch_quantize_k(tokens_bf16, token_stride, key_shift_bf16, packed,
                                            packed_pitch, sf, sf_pitch, src_tokens, dst_pages,
                                            packed_bases, sf_bases, work, layers, src_layer_stride,
                                            heads_kv, st)
                 : nvfp4::launch_quantize_v(tokens_bf16, token_stride, packed, packed_pitch, sf,
                                            sf_pitch, src_tokens, dst_pages, packed_bases, sf_bases,
                                            work, layers, src_layer_stride, heads_kv, st);
  return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "quantize_kv_pages launch");
}

int nvfp4_tail_append(const void* key, const void* value, int64_t key_token_stride,
                      int64_t value_token_stride, const void* key_shift_bf16, void* tail_key,
                      void* tail_value, int64_t tail_slot_stride, const int32_t* query_start_loc,
                      const int32_t* seq_lens, const int32_t* seqused_fp4, const int32_t* row_to_slot,
                      int num_tokens, int num_reqs, int heads_kv, void* stream) {
  if (num_tokens < 0 || num_reqs < 0) return fail(NVFP4_ERR_INVALID, "negative token or row count");
  if (num_tokens == 0 || num_reqs == 0) return NVFP4_OK;
  if (!key || !value || !tail_key || !tail_value || !query_start_loc || !seq_lens || !seqused_fp4 || !row_to_slot)
    return fail(NVFP4_ERR_INVALID, "tail_append: null argument");
  if (heads_kv < 1) return fail(NVFP4_ERR_INVALID, "heads_kv must be positive");
  const int64_t width = (int64_t)heads_kv * 128;
  if (key_token_stride < width || value_token_stride < width || (key_token_stride % 8) ||
      (value_token_stride % 8) || tail_slot_stride < 128 * width || !aligned16(key) ||
      !aligned16(value) || !aligned16(tail_key) || !aligned16(tail_value) ||
      (key_shift_bf16 && !aligned16(key_shift_bf16)))
    return fail(NVFP4_ERR_INVALID, "tail_append: strides must cover a token and keep 16-byte alignment");
  cudaError_t e = nvfp4::launch_tail_append(key, value, key_token_stride, value_token_stride,
                                            key_shift_bf16, tail_key, tail_value, tail_slot_stride,
                                            query_start_loc, seq_lens, seqused_fp4, row_to_slot,
                                            num_tokens, num_reqs, heads_kv,
                                            static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "tail_append launch");
}

int nvfp4_write_kv(const void* key, const void* value, int64_t key_token_stride, int64_t value_token_stride,
                   const void* key_shift_bf16, void* k_packed, int64_t k_pitch, void* k_sf, int64_t k_sf_pitch,
                   void* v_packed, int64_t v_pitch, void* v_sf, int64_t v_sf_pitch, const int32_t* src_tokens,
                   const int32_t* dst_pages, int work, void* tail_key, void* tail_value,
                   int64_t tail_slot_stride, const int32_t* query_start_loc, const int32_t* seq_lens,
                   const int32_t* seqused_fp4, const int32_t* row_to_slot, int num_tokens, int num_reqs,
                   int heads_kv, void* stream) {
  if (num_tokens < 0 || num_reqs < 0 || work < 0) return fail(NVFP4_ERR_INVALID, "write_kv: negative count");
  if (num_tokens == 0 || num_reqs == 0) return NVFP4_OK;
  if (!key || !value || !tail_key || !tail_value || !query_start_loc || !seq_lens || !seqused_fp4 || !row_to_slot)
    return fail(NVFP4_ERR_INVALID, "write_kv: null argument");
  if (heads_kv < 1 || heads_kv > 65535 - 4) return fail(NVFP4_ERR_INVALID, "write_kv: bad heads_kv");
  if (work > 65535) return fail(NVFP4_ERR_INVALID, "write_kv: at most 65535 page-work items");
  const int64_t width = (int64_t)heads_kv * 128;
  if (key_token_stride < width || value_token_stride < width || (key_token_stride % 8) ||
      (value_token_stride % 8) || tail_slot_stride < 128 * width || !aligned16(key) || !aligned16(value) ||
      !aligned16(tail_key) || !aligned16(tail_value) || (key_shift_bf16 && !aligned16(key_shift_bf16)))
    return fail(NVFP4_ERR_INVALID, "write_kv: strides must cover a token and keep 16-byte alignment");
  if (work > 0) {
    if (!k_packed || !k_sf || !v_packed || !v_sf || !src_tokens || !dst_pages)
      return fail(NVFP4_ERR_INVALID, "write_kv: page work needs the page regions and the work table");
    const int64_t dense_packed = 128 * (int64_t)heads_kv * 64, dense_sf = (int64_t)heads_kv * 1024;
    if (k_pitch < dense_packed || v_pitch < dense_packed || k_sf_pitch < dense_sf || v_sf_pitch < dense_sf ||
        (k_pitch % 16) || (v_pitch % 16) || (k_sf_pitch % 16) || (v_sf_pitch % 16) || !aligned16(k_packed) ||
        !aligned16(k_sf) || !aligned16(v_packed) || !aligned16(v_sf))
      return fail(NVFP4_ERR_INVALID, "write_kv: page pitches must cover a dense page and keep 16-byte alignment");
  }
  cudaError_t e = nvfp4::launch_write_kv(key, value, key_token_stride, value_token_stride, key_shift_bf16,
                                         k_packed, k_pitch, k_sf, k_sf_pitch, v_packed, v_pitch, v_sf,
                                         v_sf_pitch, src_tokens, dst_pages, work, tail_key, tail_value,
                                         tail_slot_stride, query_start_loc, seq_lens, seqused_fp4, row_to_slot,
                                         num_tokens, num_reqs, heads_kv, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "write_kv launch");
}

int nvfp4_key_sum_accumulate(const void* key, int64_t key_token_stride, int num_tokens, int heads_kv,
                             double* sum, void* stream) {
  if (num_tokens < 0) return fail(NVFP4_ERR_INVALID, "key_sum_accumulate: negative token count");
  if (num_tokens == 0) return NVFP4_OK;
  if (!key || !sum) return fail(NVFP4_ERR_INVALID, "key_sum_accumulate: null argument");
  if (heads_kv < 1 || heads_kv > 4096) return fail(NVFP4_ERR_INVALID, "key_sum_accumulate: bad heads_kv");
  if (key_token_stride < (int64_t)heads_kv * 128 || (key_token_stride % 8) || !aligned16(key) ||
      (reinterpret_cast<uintptr_t>(sum) & 7))
    return fail(NVFP4_ERR_INVALID,
                "key_sum_accumulate: the token stride must cover a token and keep 16-byte alignment");
  cudaError_t e = nvfp4::launch_key_sum(key, key_token_stride, num_tokens, heads_kv, sum,
                                        static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "key_sum_accumulate launch");
}

int nvfp4_tail_reset(void* tail_key, void* tail_value, int64_t tail_layer_stride,
                     int64_t tail_slot_stride, int layers, const int32_t* query_start_loc,
                     const int32_t* seq_lens, const int32_t* row_to_slot, int num_reqs, int heads_kv,
                     void* stream) {
  if (layers < 0 || num_reqs < 0) return fail(NVFP4_ERR_INVALID, "negative layer or row count");
  if (layers == 0 || num_reqs == 0) return NVFP4_OK;
  if (!tail_key || !tail_value || !query_start_loc || !seq_lens || !row_to_slot)
    return fail(NVFP4_ERR_INVALID, "tail_reset: null argument");
  if (num_reqs > 65535) return fail(NVFP4_ERR_INVALID, "tail_reset: too many rows");
  const int64_t width = (int64_t)heads_kv * 128;
  if (heads_kv < 1 || tail_slot_stride < 128 * width || !aligned16(tail_key) || !aligned16(tail_value) ||
      (tail_slot_stride % 8) || (tail_layer_stride % 8))
    return fail(NVFP4_ERR_INVALID, "tail_reset: strides must cover a page and keep 16-byte alignment");
  cudaError_t e = nvfp4::launch_tail_reset(tail_key, tail_value, tail_layer_stride, tail_slot_stride,
                                           layers, query_start_loc, seq_lens, row_to_slot, num_reqs,
                                           heads_kv, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "tail_reset launch");
}

int nvfp4_tail_flush(const void* tail_key, const void* tail_value, int64_t src_layer_stride,
                     const int32_t* src_tokens, const int32_t* dst_pages, const int64_t* bases,
                     int64_t k_pitch, int64_t k_sf_pitch, int64_t v_pitch, int64_t v_sf_pitch,
                     int work, int layers, int heads_kv, void* stream) {
  if (work < 0 || layers < 0) return fail(NVFP4_ERR_INVALID, "negative work or layer count");
  if (work == 0 || layers == 0) return NVFP4_OK;
  if (!tail_key || !tail_value || !src_tokens || !dst_pages || !bases)
    return fail(NVFP4_ERR_INVALID, "tail_flush: null argument");
  if (heads_kv < 1 || heads_kv > 128) return fail(NVFP4_ERR_INVALID, "heads_kv out of range: %d", heads_kv);
  const int64_t dense_packed = (int64_t)128 * heads_kv * 64, dense_sf = (int64_t)heads_kv * 1024;
  if (k_pitch < dense_packed || v_pitch < dense_packed || k_sf_pitch < dense_sf || v_sf_pitch < dense_sf ||
      (k_pitch % 16) || (v_pitch % 16) || (k_sf_pitch % 16) || (v_sf_pitch % 16))
    return fail(NVFP4_ERR_INVALID, "tail_flush: page pitches must cover a dense page and be 16-byte aligned");
  if (!aligned16(tail_key) || !aligned16(tail_value))
    return fail(NVFP4_ERR_INVALID, "tail_flush: tail buffers must be 16-byte aligned");
  if (layers > 65535 || work > 65535) return fail(NVFP4_ERR_INVALID, "tail_flush: grid too large");
  cudaError_t e = nvfp4::launch_tail_flush(tail_key, tail_value, src_layer_stride, src_tokens,
                                           dst_pages, bases, k_pitch, k_sf_pitch, v_pitch, v_sf_pitch,
                                           work, layers, heads_kv, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "tail_flush launch");
}

size_t nvfp4_decode_workspace_bytes(int rows, int heads_q, int num_splits) {
  if (rows <= 0 || heads_q <= 0 || num_splits <= 1) return 0;
  return (size_t)num_splits * rows * heads_q * (128 + 1) * sizeof(float);
}

int nvfp4_decode_impl_available(int impl, int heads_q, int heads_kv) {
  if (!valid_group(heads_q, heads_kv)) return 0;
  if (impl == NVFP4_IMPL_GENERIC || impl == NVFP4_IMPL_AUTO) return 1;
  if (impl == NVFP4_IMPL_SM100) {
    nvfp4::DecodeParams p;
    std::memset(&p, 0, sizeof(p));
    p.heads_q = heads_q;
    p.heads_kv = heads_kv;
    return nvfp4::decode_sm100_supports(p) ? 1 : 0;
  }
  return 0;
}

static int decode_call(const nvfp4_decode_args* a, const nvfp4_exchange_args* x, int target_pages, void* stream);

int nvfp4_decode(const nvfp4_decode_args* a, void* stream) { return decode_call(a, nullptr, 0, stream); }

int nvfp4_decode_host_io(const nvfp4_decode_args* a, const void* q_host, size_t q_bytes, void* out_host,
                         size_t out_bytes, void* stream) {
  if (!a || !q_host || !out_host) return fail(NVFP4_ERR_INVALID, "decode_host_io: null argument");
  if (!a->q_bf16 || !a->out)
    return fail(NVFP4_ERR_INVALID, "decode_host_io: args must carry the device BF16 query buffer and out");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  // Pinned host memory is mapped into the device's address space: the kernel then reads the
  // query and writes the rows over PCIe itself (every byte crosses once, as with the copies),
  // which saves the two copy operations' own latency - a third of the step.
  if (a->flags & NVFP4_DECODE_HOST_IO_DIRECT) {
    cudaPointerAttributes qa{}, oa{};
    if (cudaPointerGetAttributes(&qa, q_host) != cudaSuccess || cudaPointerGetAttributes(&oa, out_host) != cudaSuccess ||
        qa.type != cudaMemoryTypeHost || oa.type != cudaMemoryTypeHost || !qa.devicePointer || !oa.devicePointer) {
      (void)cudaGetLastError();
      return fail(NVFP4_ERR_INVALID, "decode_host_io: the direct form needs pinned (mapped) host buffers");
    }
    nvfp4_decode_args direct = *a;
    direct.flags &= ~NVFP4_DECODE_HOST_IO_DIRECT;
    direct.q_bf16 = qa.devicePointer;
    direct.out = oa.devicePointer;
    const int rc = decode_call(&direct, nullptr, 0, stream);
    if (rc != NVFP4_OK) return rc;
    e = cudaStreamSynchronize(st);
    return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "decode_host_io: stream synchronisation");
  }
  e = cudaMemcpyAsync(const_cast<void*>(a->q_bf16), q_host, q_bytes, cudaMemcpyHostToDevice, st);
  if (e != cudaSuccess) return cuda_fail(e, "decode_host_io: query copy");
  const int rc = decode_call(a, nullptr, 0, stream);
  if (rc != NVFP4_OK) return rc;
  e = cudaMemcpyAsync(out_host, a->out, out_bytes, cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) return cuda_fail(e, "decode_host_io: result copy");
  e = cudaStreamSynchronize(st);
  return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "decode_host_io: stream synchronisation");
}

size_t nvfp4_decode_persistent_workspace_bytes(int rows, int heads_q, int heads_kv) {
  if (rows <= 0 || !valid_group(heads_q, heads_kv)) return 0;
  return nvfp4::decode_persistent_workspace_bytes(rows, heads_q, heads_kv);
}

int nvfp4_decode_persistent_supported(int rows, int heads_q, int heads_kv) {
  if (rows < 0 || !valid_group(heads_q, heads_kv)) return 0;
  nvfp4::DecodeParams p;
  std::memset(&p, 0, sizeof(p));
  p.rows = rows;
  p.heads_q = heads_q;
  p.heads_kv = heads_kv;
  return nvfp4::decode_persistent_supports(p) ? 1 : 0;
}

// Balanced split: row r is cut into ceil(pages_r / target_pages) pieces of pages plus one piece
// for its BF16 tail if it holds one (one empty piece if it has neither), so the list of pieces is
// never longer than 2 * rows + rows * max_pages / target_pages.
int64_t nvfp4_decode_balanced_capacity(int rows, int max_pages, int target_pages) {
  if (rows <= 0 || max_pages < 0 || target_pages < 1) return 0;
  return 2 * (int64_t)rows + (int64_t)rows * max_pages / target_pages;
}

namespace {
struct BalancedLayout {
  size_t o_part, lse_part, work, row_offset, row_count, counters, total;
};
BalancedLayout balanced_layout(int rows, int heads_q, int64_t capacity) {
  BalancedLayout l;
  size_t at = 0;
  auto take = [&](size_t bytes) { const size_t here = at; at += (bytes + 15) & ~(size_t)15; return here; };
  l.o_part = take((size_t)capacity * heads_q * 128 * sizeof(float));
  l.lse_part = take((size_t)capacity * heads_q * sizeof(float));
  l.work = take((size_t)capacity * sizeof(int4));
  l.row_offset = take((size_t)rows * sizeof(int32_t));
  l.row_count = take((size_t)rows * sizeof(int32_t));
  l.counters = take((size_t)rows * heads_q * sizeof(int32_t));   // arrivals per (row, KV head); heads_q bounds heads_kv
  l.total = at;
  return l;
}
}  // namespace

size_t nvfp4_decode_balanced_workspace_bytes(int rows, int heads_q, int max_pages, int target_pages) {
  const int64_t capacity = nvfp4_decode_balanced_capacity(rows, max_pages, target_pages);
  if (capacity <= 0 || heads_q <= 0) return 0;
  return balanced_layout(rows, heads_q, capacity).total;
}

int nvfp4_decode_balanced(const nvfp4_decode_args* a, int target_pages, void* stream) {
  if (!a) return fail(NVFP4_ERR_INVALID, "decode: null argument block");
  if (target_pages < 1) return fail(NVFP4_ERR_INVALID, "decode_balanced: target_pages must be at least 1, got %d", target_pages);
  if (a->num_splits != 1 || !a->out || a->o_partial || a->lse_partial || a->out_indices)
    return fail(NVFP4_ERR_INVALID,
                "decode_balanced: the split is per row; give num_splits = 1, out, and neither partial "
                "buffers nor out_indices");
  return decode_call(a, nullptr, target_pages, stream);
}

int nvfp4_decode_exchange(const nvfp4_decode_args* a, const nvfp4_exchange_args* x, void* stream) {
  if (!x) return fail(NVFP4_ERR_INVALID, "decode_exchange: null exchange block");
  if (!a) return fail(NVFP4_ERR_INVALID, "decode: null argument block");
  if (x->world < 1 || x->world > 16 || x->rank < 0 || x->rank >= x->world)
    return fail(NVFP4_ERR_INVALID, "decode_exchange: rank %d of %d is out of range (at most 16 ranks)", x->rank,
                x->world);
  if (!x->inbox_ptrs || !x->flag_ptrs || !x->epoch_state || !x->tile_counters || !x->out)
    return fail(NVFP4_ERR_INVALID, "decode_exchange: null argument");
  if (a->out || !a->o_partial || !a->lse_partial)
    return fail(NVFP4_ERR_INVALID,
                "decode_exchange: the merged rows go to the exchange block's out; give o_partial and "
                "lse_partial for the local splits and leave args.out null");
  return decode_call(a, x, 0, stream);
}

static int decode_call(const nvfp4_decode_args* a, const nvfp4_exchange_args* x, int target_pages, void* stream) {
  if (!a) return fail(NVFP4_ERR_INVALID, "decode: null argument block");
  if (a->rows < 0) return fail(NVFP4_ERR_INVALID, "decode: negative row count");
  if (a->rows == 0) return NVFP4_OK;
  if (!valid_group(a->heads_q, a->heads_kv))
    return fail(NVFP4_ERR_UNSUPPORTED,
                "decode: heads_q/heads_kv = %d/%d; the ratio must be 1 to 8, 16 or 32", a->heads_q,
                a->heads_kv);
  if (!(a->softmax_scale > 0.f) || !(a->softmax_scale < 3.0e38f))
    return fail(NVFP4_ERR_INVALID, "softmax_scale must be finite and positive");
  if (a->num_splits < 1 || a->num_splits > 1024)
    return fail(NVFP4_ERR_INVALID, "num_splits must be in [1, 1024], got %d", a->num_splits);
  if (!a->k_packed || !a->k_sf || !a->v_packed || !a->v_sf || !a->page_table || !a->seqused_fp4)
    return fail(NVFP4_ERR_INVALID, "decode: a required pointer is null");
  const bool fused_query = !a->q_fp4 && !a->q_sf;
  if (fused_query ? !a->q_bf16 : (!a->q_fp4 || !a->q_sf))
    return fail(NVFP4_ERR_INVALID,
                "decode: give q_fp4 and q_sf together, or neither and a BF16 query to quantise in the kernel");
  if (a->rows > 65535 || a->heads_kv > 65535)
    return fail(NVFP4_ERR_INVALID, "decode: rows and heads_kv are limited to 65535");
  const int64_t dense_packed = (int64_t)128 * a->heads_kv * 64, dense_sf = (int64_t)a->heads_kv * 1024;
  if (a->k_pitch < dense_packed || a->v_pitch < dense_packed || (a->k_pitch % 16) || (a->v_pitch % 16))
    return fail(NVFP4_ERR_INVALID, "decode: packed page pitch must be >= %lld bytes and 16-byte aligned",
                (long long)dense_packed);
  if (a->k_sf_pitch < dense_sf || a->v_sf_pitch < dense_sf || (a->k_sf_pitch % 16) || (a->v_sf_pitch % 16))
    return fail(NVFP4_ERR_INVALID, "decode: scale page pitch must be >= %lld bytes and 16-byte aligned",
                (long long)dense_sf);
  if ((!fused_query && (!aligned16(a->q_fp4) || !aligned16(a->q_sf))) || !aligned16(a->k_packed) || !aligned16(a->k_sf) ||
      !aligned16(a->v_packed) || !aligned16(a->v_sf))
    return fail(NVFP4_ERR_INVALID, "decode: query and page regions must be 16-byte aligned");
  if (a->max_pages < 0 || a->page_table_row_stride < a->max_pages || a->num_pages < 0)
    return fail(NVFP4_ERR_INVALID, "decode: page table extents are inconsistent");
  const bool any_tail = a->tail_key || a->tail_value || a->tail_ids || a->seqused_tail;
  const bool all_tail = a->tail_key && a->tail_value && a->tail_ids && a->seqused_tail;
  if (any_tail && !all_tail)
    return fail(NVFP4_ERR_INVALID, "decode: tail_key, tail_value, tail_ids and seqused_tail go together");
  if (all_tail && (!aligned16(a->tail_key) || !aligned16(a->tail_value) || a->tail_pages < 1))
    return fail(NVFP4_ERR_INVALID, "decode: tail buffers must be 16-byte aligned and non-empty");
  if (a->q_bf16 && (!aligned16(a->q_bf16) || (a->q_bf16_row_stride % 8) || (a->q_bf16_head_stride % 8)))
    return fail(NVFP4_ERR_INVALID, "decode: the BF16 query must keep 16-byte alignment");
  if ((a->o_partial == nullptr) != (a->lse_partial == nullptr))
    return fail(NVFP4_ERR_INVALID, "decode: o_partial and lse_partial go together");
  if (!a->out && !a->o_partial)
    return fail(NVFP4_ERR_INVALID, "decode: neither out nor the partial outputs were given");
  if (a->out_indices && a->num_splits > 1)
    return fail(NVFP4_ERR_INVALID, "decode: out_indices cannot be combined with num_splits > 1");

  nvfp4::DecodeParams p;
  std::memset(&p, 0, sizeof(p));
  p.q_fp4 = static_cast<const uint8_t*>(a->q_fp4);
  p.q_sf = static_cast<const uint8_t*>(a->q_sf);
  p.q_bf16 = static_cast<const uint16_t*>(a->q_bf16);
  p.q_row_stride = a->q_bf16_row_stride;
  p.q_head_stride = a->q_bf16_head_stride;
  p.k_packed = static_cast<const uint8_t*>(a->k_packed); p.k_pitch = a->k_pitch;
  p.k_sf = static_cast<const uint8_t*>(a->k_sf); p.k_sf_pitch = a->k_sf_pitch;
  p.v_packed = static_cast<const uint8_t*>(a->v_packed); p.v_pitch = a->v_pitch;
  p.v_sf = static_cast<const uint8_t*>(a->v_sf); p.v_sf_pitch = a->v_sf_pitch;
  p.num_pages = a->num_pages;
  p.page_table = a->page_table;
  p.page_table_row_stride = a->page_table_row_stride;
  p.max_pages = a->max_pages;
  p.seqused_fp4 = a->seqused_fp4;
  p.tail_key = static_cast<const uint16_t*>(a->tail_key);
  p.tail_value = static_cast<const uint16_t*>(a->tail_value);
  p.tail_pages = a->tail_pages;
  p.tail_ids = a->tail_ids;
  p.seqused_tail = a->seqused_tail;
  p.rows = a->rows; p.heads_q = a->heads_q; p.heads_kv = a->heads_kv;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  p.num_splits = a->num_splits;
  p.status = a->status;
  if (a->flags & ~(NVFP4_DECODE_PROGRAMMATIC_LAUNCH | NVFP4_DECODE_REUSE_WORK_LIST | NVFP4_DECODE_PERSISTENT |
                   NVFP4_DECODE_WIDE_FORM | NVFP4_DECODE_MERGE_IN_LAUNCH))
    return fail(NVFP4_ERR_INVALID, "decode: unknown flag bits %#x", a->flags);
  if ((a->flags & NVFP4_DECODE_MERGE_IN_LAUNCH) && !target_pages)
    return fail(NVFP4_ERR_INVALID, "decode: only nvfp4_decode_balanced merges pieces");
  if ((a->flags & NVFP4_DECODE_REUSE_WORK_LIST) && !target_pages)
    return fail(NVFP4_ERR_INVALID, "decode: only nvfp4_decode_balanced has a work list to reuse");
  p.pdl = (a->flags & NVFP4_DECODE_PROGRAMMATIC_LAUNCH) ? 1 : 0;
  p.wide_hint = (a->flags & NVFP4_DECODE_WIDE_FORM) ? 1 : 0;
  if ((a->append_key == nullptr) != (a->append_value == nullptr))
    return fail(NVFP4_ERR_INVALID, "decode: append_key and append_value go together");
  if (a->append_key) {
    if (!all_tail)
      return fail(NVFP4_ERR_INVALID, "decode: the fused tail append needs the tail arguments");
    if (!aligned16(a->append_key) || !aligned16(a->append_value) || (a->key_shift && !aligned16(a->key_shift)) ||
        (a->append_key_token_stride % 8) || (a->append_value_token_stride % 8) ||
        a->append_key_token_stride < (int64_t)a->heads_kv * 128 ||
        a->append_value_token_stride < (int64_t)a->heads_kv * 128)
      return fail(NVFP4_ERR_INVALID,
                  "decode: the appended tokens must be 16-byte aligned [rows][heads_kv][128] BF16 rows");
    p.append_key = static_cast<const uint16_t*>(a->append_key);
    p.append_value = static_cast<const uint16_t*>(a->append_value);
    p.append_key_stride = a->append_key_token_stride;
    p.append_value_stride = a->append_value_token_stride;
    p.key_shift = static_cast<const uint16_t*>(a->key_shift);
  } else if (a->key_shift) {
    return fail(NVFP4_ERR_INVALID, "decode: key_shift is only read by the fused tail append");
  }

  float* o_part = a->o_partial;
  float* lse_part = a->lse_partial;
  const bool direct = a->num_splits == 1 && a->out != nullptr && !a->o_partial && !target_pages;
  BalancedLayout bal{};
  int64_t capacity = 0;
  if (target_pages) {
    capacity = nvfp4_decode_balanced_capacity(a->rows, a->max_pages, target_pages);
    if (capacity > 65535)
      return fail(NVFP4_ERR_INVALID, "decode_balanced: %lld pieces; raise target_pages", (long long)capacity);
    bal = balanced_layout(a->rows, a->heads_q, capacity);
    if (!a->workspace || a->workspace_bytes < bal.total)
      return fail(NVFP4_ERR_INVALID, "decode_balanced: needs a workspace of %zu bytes, got %zu", bal.total,
                  a->workspace_bytes);
    if (!aligned16(a->workspace)) return fail(NVFP4_ERR_INVALID, "decode: workspace must be 16-byte aligned");
    char* base = static_cast<char*>(a->workspace);
    p.emit_partial = 1;
    p.o_partial = o_part = reinterpret_cast<float*>(base + bal.o_part);
    p.lse_partial = lse_part = reinterpret_cast<float*>(base + bal.lse_part);
    p.work_list = reinterpret_cast<const int4*>(base + bal.work);
    p.work_capacity = (int)capacity;
    // on request the row's pieces are merged by the piece that arrives last instead of a merge launch
    p.list_row_offset = reinterpret_cast<const int32_t*>(base + bal.row_offset);
    p.list_row_count = reinterpret_cast<const int32_t*>(base + bal.row_count);
    p.list_counters = (a->flags & NVFP4_DECODE_MERGE_IN_LAUNCH) ? reinterpret_cast<int*>(base + bal.counters) : nullptr;
    p.out = static_cast<uint16_t*>(a->out);
  } else if (direct) {
    p.emit_partial = 0;
    p.out = static_cast<uint16_t*>(a->out);
    p.out_indices = a->out_indices;
  } else {
    if (!o_part) {
      const size_t need = nvfp4_decode_workspace_bytes(a->rows, a->heads_q, a->num_splits);
      if (!a->workspace || a->workspace_bytes < need)
        return fail(NVFP4_ERR_INVALID, "decode: num_splits=%d needs a workspace of %zu bytes, got %zu",
                    a->num_splits, need, a->workspace_bytes);
      if (!aligned16(a->workspace)) return fail(NVFP4_ERR_INVALID, "decode: workspace must be 16-byte aligned");
      o_part = static_cast<float*>(a->workspace);
      lse_part = o_part + (size_t)a->num_splits * a->rows * a->heads_q * 128;
    }
    p.emit_partial = 1;
    p.o_partial = o_part;
    p.lse_partial = lse_part;
  }

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int impl = a->impl;
  if (impl == NVFP4_IMPL_AUTO) impl = nvfp4::decode_sm100_supports(p) ? NVFP4_IMPL_SM100 : NVFP4_IMPL_GENERIC;
  if (a->flags & NVFP4_DECODE_PERSISTENT) {
    if (!direct || x)
      return fail(NVFP4_ERR_INVALID,
                  "decode: the persistent launch writes the final rows only (num_splits = 1, out given, no "
                  "partial buffers, no exchange, not nvfp4_decode_balanced)");
    if (impl != NVFP4_IMPL_SM100 || !nvfp4::decode_persistent_supports(p))
      return fail(NVFP4_ERR_UNSUPPORTED,
                  "decode: the persistent launch takes 1, 2, 4 or 8 query heads per KV head on the tensor-core "
                  "kernel (see nvfp4_decode_persistent_supported)");
    const size_t need = nvfp4::decode_persistent_workspace_bytes(a->rows, a->heads_q, a->heads_kv);
    if (!a->workspace || a->workspace_bytes < need)
      return fail(NVFP4_ERR_INVALID, "decode: the persistent launch needs a workspace of %zu bytes, got %zu", need,
                  a->workspace_bytes);
    if (!aligned16(a->workspace)) return fail(NVFP4_ERR_INVALID, "decode: workspace must be 16-byte aligned");
    cudaError_t pe = nvfp4::launch_decode_persistent(p, a->workspace, st);
    return pe == cudaSuccess ? NVFP4_OK : cuda_fail(pe, "persistent decode launch");
  }
  if (p.pdl && (impl != NVFP4_IMPL_SM100 || x))
    return fail(NVFP4_ERR_UNSUPPORTED,
                "decode: programmatic launch is carried by the plain tensor-core decode only");
  if (x) {
    if (impl != NVFP4_IMPL_SM100 || !nvfp4::decode_sm100_supports(p))
      return fail(NVFP4_ERR_UNSUPPORTED, "decode_exchange: only the tensor-core kernel carries the exchange");
    if (a->num_splits > 256)
      return fail(NVFP4_ERR_UNSUPPORTED, "decode_exchange: at most 256 local splits");
    if (a->heads_q / a->heads_kv > 8)
      return fail(NVFP4_ERR_UNSUPPORTED,
                  "decode_exchange: at most 8 query heads per KV head (use nvfp4_push_merge for 16 and 32)");
    if (x->world * (a->heads_q / a->heads_kv) > 128)
      return fail(NVFP4_ERR_UNSUPPORTED, "decode_exchange: world * (heads_q / heads_kv) must not exceed 128");
    p.xchg_inbox = x->inbox_ptrs;
    p.xchg_flags = x->flag_ptrs;
    p.xchg_epoch_state = x->epoch_state;
    p.xchg_counters = x->tile_counters;
    p.xchg_out = x->out;
    p.xchg_out_f32 = x->out_is_f32;
    p.xchg_rank = x->rank;
    p.xchg_world = x->world;
  }
  cudaError_t e;
  if (target_pages) {
    if (impl != NVFP4_IMPL_SM100 || !nvfp4::decode_sm100_supports(p) || p.pdl)
      return fail(NVFP4_ERR_UNSUPPORTED,
                  "decode_balanced: carried by the tensor-core kernel only, without programmatic launch");
    char* base = static_cast<char*>(a->workspace);
    e = (a->flags & NVFP4_DECODE_REUSE_WORK_LIST) ? cudaSuccess : nvfp4::launch_balanced_worklist(a->seqused_fp4, (a->tail_key && a->seqused_tail) ? a->seqused_tail : nullptr, a->rows, a->max_pages, target_pages,
                                        reinterpret_cast<int4*>(base + bal.work), (int)capacity,
                                        reinterpret_cast<int32_t*>(base + bal.row_offset),
                                        reinterpret_cast<int32_t*>(base + bal.row_count),
                                        reinterpret_cast<int32_t*>(base + bal.counters), a->rows * a->heads_q,
                                        a->status, st);
    if (e != cudaSuccess) return cuda_fail(e, "work list launch");
  }
  if (impl == NVFP4_IMPL_SM100) {
    if (!nvfp4::decode_sm100_supports(p))
      return fail(NVFP4_ERR_UNSUPPORTED, "decode: the tensor-core kernel takes 1 to 8, 16 or 32 query heads per KV head");
    e = nvfp4::launch_decode_sm100(p, st);
  } else if (impl == NVFP4_IMPL_GENERIC) {
    e = nvfp4::launch_decode_generic(p, st);
  } else {
    return fail(NVFP4_ERR_INVALID, "decode: unknown impl %d", a->impl);
  }
  if (e != cudaSuccess) return cuda_fail(e, "decode launch");

  if (target_pages && !(a->flags & NVFP4_DECODE_MERGE_IN_LAUNCH)) {
    const char* base = static_cast<const char*>(a->workspace);
    e = nvfp4::launch_lse_merge_ranges(o_part, lse_part, reinterpret_cast<const int32_t*>(base + bal.row_offset),
                                       reinterpret_cast<const int32_t*>(base + bal.row_count), a->rows,
                                       a->heads_q, a->out, st);
    if (e != cudaSuccess) return cuda_fail(e, "lse_merge launch");
  } else if (!target_pages && !direct && a->out) {
    e = nvfp4::launch_lse_merge(o_part, (int64_t)a->rows * a->heads_q * 128, lse_part,
                                (int64_t)a->rows * a->heads_q, nullptr, nullptr, a->num_splits,
                                a->rows, a->heads_q, a->out, 0, a->out_indices, nullptr, st);
    if (e != cudaSuccess) return cuda_fail(e, "lse_merge launch");
  }
  return NVFP4_OK;
}

int nvfp4_lse_merge(const float* o_parts, int64_t o_split_stride, const float* lse_parts,
                    int64_t lse_split_stride, int num_splits, int rows, int heads_q, void* out,
                    int out_is_f32, const int32_t* out_indices, float* lse_out, void* stream) {
  if (rows < 0 || heads_q < 1 || num_splits < 1)
    return fail(NVFP4_ERR_INVALID, "lse_merge: bad extents (%d rows, %d heads, %d splits)", rows, heads_q, num_splits);
  if (rows == 0) return NVFP4_OK;
  if (!o_parts || !lse_parts || (!out && !lse_out)) return fail(NVFP4_ERR_INVALID, "lse_merge: null argument");
  if (rows > 65535) return fail(NVFP4_ERR_INVALID, "lse_merge: too many rows");
  cudaError_t e = nvfp4::launch_lse_merge(o_parts, o_split_stride, lse_parts, lse_split_stride, nullptr,
                                          nullptr, num_splits, rows, heads_q, out, out_is_f32,
                                          out_indices, lse_out, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "lse_merge launch");
}

int nvfp4_lse_merge_ptrs(const float* const* o_part_ptrs, const float* const* lse_part_ptrs,
                         int num_splits, int rows, int heads_q, void* out, int out_is_f32,
                         const int32_t* out_indices, float* lse_out, void* stream) {
  if (rows < 0 || heads_q < 1 || num_splits < 1)
    return fail(NVFP4_ERR_INVALID, "lse_merge_ptrs: bad extents (%d rows, %d heads, %d splits)", rows, heads_q, num_splits);
  if (rows == 0) return NVFP4_OK;
  if (!o_part_ptrs || !lse_part_ptrs || (!out && !lse_out))
    return fail(NVFP4_ERR_INVALID, "lse_merge_ptrs: null argument");
  if (rows > 65535) return fail(NVFP4_ERR_INVALID, "lse_merge_ptrs: too many rows");
  cudaError_t e = nvfp4::launch_lse_merge(nullptr, 0, nullptr, 0, o_part_ptrs, lse_part_ptrs, num_splits,
                                          rows, heads_q, out, out_is_f32, out_indices, lse_out,
                                          static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "lse_merge_ptrs launch");
}

namespace {
int control_call(const int32_t* block_table, int64_t block_table_stride, int block_table_columns,
                 const int32_t* seq_lens, const int32_t* query_start_loc, int32_t* slot_keys,
                 int32_t* slot_last_seq, int64_t* slot_last_seen, int64_t* step, int32_t* row_to_slot,
                 int32_t* token_to_slot, int32_t* seqused_fp4, int32_t* seqused_residual,
                 int32_t* promotion_source_tokens, int32_t* promotion_pages, int32_t* error_code,
                 int num_reqs, int num_actual_tokens, int num_slots, bool with_list, int decode_rows,
                 int max_pages, int target_pages, int heads_q, void* workspace, size_t workspace_bytes,
                 void* stream) {
  if (num_slots < 1 || num_slots > 128)
    return fail(NVFP4_ERR_INVALID, "control_step: the slot table holds 1 to 128 slots, got %d", num_slots);
  if (num_reqs < 0 || num_reqs > num_slots)
    return fail(NVFP4_ERR_INVALID, "control_step: %d rows exceeds the %d tail slots", num_reqs, num_slots);
  if (num_actual_tokens < 0 || block_table_columns < 1)
    return fail(NVFP4_ERR_INVALID, "control_step: bad extents");
  if (!block_table || !seq_lens || !query_start_loc || !slot_keys || !slot_last_seq || !slot_last_seen ||
      !step || !row_to_slot || !token_to_slot || !seqused_fp4 || !seqused_residual ||
      !promotion_source_tokens || !promotion_pages || !error_code)
    return fail(NVFP4_ERR_INVALID, "control_step: null argument");
  nvfp4::ControlArgs a{block_table, block_table_stride, block_table_columns, seq_lens, query_start_loc,
                       slot_keys, slot_last_seq, slot_last_seen, step, row_to_slot, token_to_slot,
                       seqused_fp4, seqused_residual, promotion_source_tokens, promotion_pages, error_code,
                       num_reqs, num_actual_tokens, num_slots, nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0, 0};
  if (with_list) {
    if (decode_rows < 1 || decode_rows > num_reqs || max_pages < 0 || target_pages < 1 || heads_q < 1)
      return fail(NVFP4_ERR_INVALID,
                  "control_step_balanced: needs 1 <= decode_rows <= num_reqs, max_pages >= 0, target_pages >= 1");
    const int64_t capacity = nvfp4_decode_balanced_capacity(decode_rows, max_pages, target_pages);
    if (capacity > 65535)
      return fail(NVFP4_ERR_INVALID, "control_step_balanced: %lld pieces; raise target_pages", (long long)capacity);
    const BalancedLayout bal = balanced_layout(decode_rows, heads_q, capacity);
    if (!workspace || workspace_bytes < bal.total || !aligned16(workspace))
      return fail(NVFP4_ERR_INVALID, "control_step_balanced: needs a 16-byte aligned workspace of %zu bytes, got %zu",
                  bal.total, workspace_bytes);
    char* base = static_cast<char*>(workspace);
    a.work = reinterpret_cast<int4*>(base + bal.work);
    a.work_row_offset = reinterpret_cast<int32_t*>(base + bal.row_offset);
    a.work_row_count = reinterpret_cast<int32_t*>(base + bal.row_count);
    a.work_counters = reinterpret_cast<int32_t*>(base + bal.counters);
    a.work_counter_words = decode_rows * heads_q;
    a.work_rows = decode_rows;
    a.work_capacity = (int)capacity;
    a.work_max_pages = max_pages;
    a.work_target_pages = target_pages;
  }
  cudaError_t e = nvfp4::launch_control(a, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "control_step launch");
}
}  // namespace

int nvfp4_control_step(const int32_t* block_table, int64_t block_table_stride, int block_table_columns,
                       const int32_t* seq_lens, const int32_t* query_start_loc, int32_t* slot_keys,
                       int32_t* slot_last_seq, int64_t* slot_last_seen, int64_t* step, int32_t* row_to_slot,
                       int32_t* token_to_slot, int32_t* seqused_fp4, int32_t* seqused_residual,
                       int32_t* promotion_source_tokens, int32_t* promotion_pages, int32_t* error_code,
                       int num_reqs, int num_actual_tokens, int num_slots, void* stream) {
  return control_call(block_table, block_table_stride, block_table_columns, seq_lens, query_start_loc, slot_keys,
                      slot_last_seq, slot_last_seen, step, row_to_slot, token_to_slot, seqused_fp4,
                      seqused_residual, promotion_source_tokens, promotion_pages, error_code, num_reqs,
                      num_actual_tokens, num_slots, false, 0, 0, 0, 0, nullptr, 0, stream);
}

int nvfp4_control_step_balanced(const int32_t* block_table, int64_t block_table_stride, int block_table_columns,
                                const int32_t* seq_lens, const int32_t* query_start_loc, int32_t* slot_keys,
                                int32_t* slot_last_seq, int64_t* slot_last_seen, int64_t* step,
                                int32_t* row_to_slot, int32_t* token_to_slot, int32_t* seqused_fp4,
                                int32_t* seqused_residual, int32_t* promotion_source_tokens,
                                int32_t* promotion_pages, int32_t* error_code, int num_reqs,
                                int num_actual_tokens, int num_slots, int decode_rows, int max_pages,
                                int target_pages, int heads_q, void* workspace, size_t workspace_bytes,
                                void* stream) {
  return control_call(block_table, block_table_stride, block_table_columns, seq_lens, query_start_loc, slot_keys,
                      slot_last_seq, slot_last_seen, step, row_to_slot, token_to_slot, seqused_fp4,
                      seqused_residual, promotion_source_tokens, promotion_pages, error_code, num_reqs,
                      num_actual_tokens, num_slots, true, decode_rows, max_pages, target_pages, heads_q,
                      workspace, workspace_bytes, stream);
}

int nvfp4_work_table(const int32_t* query_start_loc, const int32_t* seqused_fp4, const int32_t* row_to_slot,
                     const int32_t* block_table, int64_t block_table_stride, int32_t* source_tokens,
                     int32_t* destination_pages, int num_reqs, int columns_per_row, void* stream) {
  if (num_reqs < 0 || columns_per_row < 0 || num_reqs > 65535)
    return fail(NVFP4_ERR_INVALID, "work_table: bad extents");
  if (num_reqs == 0 || columns_per_row == 0) return NVFP4_OK;
  if (!query_start_loc || !seqused_fp4 || !row_to_slot || !block_table || !source_tokens || !destination_pages)
    return fail(NVFP4_ERR_INVALID, "work_table: null argument");
  cudaError_t e = nvfp4::launch_work_table(query_start_loc, seqused_fp4, row_to_slot, block_table,
                                           block_table_stride, source_tokens, destination_pages, num_reqs,
                                           columns_per_row, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "work_table launch");
}

int nvfp4_peer_merge(const float* const* o_part_ptrs, const float* const* lse_part_ptrs,
                     int32_t* const* flag_ptrs, int rank, int world, int epoch, int32_t* epoch_state,
                     int rows, int heads_q, void* out, int out_is_f32, uint32_t* status, void* stream) {
  if (world < 1 || world > 128 || rank < 0 || rank >= world)
    return fail(NVFP4_ERR_INVALID, "peer_merge: rank %d of %d is out of range (at most 128 ranks)", rank, world);
  if (rows < 0 || heads_q < 1) return fail(NVFP4_ERR_INVALID, "peer_merge: bad extents");
  if (rows == 0) return NVFP4_OK;
  if (!o_part_ptrs || !lse_part_ptrs || !flag_ptrs || !out)
    return fail(NVFP4_ERR_INVALID, "peer_merge: null argument");
  if (rows > 65535) return fail(NVFP4_ERR_INVALID, "peer_merge: too many rows");
  cudaError_t e = nvfp4::launch_peer_merge(o_part_ptrs, lse_part_ptrs, flag_ptrs, rank, world, epoch,
                                           epoch_state, rows, heads_q, out, out_is_f32, status,
                                           static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "peer_merge launch");
}

int nvfp4_push_merge(const float* o_local, int64_t o_split_stride, const float* lse_local,
                     int64_t lse_split_stride, int local_splits, float* const* inbox_ptrs,
                     int32_t* const* flag_ptrs, int rank, int world, int epoch, int32_t* epoch_state,
                     int rows, int heads_q, void* out, int out_is_f32, uint32_t* status, void* stream) {
  if (world < 1 || world > 128 || rank < 0 || rank >= world)
    return fail(NVFP4_ERR_INVALID, "push_merge: rank %d of %d is out of range (at most 128 ranks)", rank, world);
  if (rows < 0 || heads_q < 1 || local_splits < 1) return fail(NVFP4_ERR_INVALID, "push_merge: bad extents");
  if (rows == 0) return NVFP4_OK;
  if (!o_local || !lse_local || !inbox_ptrs || !flag_ptrs || !out)
    return fail(NVFP4_ERR_INVALID, "push_merge: null argument");
  if (rows > 65535) return fail(NVFP4_ERR_INVALID, "push_merge: too many rows");
  cudaError_t e = nvfp4::launch_push_merge(o_local, o_split_stride, lse_local, lse_split_stride, local_splits,
                                           inbox_ptrs, flag_ptrs, rank, world, epoch, epoch_state, rows,
                                           heads_q, out, out_is_f32, status, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? NVFP4_OK : cuda_fail(e, "push_merge launch");
}

size_t nvfp4_push_merge_inbox_floats(int world, int rows, int heads_q) {
  if (world < 1 || rows < 0 || heads_q < 1) return 0;
  return (size_t)2 * world * rows * heads_q * 132;
}

}  // extern "C"
