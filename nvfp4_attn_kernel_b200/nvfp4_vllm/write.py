"""Placing a step's K/V into the NVFP4 pages and the BF16 tail.

Same functions and arguments as the reference project's ``src/nvfp4_vllm/write.py``
(``reset_new_request_tails`` :182-215, ``PageWorkTable`` :218-277, ``write_kv`` :280-337).
Every decision is taken on the device; launch shapes come from host integers only.
``write_kv`` additionally takes ``key_shift``: the per-channel shift is then subtracted inside
the page quantiser and the tail copy instead of by a separate ``torch.sub``.
"""

from __future__ import annotations

import torch

from .. import _lib
PAGE_SIZE = 128


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def reset_new_request_tails(*, tail_key: torch.Tensor, tail_value: torch.Tensor,
                            query_start_loc: torch.Tensor, seq_lens: torch.Tensor,
                            row_to_slot: torch.Tensor) -> None:
    """Zero every layer's tail page of the rows that start a request this step
    (``seq_len <= query_len``).  ``tail_*``: ``[layers, slots, 128, heads, head_dim]``."""
    layers, _, _, heads, _ = tail_key.shape
    with torch.cuda.device(tail_key.device):
        _lib.check(_lib.load().nvfp4_tail_reset(
            tail_key.data_ptr(), tail_value.data_ptr(), tail_key.stride(0), tail_key.stride(1),
            layers, query_start_loc.data_ptr(), seq_lens.data_ptr(), row_to_slot.data_ptr(),
            seq_lens.shape[0], heads, _stream(tail_key.device)))


def accumulate_key_sum(key: torch.Tensor, key_sum: torch.Tensor) -> None:
    """``key_sum += key.double().sum(dim=0)`` in one launch: the accumulation the key-shift
    calibration runs per layer and step (reference: ``NVFP4Impl.do_kv_cache_update``,
    ``src/nvfp4_vllm/impl.py:137-144``).  ``key``: ``[tokens, heads, 128]`` BF16 with dense
    tokens (any token stride that keeps 16-byte alignment); ``key_sum``: ``[heads, 128]`` FP64,
    contiguous, on the same device."""
    tokens, heads, dim = key.shape
    if key.dtype is not torch.bfloat16 or dim != 128 or key.stride(2) != 1 or key.stride(1) != dim:
        raise ValueError("key must be BF16 [tokens, heads, 128] with dense tokens")
    if key_sum.dtype is not torch.float64 or tuple(key_sum.shape) != (heads, dim) or \
            not key_sum.is_contiguous() or key_sum.device != key.device:
        raise ValueError("key_sum must be a contiguous FP64 [heads, 128] tensor on key's device")
    with torch.cuda.device(key.device):
        _lib.check(_lib.load().nvfp4_key_sum_accumulate(
            key.data_ptr(), key.stride(0) if tokens > 1 else heads * dim, tokens, heads,
            key_sum.data_ptr(), _stream(key.device)))


class PageWorkTable:
    """Which full pages this step must quantise: a dense rows x columns rectangle, -1 = none."""

    def __init__(self, *, max_num_seqs: int, max_num_batched_tokens: int, device) -> None:
        self.max_num_seqs = max_num_seqs
        self.max_columns = max_num_batched_tokens // PAGE_SIZE + 1
        capacity = max_num_seqs * self.max_columns
        self.source_tokens = torch.empty(capacity, dtype=torch.int32, device=device)
        self.destination_pages = torch.full((capacity,), -1, dtype=torch.int32, device=device)

    def build(self, *, query_start_loc: torch.Tensor, seqused_fp4: torch.Tensor,
              row_to_slot: torch.Tensor, block_table: torch.Tensor, num_reqs: int,
              max_query_len: int) -> tuple[torch.Tensor, torch.Tensor]:
        if max_query_len <= 1:   # a pure decode step brings no full page
            return self.source_tokens[:0], self.destination_pages[:0]
        columns = min(max_query_len // PAGE_SIZE + 1, self.max_columns, block_table.shape[1])
        items = num_reqs * columns
        with torch.cuda.device(block_table.device):
            _lib.check(_lib.load().nvfp4_work_table(
                query_start_loc.data_ptr(), seqused_fp4.data_ptr(), row_to_slot.data_ptr(),
                block_table.data_ptr(), block_table.stride(0), self.source_tokens.data_ptr(),
                self.destination_pages.data_ptr(), num_reqs, columns, _stream(block_table.device)))
        return self.source_tokens[:items], self.destination_pages[:items]


def write_kv(*, key: torch.Tensor, value: torch.Tensor, key_pages_fp4: torch.Tensor,
             key_scales: torch.Tensor, value_pages_fp4: torch.Tensor, value_scales: torch.Tensor,
             tail_key: torch.Tensor, tail_value: torch.Tensor, source_tokens: torch.Tensor,
             destination_pages: torch.Tensor, query_start_loc: torch.Tensor,
             seq_lens: torch.Tensor, seqused_fp4: torch.Tensor, row_to_slot: torch.Tensor,
             num_actual_tokens: int, key_shift: torch.Tensor | None = None) -> None:
    """One layer's K/V of this step: full pages quantised into their blocks, the rest copied
    to the row's tail slot.  ``tail_*`` is this layer's ``[slots, 128, heads, head_dim]``.
    ONE launch (``nvfp4_write_kv``) where the reference issues two page quantisers and a tail
    copy."""
    key = key[:num_actual_tokens]
    value = value[:num_actual_tokens]
    work = destination_pages.numel()
    heads = tail_key.shape[2]
    if key.dtype is not torch.bfloat16 or value.dtype is not torch.bfloat16:
        raise ValueError("key and value must be BF16")
    if key.ndim != 3 or key.stride(2) != 1 or key.stride(1) != key.shape[2] or \
            value.ndim != 3 or value.stride(2) != 1 or value.stride(1) != value.shape[2]:
        raise ValueError("key and value must be [tokens, heads, head_dim] with contiguous tokens")
    if work:
        if source_tokens.numel() != work:
            raise ValueError("source_tokens and destination_pages must have the same length")
        k_pitch = key_pages_fp4.stride(0) * key_pages_fp4.element_size()
        v_pitch = value_pages_fp4.stride(0) * value_pages_fp4.element_size()
        regions = (key_pages_fp4.data_ptr(), k_pitch, key_scales.data_ptr(), key_scales.stride(0),
                   value_pages_fp4.data_ptr(), v_pitch, value_scales.data_ptr(), value_scales.stride(0),
                   source_tokens.data_ptr(), destination_pages.data_ptr())
    else:
        regions = (None, 0, None, 0, None, 0, None, 0, None, None)
    with torch.cuda.device(key.device):
        _lib.check(_lib.load().nvfp4_write_kv(
            key.data_ptr(), value.data_ptr(), key.stride(0), value.stride(0), _lib.ptr(key_shift),
            *regions, work, tail_key.data_ptr(), tail_value.data_ptr(), tail_key.stride(0),
            query_start_loc.data_ptr(), seq_lens.data_ptr(), seqused_fp4.data_ptr(),
            row_to_slot.data_ptr(), num_actual_tokens, seq_lens.shape[0], heads, _stream(key.device)))
