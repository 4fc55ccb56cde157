"""Query quantisation into buffers the caller already owns.

Counterpart of the reference project's ``quantize_decode_q_to_padded_fp4``
(``src/nvfp4_decode_kernel/quantize_q_kernel.py:304-505``): same arguments, same refusals, the
work done by ``nvfp4_quantize_q`` of the C ABI.  ``query_scales_out`` is the seven-axis view
``(32, 4, 1, 4, 2, heads_kv, rows)`` over ``[rows, 1, heads, 2, 32, 4, 4]`` bytes that
:func:`nvfp4_decode_kernel._quantize.query_scale_view` builds; only the live slots of every KV
head's scale block are written, so the storage must have been zeroed once.
"""

from __future__ import annotations

import torch

from .. import _lib

PAGE_SIZE = 128


def quantize_decode_q_to_padded_fp4(
    query: torch.Tensor,
    query_fp4_out: torch.Tensor,
    query_scales_out: torch.Tensor,
    query_padded_out: torch.Tensor | None = None,
    *,
    row_indices: torch.Tensor | None = None,
    heads_kv: int | None = None,
) -> None:
    """Quantise the selected BF16 query rows into ``query_fp4_out`` / ``query_scales_out`` and,
    when given, copy each BF16 row into ``query_padded_out[row, 0]``."""
    if query.dtype is not torch.bfloat16 or not query.is_cuda:
        raise ValueError("query must be a BF16 CUDA tensor")
    if query.ndim != 3 or query.stride(-1) != 1:
        raise ValueError("query must have shape [rows, heads, head_dim]")
    source_rows, heads, head_dim = query.shape
    heads_kv = heads if heads_kv is None else heads_kv
    if heads_kv < 1 or heads % heads_kv:
        raise ValueError("query heads must be divisible by heads_kv")
    if head_dim != 128:
        raise ValueError("query head_dim must be 128")
    rows = query_fp4_out.shape[0]
    if row_indices is None:
        if source_rows != rows:
            raise ValueError("query rows must match output rows")
    elif (
        row_indices.dtype is not torch.int32
        or row_indices.device != query.device
        or not row_indices.is_contiguous()
        or tuple(row_indices.shape) != (rows,)
    ):
        raise ValueError("row_indices must be contiguous INT32 CUDA with shape [rows]")
    fp4_shape = (rows, 1, heads, head_dim // 2)
    if (
        tuple(query_fp4_out.shape) != fp4_shape
        or query_fp4_out.dtype is not torch.float4_e2m1fn_x2
        or query_fp4_out.device != query.device
        or not query_fp4_out.is_contiguous()
    ):
        raise ValueError(f"query_fp4_out must have shape {fp4_shape}")
    sf_shape = (32, 4, 1, 4, head_dim // 64, heads_kv, rows)
    row_stride = heads * (head_dim // 64) * 512
    if (
        tuple(query_scales_out.shape) != sf_shape
        or query_scales_out.dtype is not torch.uint8
        or query_scales_out.device != query.device
    ):
        raise ValueError(f"query_scales_out must have shape {sf_shape}")
    strides = query_scales_out.stride()
    want = (16, 4, None, 1, 512, 1024, row_stride)
    if any(w is not None and s != w and n > 1 for s, w, n in zip(strides, want, sf_shape)):
        raise ValueError(f"query_scales_out must be the scale view with strides {want}, got {strides}")
    if query_padded_out is not None and (
        query_padded_out.ndim != 4
        or query_padded_out.shape[0] < rows
        or tuple(query_padded_out.shape[1:]) != (PAGE_SIZE, heads, head_dim)
        or query_padded_out.dtype is not torch.bfloat16
        or query_padded_out.device != query.device
        or not query_padded_out.is_contiguous()
    ):
        raise ValueError(
            f"query_padded_out must have shape [at least {rows}, {PAGE_SIZE}, {heads}, {head_dim}]"
        )
    if not rows:
        return
    with torch.cuda.device(query.device):
        _lib.check(
            _lib.load().nvfp4_quantize_q(
                query.data_ptr(),
                query.stride(0),
                query.stride(1),
                _lib.ptr(row_indices),
                query_fp4_out.data_ptr(),
                query_scales_out.data_ptr(),
                _lib.ptr(query_padded_out),
                rows,
                heads,
                heads_kv,
                torch.cuda.current_stream().cuda_stream,
            )
        )
