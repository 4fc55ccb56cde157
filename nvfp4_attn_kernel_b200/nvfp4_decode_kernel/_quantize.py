"""Query quantisation to NVFP4.

Same contract as the reference project's ``quantize_query``
(``src/nvfp4_decode_kernel/_quantize.py:14-117``): packed query
``[rows, 1, heads, 64]`` (``float4_e2m1fn_x2``) and a uint8 scale view of shape
``(32, 4, 1, 4, 2, heads_kv, rows)`` over storage ``[rows, 1, heads, 2, 32, 4, 4]``.
"""

from __future__ import annotations

import torch

from .. import _lib
from .quantize_kv_kernel import quantize_key_pages, quantize_value_pages  # noqa: F401  (re-export)

PAGE_SIZE = 128


def query_scale_view(storage: torch.Tensor, rows: int, heads: int, heads_kv: int) -> torch.Tensor:
    """The decode kernel's view of the query scale bytes."""
    rest_k = storage.shape[3]
    row_stride = heads * rest_k * 512
    return storage.as_strided(
        (32, 4, 1, 4, rest_k, heads_kv, rows),
        (16, 4, row_stride, 1, 512, rest_k * 512, row_stride),
    )


def quantize_query(
    query: torch.Tensor,
    *,
    row_indices: torch.Tensor | None = None,
    query_padded_out: torch.Tensor | None = None,
    heads_kv: int | None = None,
    query_fp4_scratch: torch.Tensor | None = None,
    query_scales_scratch: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantise BF16 decode rows; see the module docstring for the layouts.

    A caller-owned scale buffer must arrive zeroed once: only the
    ``heads // heads_kv`` live slots of each KV head's 128-slot scale block are
    written.  ``query_padded_out`` (``[>= rows, 128, heads, head_dim]`` BF16)
    receives the BF16 row in ``[row, 0, head, :]``.
    """
    if query.dtype is not torch.bfloat16 or not query.is_cuda:
        raise ValueError("query must be a BF16 CUDA tensor")
    if query.ndim != 3 or query.stride(-1) != 1:
        raise ValueError("query must have shape [rows, heads, head_dim]")
    if row_indices is not None and (
        row_indices.dtype is not torch.int32
        or not row_indices.is_cuda
        or row_indices.ndim != 1
        or not row_indices.is_contiguous()
    ):
        raise ValueError("row_indices must be contiguous 1-D INT32 CUDA")
    _, heads, head_dim = query.shape
    heads_kv = heads if heads_kv is None else heads_kv
    if heads_kv < 1 or heads % heads_kv:
        raise ValueError("query heads must be divisible by heads_kv")
    if head_dim != 128:
        raise ValueError("query head_dim must be 128")
    rows = query.shape[0] if row_indices is None else row_indices.shape[0]
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

    packed = (
        torch.empty(rows, 1, heads, head_dim // 2, dtype=torch.uint8, device=query.device)
        if query_fp4_scratch is None
        else query_fp4_scratch[:rows]
    )
    storage = (
        torch.zeros(rows, 1, heads, head_dim // 64, 32, 4, 4, dtype=torch.uint8,
                    device=query.device)
        if query_scales_scratch is None
        else query_scales_scratch[:rows]
    )
    if rows:
        with torch.cuda.device(query.device):
            _lib.check(
                _lib.load().nvfp4_quantize_q(
                    query.data_ptr(),
                    query.stride(0),
                    query.stride(1),
                    _lib.ptr(row_indices),
                    packed.data_ptr(),
                    storage.data_ptr(),
                    _lib.ptr(query_padded_out),
                    rows,
                    heads,
                    heads_kv,
                    torch.cuda.current_stream().cuda_stream,
                )
            )
    return packed.view(torch.float4_e2m1fn_x2), query_scale_view(storage, rows, heads, heads_kv)
