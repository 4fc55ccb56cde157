"""LSE-weighted merge of split-KV partial results.

Python face of ``nvfp4_lse_merge``; argument meaning follows the reference
project's ``flash_attn_combine`` (``src/nvfp4_decode_kernel/split_k_combine.py:694-768``):
``out_partial`` is ``[splits, rows, 1, heads, 128]`` fp32 (normalised partial
outputs), ``lse_partial`` is ``[splits, rows, 1, heads]`` fp32 natural-log LSEs
(``-inf`` = empty split).  Work is issued on the current stream of the
partials' device.
"""

from __future__ import annotations

import torch

from .. import _lib


def flash_attn_combine(out_partial, lse_partial, out=None, out_dtype=None, return_lse=True):
    if out_partial.dtype is not torch.float32 or lse_partial.dtype is not torch.float32:
        raise ValueError("partials must be FP32")
    if out_partial.ndim != 5 or out_partial.shape[-1] != 128:
        raise ValueError("out_partial must have shape [splits, rows, seqlen, heads, 128]")
    splits, rows, seqlen, heads, dim = out_partial.shape
    if tuple(lse_partial.shape) != (splits, rows, seqlen, heads):
        raise ValueError("lse_partial must have shape [splits, rows, seqlen, heads]")
    if not out_partial.is_contiguous():
        raise ValueError("out_partial must be contiguous")
    if out_dtype is None:
        out_dtype = out_partial.dtype if out is None else out.dtype
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("out_dtype must be BF16 or FP32")
    if out is None:
        out = torch.empty(rows, seqlen, heads, dim, dtype=out_dtype, device=out_partial.device)
    elif out.dtype is not out_dtype or tuple(out.shape) != (rows, seqlen, heads, dim) or not out.is_contiguous():
        raise ValueError("out must be contiguous with shape [rows, seqlen, heads, 128]")
    lse_c = lse_partial.contiguous()
    lse = (
        torch.empty(rows, seqlen, heads, dtype=torch.float32, device=out_partial.device)
        if return_lse
        else None
    )
    with torch.cuda.device(out_partial.device):
        _lib.check(
            _lib.load().nvfp4_lse_merge(
                out_partial.data_ptr(),
                rows * seqlen * heads * dim,
                lse_c.data_ptr(),
                rows * seqlen * heads,
                splits,
                rows * seqlen,
                heads,
                out.data_ptr(),
                1 if out_dtype is torch.float32 else 0,
                None,
                _lib.ptr(lse),
                torch.cuda.current_stream(out_partial.device).cuda_stream,
            )
        )
    return out, lse
