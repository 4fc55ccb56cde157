"""K/V page quantisers (BF16 -> packed E2M1 + E4M3 block-16 scales).

Same entry points and tensor contracts as the reference project's
``src/nvfp4_decode_kernel/quantize_kv_kernel.py`` (:661-822); the device work
is done by ``nvfp4_quantize_kv_pages`` of the C ABI.  On top of the reference's
arguments every function takes an optional ``key_shift`` / stream-ordered fused
shift (K only): ``k <- bf16(k - shift)`` before quantising, which replaces the
separate ``torch.sub`` of ``nvfp4_vllm/impl.py:152``.
"""

from __future__ import annotations

import torch

from .. import _lib

PAGE_SIZE = 128
HEAD_DIM = 128
SF_VEC_SIZE = 16
_ATOM_BYTES = 512


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dense_strides(shape: tuple[int, ...]) -> tuple[int, ...]:
    strides, step = [], 1
    for extent in reversed(shape):
        strides.append(step)
        step *= extent
    return tuple(reversed(strides))


def scale_view(storage: torch.Tensor, pages: int, heads: int, page_pitch: int | None = None,
               offset: int = 0) -> torch.Tensor:
    """Seven-axis view ``[pages, 32, 4, 1, 4, 2, heads]`` over scale bytes."""
    head_stride = 2 * _ATOM_BYTES
    pitch = heads * head_stride if page_pitch is None else page_pitch
    return storage.as_strided(
        (pages, 32, 4, 1, 4, 2, heads),
        (pitch, 16, 4, head_stride, 1, _ATOM_BYTES, head_stride),
        offset,
    )


def _check_pages(pages: torch.Tensor, name: str) -> tuple[int, int]:
    if (
        pages.dtype is not torch.bfloat16
        or not pages.is_cuda
        or pages.ndim != 4
        or not pages.is_contiguous()
    ):
        raise ValueError(
            f"{name} must be contiguous BF16 CUDA with shape [pages, 128, heads, 128]"
        )
    count, page, heads, dim = pages.shape
    if count < 1 or page != PAGE_SIZE or dim != HEAD_DIM:
        raise ValueError(f"{name} must have shape [pages, 128, heads, 128]")
    return count, heads


def _check_tokens(tokens: torch.Tensor, name: str) -> int:
    if (
        tokens.dtype is not torch.bfloat16
        or not tokens.is_cuda
        or tokens.ndim != 3
        or tokens.shape[2] != HEAD_DIM
        or tokens.stride(2) != 1
        or tokens.stride(1) != HEAD_DIM
    ):
        raise ValueError(
            f"{name} must be BF16 CUDA of shape [tokens, heads, 128], dense within a token"
        )
    return tokens.shape[1]


def _check_destination(packed: torch.Tensor, scales: torch.Tensor, heads: int,
                       inner: tuple[int, ...]) -> None:
    if (
        packed.dtype is not torch.uint8
        or not packed.is_cuda
        or tuple(packed.shape[1:]) != inner
        or packed.stride()[1:] != _dense_strides(inner)
    ):
        raise ValueError(
            f"packed destination must be uint8 CUDA pages of {inner}, dense within a page"
        )
    want_shape = (32, 4, 1, 4, 2, heads)
    want_strides = (16, 4, 2 * _ATOM_BYTES, 1, _ATOM_BYTES, 2 * _ATOM_BYTES)
    if (
        scales.element_size() != 1
        or not scales.is_cuda
        or tuple(scales.shape[1:]) != want_shape
        or scales.stride()[1:] != want_strides
    ):
        raise ValueError("scale destination must use the quantizer's own scale layout")
    if packed.shape[0] != scales.shape[0]:
        raise ValueError("packed and scale destinations must have equal pages")


def _check_indices(index: torch.Tensor | None) -> None:
    if index is None:
        return
    if (
        index.dtype is not torch.int32
        or not index.is_cuda
        or index.ndim != 1
        or not index.is_contiguous()
    ):
        raise ValueError("work indices must be contiguous 1-D int32 CUDA")


def _check_bases(bases: torch.Tensor | None) -> int:
    if bases is None:
        return 1
    if (
        bases.dtype is not torch.int64
        or not bases.is_cuda
        or bases.ndim != 2
        or bases.shape[0] != 2
        or bases.shape[1] < 1
        or not bases.is_contiguous()
    ):
        raise ValueError(
            "destination_bases must be a contiguous int64 CUDA tensor of shape "
            "[2, layers] holding the packed and scale base addresses"
        )
    return bases.shape[1]


def _check_shift(key_shift: torch.Tensor | None, layers: int, heads: int,
                 device: torch.device) -> None:
    if key_shift is None:
        return
    ok_shapes = ((layers, heads, HEAD_DIM),) + (((heads, HEAD_DIM),) if layers == 1 else ())
    if (
        key_shift.dtype is not torch.bfloat16
        or key_shift.device != device
        or tuple(key_shift.shape) not in ok_shapes
        or not key_shift.is_contiguous()
    ):
        raise ValueError(
            f"key_shift must be contiguous BF16 on {device} shaped [layers, heads, 128]"
        )


def _launch(which: int, tokens: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor,
            source_tokens, destination_pages, destination_bases, key_shift, heads: int,
            work: int) -> None:
    layers = _check_bases(destination_bases)
    _check_indices(source_tokens)
    _check_indices(destination_pages)
    if tokens.shape[0] % layers:
        raise ValueError(
            f"a source of {tokens.shape[0]} tokens does not divide into {layers} layers"
        )
    _check_shift(key_shift, layers, heads, tokens.device)
    packed_bases = sf_bases = None
    if destination_bases is not None:
        packed_bases = destination_bases[0].data_ptr()
        sf_bases = destination_bases[1].data_ptr()
    lib = _lib.load()
    with torch.cuda.device(tokens.device):
        _lib.check(
            lib.nvfp4_quantize_kv_pages(
                which,
                tokens.data_ptr(),
                tokens.stride(0),
                _lib.ptr(key_shift),
                packed.data_ptr(),
                packed.stride(0) * packed.element_size(),
                scales.data_ptr(),
                scales.stride(0),
                _lib.ptr(source_tokens),
                _lib.ptr(destination_pages),
                packed_bases,
                sf_bases,
                work,
                layers,
                tokens.shape[0] // layers,
                heads,
                _stream(),
            )
        )


def quantize_key_tokens_into(
    key_tokens: torch.Tensor,
    key_pages_fp4: torch.Tensor,
    key_scales: torch.Tensor,
    source_tokens: torch.Tensor,
    destination_pages: torch.Tensor,
    destination_bases: torch.Tensor | None = None,
    *,
    key_shift: torch.Tensor | None = None,
) -> None:
    """Quantise K pages out of a flat token buffer into a paged destination.

    Work item ``w`` reads the 128 tokens that start at ``source_tokens[w]`` and
    writes page ``destination_pages[w]`` (negative = skip).  The destinations may
    be strided along their page axis.  ``destination_bases`` (int64 ``[2, layers]``:
    packed and scale base addresses) repeats the work once per layer against a
    source that stacks the layers along the token axis.
    """
    heads = _check_tokens(key_tokens, "key_tokens")
    _check_destination(key_pages_fp4, key_scales, heads, (PAGE_SIZE, heads, HEAD_DIM // 2))
    work = source_tokens.numel()
    if destination_pages.numel() != work:
        raise ValueError("source_tokens and destination_pages must agree")
    _launch(0, key_tokens, key_pages_fp4, key_scales, source_tokens, destination_pages,
            destination_bases, key_shift, heads, work)


def quantize_value_tokens_into(
    value_tokens: torch.Tensor,
    value_pages_fp4: torch.Tensor,
    value_scales: torch.Tensor,
    source_tokens: torch.Tensor,
    destination_pages: torch.Tensor,
    destination_bases: torch.Tensor | None = None,
) -> None:
    """Quantise V pages out of a flat token buffer; same indexing contract as K."""
    heads = _check_tokens(value_tokens, "value_tokens")
    _check_destination(value_pages_fp4, value_scales, heads, (heads, HEAD_DIM, PAGE_SIZE // 2))
    work = source_tokens.numel()
    if destination_pages.numel() != work:
        raise ValueError("source_tokens and destination_pages must agree")
    _launch(1, value_tokens, value_pages_fp4, value_scales, source_tokens, destination_pages,
            destination_bases, None, heads, work)


def quantize_key_pages(
    key_pages: torch.Tensor, *, key_shift: torch.Tensor | None = None
) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 K pages ``[pages, 128, heads, 128]`` -> (uint8 ``[pages, 128, heads, 64]``,
    float8_e4m3fn scales ``[pages, 32, 4, 1, 4, 2, heads]``)."""
    count, heads = _check_pages(key_pages, "key_pages")
    packed = torch.empty(count, PAGE_SIZE, heads, HEAD_DIM // 2, dtype=torch.uint8,
                         device=key_pages.device)
    storage = torch.empty(count * heads * 2 * _ATOM_BYTES, dtype=torch.uint8,
                          device=key_pages.device)
    scales = scale_view(storage, count, heads)
    _launch(0, key_pages.reshape(-1, heads, HEAD_DIM), packed, scales, None, None, None,
            key_shift, heads, count)
    return packed, scales.view(torch.float8_e4m3fn)


def quantize_value_pages(value_pages: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 V pages ``[pages, 128, heads, 128]`` -> (uint8 ``[pages, heads, 128, 64]`` with the
    token axis packed, float8_e4m3fn scales ``[pages, 32, 4, 1, 4, 2, heads]``)."""
    count, heads = _check_pages(value_pages, "value_pages")
    packed = torch.empty(count, heads, HEAD_DIM, PAGE_SIZE // 2, dtype=torch.uint8,
                         device=value_pages.device)
    storage = torch.empty(count * heads * 2 * _ATOM_BYTES, dtype=torch.uint8,
                          device=value_pages.device)
    scales = scale_view(storage, count, heads)
    _launch(1, value_pages.reshape(-1, heads, HEAD_DIM), packed, scales, None, None, None,
            None, heads, count)
    return packed, scales.view(torch.float8_e4m3fn)
