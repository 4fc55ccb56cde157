"""A vLLM KV-cache block seen as one NVFP4 page: packed K, K scales, packed V, V scales, one
after another inside the block (block-major).  Counterpart of the reference project's
``src/nvfp4_vllm/layout.py:28-103``."""

from __future__ import annotations

import torch

from ..nvfp4_decode_kernel.quantize_kv_kernel import scale_view

PAGE_SIZE = 128


def page_bytes(num_kv_heads: int, head_dim: int = 128, device: str | None = None) -> int:
    """Bytes one block must provide: ``2 * 128 * Hkv * (D/2 + D/16)``."""
    return 2 * PAGE_SIZE * num_kv_heads * (head_dim // 2 + head_dim // 16)


def carve(kv_cache: torch.Tensor, num_kv_heads: int, head_dim: int) -> tuple[torch.Tensor, ...]:
    """View one layer's ``[blocks, bytes]`` array as the four regions, page stride = block pitch."""
    if kv_cache.ndim != 2 or kv_cache.element_size() != 1:
        raise ValueError(
            f"expected a [blocks, bytes] byte cache, got {tuple(kv_cache.shape)} of {kv_cache.dtype}"
        )
    if head_dim != 128:
        raise ValueError("the NVFP4 page layout is defined for head_dim 128")
    blocks, pitch = kv_cache.shape
    if kv_cache.stride() != (pitch, 1):
        raise ValueError("the block array must be contiguous")
    required = page_bytes(num_kv_heads, head_dim)
    if pitch != required:
        raise ValueError(
            f"a block of {pitch} bytes cannot hold {required} bytes of NVFP4 page; the "
            "backend's page size and this layout disagree"
        )
    flat = kv_cache.view(torch.uint8).reshape(-1)
    base = 0  # reshape(-1) of a contiguous view keeps the storage offset
    packed = PAGE_SIZE * num_kv_heads * 64
    scales = num_kv_heads * 1024
    key_packed = flat.as_strided((blocks, PAGE_SIZE, num_kv_heads, 64),
                                 (pitch, num_kv_heads * 64, 64, 1), flat.storage_offset() + base)
    key_scales = scale_view(flat, blocks, num_kv_heads, pitch, flat.storage_offset() + packed)
    value_packed = flat.as_strided((blocks, num_kv_heads, 128, 64), (pitch, 128 * 64, 64, 1),
                                   flat.storage_offset() + packed + scales)
    value_scales = scale_view(flat, blocks, num_kv_heads, pitch,
                              flat.storage_offset() + 2 * packed + scales)
    return (key_packed, key_scales.view(torch.float8_e4m3fn), value_packed,
            value_scales.view(torch.float8_e4m3fn))
