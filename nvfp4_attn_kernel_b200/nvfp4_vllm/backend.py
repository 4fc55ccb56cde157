"""Attention backend that declares the NVFP4 KV-cache page to vLLM.

Same class surface as the reference project's ``src/nvfp4_vllm/backend.py:44-152``: name
``CUSTOM``, 128-token blocks only, compute capability 10.x only, a flat
``(num_blocks, page_bytes)`` cache shape.
"""

from __future__ import annotations

from typing import ClassVar

import torch
from vllm.config import get_current_vllm_config_or_none
from vllm.v1.attention.backends.flash_attn import FlashAttentionBackend

from .guards import NVFP4

PAGE_SIZE = 128
HEAD_SIZE = 128
SM100 = 10


def _cache_dtype() -> str | None:
    config = get_current_vllm_config_or_none()
    if config is None or config.cache_config is None:
        return None
    return config.cache_config.cache_dtype


def nvfp4_page_size_bytes(block_size: int, num_kv_heads: int, head_size: int) -> int:
    """Bytes of one K+V page of one layer: two E2M1 values per byte plus one E4M3 scale byte per
    16 values.  Must equal what vLLM budgets in ``AttentionSpec.real_page_size_bytes``."""
    return 2 * block_size * num_kv_heads * (head_size // 2 + head_size // 16)


class NVFP4Backend(FlashAttentionBackend):
    """Paged NVFP4 KV cache; FlashAttention for everything that is not the NVFP4 cache."""

    supported_kv_cache_dtypes: ClassVar[list[str]] = [
        *FlashAttentionBackend.supported_kv_cache_dtypes, NVFP4,
    ]

    @staticmethod
    def get_name() -> str:
        return "CUSTOM"  # vLLM resolves AttentionBackendEnum[get_name()]

    @staticmethod
    def get_impl_cls() -> type:
        from .impl import NVFP4Impl

        return NVFP4Impl

    @staticmethod
    def get_builder_cls() -> type:
        from .builder import NVFP4MetadataBuilder

        return NVFP4MetadataBuilder

    @staticmethod
    def get_supported_kernel_block_sizes() -> list[int]:
        return [PAGE_SIZE]  # V is quantised along tokens a whole page at a time

    @classmethod
    def supports_kv_cache_dtype(cls, kv_cache_dtype) -> bool:
        # FlashAttention's own check is a fixed list
        return kv_cache_dtype == NVFP4 or super().supports_kv_cache_dtype(kv_cache_dtype)

    @classmethod
    def supports_block_size(cls, block_size: int | None) -> bool:
        return block_size is None or block_size == PAGE_SIZE

    @classmethod
    def supports_compute_capability(cls, capability) -> bool:
        return capability.major == SM100

    @classmethod
    def supports_kv_connector(cls) -> bool:
        return False  # connectors move pages by address and size, not by this layout

    @classmethod
    def supports_combination(cls, head_size, dtype, kv_cache_dtype, *rest, **more) -> str | None:
        # the trailing arguments differ between vLLM releases (0.22 has no use_mm_prefix); only the
        # first three matter here
        if kv_cache_dtype == NVFP4 and head_size != HEAD_SIZE:
            return f"NVFP4 decode is compiled for head_size {HEAD_SIZE}, got {head_size}"
        return None

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> tuple[int, ...]:
        if cache_dtype_str != NVFP4:
            return FlashAttentionBackend.get_kv_cache_shape(
                num_blocks, block_size, num_kv_heads, head_size, cache_dtype_str=cache_dtype_str)
        return (num_blocks, nvfp4_page_size_bytes(block_size, num_kv_heads, head_size))

    @staticmethod
    def get_kv_cache_stride_order(include_num_layers_dimension: bool = False) -> tuple[int, ...]:
        if _cache_dtype() == NVFP4:
            raise NotImplementedError  # identity order: a flat byte page
        return FlashAttentionBackend.get_kv_cache_stride_order(include_num_layers_dimension)
