"""Sealing filled BF16 tail pages into the NVFP4 cache, after the last layer's attention.

Counterpart of the reference project's ``src/nvfp4_vllm/promote.py:33-62``: the launch shape is a
constant of the engine (the whole slot table, every layer); rows that did not fill a page carry
-1 and are skipped on the device.  K and V of all layers go in ONE launch (``nvfp4_tail_flush``).
"""

from __future__ import annotations

import torch

from .. import _lib


def launch(metadata, runtime) -> None:
    """Quantise every filled tail page into its block, for every layer."""
    bases = runtime.destination_bases            # int64 [4, layers]
    key_packed, key_scales, value_packed, value_scales = runtime.layer_regions(0)
    tail = runtime.tail_key
    layers, slots = tail.shape[0], tail.shape[1]
    with torch.cuda.device(tail.device):
        _lib.check(_lib.load().nvfp4_tail_flush(
            runtime.tail_key.data_ptr(), runtime.tail_value.data_ptr(), slots * 128,
            metadata.promotion_source_tokens.data_ptr(), metadata.promotion_pages.data_ptr(),
            bases.data_ptr(),
            key_packed.stride(0) * key_packed.element_size(), key_scales.stride(0),
            value_packed.stride(0) * value_packed.element_size(), value_scales.stride(0),
            metadata.promotion_pages.numel(), layers, runtime.num_kv_heads,
            torch.cuda.current_stream(tail.device).cuda_stream))
