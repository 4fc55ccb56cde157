"""Attention implementation over the NVFP4 KV cache.

Counterpart of the reference project's ``src/nvfp4_vllm/impl.py`` (``do_kv_cache_update`` :103-173,
``forward`` :175-225, ``_decode`` :227-268, ``_prefill`` :270-304).  The decode prefix of a step
reads FP4 pages + BF16 tail through ``fp4_decode``; the prefill suffix runs cache-free
FlashAttention over this pass's own K/V; the last layer seals filled tail pages.
The key shift is fused into the page quantiser and the tail copy (``write_kv(key_shift=...)``)
instead of a separate ``torch.sub``.
"""

from __future__ import annotations

import torch
from vllm.config import get_current_vllm_config
from vllm.forward_context import get_forward_context
from vllm.model_executor.layers.attention.attention import get_attention_context
from vllm.v1.attention.backends.flash_attn import FlashAttentionImpl

from ..nvfp4_decode_kernel import fp4_decode
from . import promote
from .guards import NVFP4, check_layer_supported, check_supported
from .runtime import LayerRuntime, piece_pages
from .write import accumulate_key_sum, reset_new_request_tails, write_kv


# A step of one-token rows only (pure decode) needs no page quantisation, and its tail copy can
# ride in the decode launch: False keeps the reference's separate write_kv launch.
FUSE_TAIL_APPEND = True



class NVFP4Impl(FlashAttentionImpl):
    def __init__(self, *args, **kwargs) -> None:
        config = get_current_vllm_config()
        check_supported(config)   # before super(): report an unsupported engine as such
        super().__init__(*args, **kwargs)
        cache = config.cache_config
        self.nvfp4 = cache is not None and cache.cache_dtype == NVFP4
        self.num_slots = 0
        self.max_pages = 0
        if self.nvfp4:
            check_layer_supported(self)
            # prefill attends this pass's BF16 K/V and decode quantises to FP4, never FP8
            self.supports_quant_query_input = False
            self.num_slots = config.scheduler_config.max_num_seqs
            self.max_pages = -(-int(getattr(config.model_config, "max_model_len", 0) or 0) // 128)
        self.runtime: LayerRuntime | None = None
        self.layer_index = 0
        self._fused_kv = None   # (key, value, shift) of a pure decode step, appended by the decode launch

    def _bind_runtime(self, device: torch.device) -> None:
        """Create the model's shared state once (in the profile run, so that vLLM subtracts it
        from the cache budget) and hand it to every NVFP4 layer."""
        modules = [m for m in get_forward_context().no_compile_layers.values()
                   if isinstance(getattr(m, "impl", None), NVFP4Impl)]
        if not any(m.impl is self for m in modules):
            raise ValueError(
                "an NVFP4 layer is running outside the forward context that lists it, so the "
                "write path cannot be shared with its peers"
            )
        shapes = {(m.impl.num_heads, m.impl.num_kv_heads, m.impl.head_size) for m in modules}
        if len(shapes) != 1:
            raise ValueError(f"NVFP4 needs one attention shape across layers, found {shapes}")
        num_heads, num_kv_heads, head_dim = shapes.pop()
        runtime = LayerRuntime(num_layers=len(modules), num_slots=self.num_slots,
                               num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                               device=device, max_pages=self.max_pages)
        for index, module in enumerate(modules):
            module.impl.runtime = runtime
            module.impl.layer_index = index

    def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping) -> None:
        if not self.nvfp4:
            super().do_kv_cache_update(layer, key, value, kv_cache, slot_mapping)
            return
        metadata, _, _, _ = get_attention_context(layer.layer_name)
        if metadata is None or self.runtime is None:   # profile run: no cache to write into
            return
        runtime = self.runtime
        if self.layer_index == 0:
            # a slot's previous tenant is erased from every layer before any layer writes
            reset_new_request_tails(tail_key=runtime.tail_key, tail_value=runtime.tail_value,
                                    query_start_loc=metadata.query_start_loc,
                                    seq_lens=metadata.seq_lens, row_to_slot=metadata.row_to_slot)
        shift = None
        if runtime.key_shift_sum is not None:
            accumulate_key_sum(key[: metadata.num_actual_tokens], runtime.key_shift_sum[self.layer_index])
            if self.layer_index == 0:
                runtime.key_shift_tokens += metadata.num_actual_tokens
        elif runtime.active_key_shift is not None:
            shift = runtime.active_key_shift[self.layer_index]
        key_fp4, key_sf, value_fp4, value_sf = runtime.views(self.layer_index, kv_cache)
        rows = metadata.decode_prefix_rows
        self._fused_kv = None
        if (FUSE_TAIL_APPEND and rows and metadata.decode_prefix_tokens == metadata.num_actual_tokens
                and key.shape[0] >= rows and value.shape[0] >= rows):
            # one-token rows only: nothing to quantise, and the decode launch stores each row's
            # token itself (rows padded in for a CUDA graph have an empty tail and store nothing)
            self._fused_kv = (key[:rows], value[:rows], shift)
            return
        write_kv(key=key, value=value, key_pages_fp4=key_fp4, key_scales=key_sf,
                 value_pages_fp4=value_fp4, value_scales=value_sf,
                 tail_key=runtime.tail_key[self.layer_index],
                 tail_value=runtime.tail_value[self.layer_index],
                 source_tokens=metadata.source_tokens, destination_pages=metadata.destination_pages,
                 query_start_loc=metadata.query_start_loc, seq_lens=metadata.seq_lens,
                 seqused_fp4=metadata.seqused_fp4, row_to_slot=metadata.row_to_slot,
                 num_actual_tokens=metadata.num_actual_tokens, key_shift=shift)

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None,
                output_scale=None, output_block_scale=None):
        if not self.nvfp4:
            return super().forward(layer, query, key, value, kv_cache, attn_metadata, output,
                                   output_scale, output_block_scale)
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError(
                "fused output quantization is not supported by the NVFP4 attention path"
            )
        if self.runtime is None:
            self._bind_runtime(query.device)
        if attn_metadata is None:   # profile run: nothing to read, and NaNs must not propagate
            return output.zero_()
        self.runtime.expect_layer(self.layer_index)
        rows = attn_metadata.decode_prefix_rows
        tokens = attn_metadata.decode_prefix_tokens
        if rows:
            self._decode(rows, query, kv_cache, attn_metadata, output)
        if tokens < attn_metadata.num_actual_tokens:
            self._prefill(tokens, query, key, value, attn_metadata, output)
        if self.layer_index == self.runtime.num_layers - 1:
            promote.launch(attn_metadata, self.runtime)
        return output

    def _decode(self, rows, query, kv_cache, attn_metadata, output) -> None:
        runtime = self.runtime
        key_fp4, key_sf, value_fp4, value_sf = runtime.views(self.layer_index, kv_cache)
        pages = attn_metadata.decode_page_columns
        extra = self._take_fused_kv()
        piece = piece_pages(rows, key_fp4.shape[2], pages, runtime.sm_count)
        space = runtime.balance_workspace(rows, query.shape[1], pages, piece) if piece else None
        if space is not None:
            # Rows longer than a piece are cut by their own device-side lengths (the list of pieces
            # is built on the device, so a captured CUDA graph follows the lengths of every
            # replay); the lengths are the step's, so the step's first cut layer builds the list
            # and the others reuse it - but only a list that was built for this very step and
            # shape in this very scratch (layer 0 starts a step; a layer that finds no such list,
            # e.g. because the first layers of a model do not come through here, builds it).
            key = (attn_metadata.seqused_fp4.data_ptr(), rows, pages, piece, space.data_ptr())
            if self.layer_index == 0:
                runtime.work_list_reusable(None)
            extra.update(balance_pages=piece, balance_workspace=space,
                         balance_reuse=runtime.work_list_reusable(key))
        fp4_decode(
            query=query[:rows], key_pages_fp4=key_fp4, key_scales=key_sf,
            value_pages_fp4=value_fp4, value_scales=value_sf,
            fp4_page_table=attn_metadata.block_table[:rows, :pages],
            seqused_fp4=attn_metadata.seqused_fp4[:rows],
            residual_key_pages_bf16=runtime.tail_key[self.layer_index],
            residual_value_pages_bf16=runtime.tail_value[self.layer_index],
            residual_page_ids=attn_metadata.row_to_slot[:rows],
            seqused_residual=attn_metadata.seqused_residual[:rows],
            softmax_scale=self.scale,
            trusted_metadata=True,   # produced on the device this same step; never read back
            query_padded_scratch=runtime.query_padded, query_fp4_scratch=runtime.query_fp4,
            query_scales_scratch=runtime.query_scales, out=output[:rows], **extra)

    def _take_fused_kv(self) -> dict:
        fused, self._fused_kv = self._fused_kv, None
        if fused is None:
            return {}
        key, value, shift = fused
        return dict(append_key=key, append_value=value, key_shift=shift)

    def _prefill(self, tokens, query, key, value, attn_metadata, output) -> None:
        starts = attn_metadata.prefill_query_start_loc
        end = attn_metadata.num_actual_tokens
        # bound at call time: the symbol exists only where vLLM found a CUDA platform
        from vllm.v1.attention.backends.fa_utils import flash_attn_varlen_func

        flash_attn_varlen_func(
            q=query[tokens:end], k=key[tokens:end], v=value[tokens:end], out=output[tokens:end],
            cu_seqlens_q=starts, max_seqlen_q=attn_metadata.max_query_len,
            cu_seqlens_k=starts, max_seqlen_k=attn_metadata.max_query_len,
            softmax_scale=self.scale, causal=attn_metadata.causal,
            fa_version=self.vllm_flash_attn_version)
