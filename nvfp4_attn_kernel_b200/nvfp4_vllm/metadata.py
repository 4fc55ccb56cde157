"""Per-step attention metadata of the NVFP4 KV cache: FlashAttention's own fields plus what the
slot control plane resolved for this step.  Counterpart of the reference project's
``src/nvfp4_vllm/metadata.py:28-136``.  All tensors stay on the device; the ints are host values
taken from CPU-side batch descriptions."""

from __future__ import annotations

from dataclasses import dataclass, fields

import torch
from vllm.v1.attention.backends.flash_attn import FlashAttentionMetadata

from .control import ControlOutputs


@dataclass(kw_only=True)
class NVFP4Metadata(FlashAttentionMetadata):
    row_to_slot: torch.Tensor              # [num_reqs] int32, -1 = padding row
    token_to_slot: torch.Tensor            # [num_actual_tokens] int32
    seqused_fp4: torch.Tensor              # [num_reqs] int32, whole pages
    seqused_residual: torch.Tensor         # [num_reqs] int32, tokens in the BF16 tail
    promotion_source_tokens: torch.Tensor  # [max_num_seqs] int32 (full width: it is a launch grid)
    promotion_pages: torch.Tensor          # [max_num_seqs] int32, -1 = nothing to seal
    decode_prefix_rows: int                # rows [0, n) emit exactly one token
    decode_prefix_tokens: int              # where the prefill tokens begin
    prefill_query_start_loc: torch.Tensor  # query_start_loc rebased on the first prefill token
    decode_page_columns: int               # page-table columns the decode kernel has to walk
    source_tokens: torch.Tensor            # [work] int32, first token of each full page of this step
    destination_pages: torch.Tensor        # [work] int32, its block, -1 = no work

    @classmethod
    def from_flash(cls, base: FlashAttentionMetadata, outputs: ControlOutputs, *,
                   source_tokens: torch.Tensor, destination_pages: torch.Tensor,
                   decode_prefix_rows: int, decode_prefix_tokens: int,
                   prefill_query_start_loc: torch.Tensor,
                   decode_page_columns: int) -> "NVFP4Metadata":
        carried = {f.name: getattr(base, f.name) for f in fields(base)}
        return cls(
            **carried,
            row_to_slot=outputs.row_to_slot,
            token_to_slot=outputs.token_to_slot,
            seqused_fp4=outputs.seqused_fp4,
            seqused_residual=outputs.seqused_residual,
            promotion_source_tokens=outputs.promotion_source_tokens,
            promotion_pages=outputs.promotion_pages,
            decode_prefix_rows=decode_prefix_rows,
            decode_prefix_tokens=decode_prefix_tokens,
            prefill_query_start_loc=prefill_query_start_loc,
            decode_page_columns=decode_page_columns,
            source_tokens=source_tokens,
            destination_pages=destination_pages,
        )
