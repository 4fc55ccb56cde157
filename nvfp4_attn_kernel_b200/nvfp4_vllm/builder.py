"""Metadata builder: advances the tail-slot control plane once per scheduler step.

Counterpart of the reference project's ``src/nvfp4_vllm/builder.py`` (``decode_split`` :62-107,
``NVFP4MetadataBuilder`` :110-290).  ``build`` launches the control kernel and the page work
table, derives the decode prefix from host data the model runner already has, and reads nothing
back from the device (unless ``NVFP4_DEBUG=1``).
"""

from __future__ import annotations

import os

import torch
from vllm.v1.attention.backend import AttentionCGSupport
from vllm.v1.attention.backends.flash_attn import FlashAttentionMetadataBuilder
from vllm.v1.attention.backends.utils import split_decodes_and_prefills

from .control import ControlPlane
from .guards import NVFP4, check_supported
from .metadata import NVFP4Metadata
from .runtime import PAGE_SIZE
from .write import PageWorkTable

# "1": read the sticky error word after every step (one host synchronisation per step) so that
# the step that breaks an invariant is the step that raises.  For bisecting, not for production.
DEBUG_ENV = "NVFP4_DEBUG"


def decode_split(common_attn_metadata) -> tuple[int, int]:
    """Rows and tokens of this step's decode prefix (one-token rows sorted to the front).

    Uses ``query_start_loc_cpu`` only, so it costs no synchronisation.  Rows padded in for a full
    CUDA graph carry no token and stay inside the prefix as a suffix of it.  Raises when the
    batch is not sorted the way the read path needs.
    """
    num_decodes, _, num_decode_tokens, _ = split_decodes_and_prefills(
        common_attn_metadata, decode_threshold=1)
    starts = common_attn_metadata.query_start_loc_cpu
    rows = common_attn_metadata.num_reqs
    query_lens = starts[1:rows + 1] - starts[:rows]
    decode_lens = query_lens[:num_decodes]
    scheduled = int((decode_lens > 0).sum())
    sorted_ok = bool((decode_lens[:scheduled] == 1).all()) and bool((query_lens[num_decodes:] > 1).all())
    if not sorted_ok:
        raise ValueError(
            "the NVFP4 read path needs one-token requests at the front of the batch, but query "
            f"lengths are {query_lens.tolist()} with a decode prefix of {num_decodes}"
        )
    return num_decodes, num_decode_tokens


class NVFP4MetadataBuilder(FlashAttentionMetadataBuilder):
    """FlashAttention's builder plus this step's slot assignment (pass-through for other cache
    dtypes)."""

    @classmethod
    def get_cudagraph_support(cls, vllm_config, kv_cache_spec) -> AttentionCGSupport:
        cache = vllm_config.cache_config
        if cache is None or cache.cache_dtype != NVFP4:
            return super().get_cudagraph_support(vllm_config, kv_cache_spec)
        # a prefill runs varlen FlashAttention over a changing token count: only uniform
        # one-token decode batches can be frozen into a graph
        return AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE

    def __init__(self, kv_cache_spec, layer_names, vllm_config, device: torch.device) -> None:
        super().__init__(kv_cache_spec, layer_names, vllm_config, device)
        cache = vllm_config.cache_config
        self.nvfp4 = cache is not None and cache.cache_dtype == NVFP4
        self.built_for_capture = False
        self.capturing = False
        self.plane = None
        if not self.nvfp4:
            return
        self.debug = os.environ.get(DEBUG_ENV) == "1"
        # one-token requests to the front of the batch: the decode rows become a prefix slice
        self._init_reorder_batch_threshold(1)
        check_supported(vllm_config)
        sched = vllm_config.scheduler_config
        self.plane = ControlPlane(max_num_seqs=sched.max_num_seqs,
                                  max_num_batched_tokens=sched.max_num_batched_tokens, device=device)
        self.work_table = PageWorkTable(max_num_seqs=sched.max_num_seqs,
                                        max_num_batched_tokens=sched.max_num_batched_tokens,
                                        device=device)

    def build_for_cudagraph_capture(self, common_attn_metadata):
        """Metadata for a batch that is recorded, not served; remembers that capture happened so
        that the first real step afterwards starts from an empty slot table."""
        self.capturing = True
        try:
            return super().build_for_cudagraph_capture(common_attn_metadata)
        finally:
            self.capturing = False
            if self.nvfp4:
                self.built_for_capture = True

    def build(self, common_prefix_len: int, common_attn_metadata, fast_build: bool = False):
        base = super().build(common_prefix_len, common_attn_metadata, fast_build)
        if not self.nvfp4:
            return base
        if self.built_for_capture and not self.capturing:
            self.built_for_capture = False
            self.plane.reset()
        meta = common_attn_metadata
        outputs = self.plane.prepare(
            block_table=meta.block_table_tensor, seq_lens=meta.seq_lens,
            query_start_loc=meta.query_start_loc, num_reqs=meta.num_reqs,
            num_actual_tokens=meta.num_actual_tokens)
        if self.debug:
            self.plane.raise_for_errors()
        source_tokens, destination_pages = self.work_table.build(
            query_start_loc=meta.query_start_loc, seqused_fp4=outputs.seqused_fp4,
            row_to_slot=outputs.row_to_slot, block_table=meta.block_table_tensor,
            num_reqs=meta.num_reqs, max_query_len=meta.max_query_len)
        decode_rows, decode_tokens = decode_split(meta)
        prefill_starts = meta.query_start_loc
        if decode_tokens:
            prefill_starts = prefill_starts[decode_rows:] - decode_tokens
        return NVFP4Metadata.from_flash(
            base, outputs, source_tokens=source_tokens, destination_pages=destination_pages,
            decode_prefix_rows=decode_rows, decode_prefix_tokens=decode_tokens,
            prefill_query_start_loc=prefill_starts,
            # a row's last page is always its tail's, never an FP4 one
            decode_page_columns=max(1, (meta.max_seq_len - 1) // PAGE_SIZE))
