"""Per-step bookkeeping of the BF16 tail slots, resolved on the device.

Same class surface, buffers and error flags as the reference project's
``src/nvfp4_vllm/control.py`` (``ControlPlane`` :360-511, flags :84-98); the single-CTA kernel
behind it is ``nvfp4_control_step`` of the C ABI instead of a Triton kernel.  Nothing here reads
device values back, and ``prepare`` can be captured into a CUDA graph.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _lib

PAGE_SIZE = 128
# One BF16 tail slot per running request; the engine is validated up to this many.
MAX_SUPPORTED_SLOTS = 32

FREE_KEY = -1
NULL_BLOCK = 0        # vLLM's block pool never hands block 0 to a request
INACTIVE_ROW = -1     # a row or token that owns no tail slot

ERR_CONTINUATION_PREFILL = 1
ERR_SLOT_LOST = 2
ERR_STALE_SLOT_HISTORY = 4
ERR_NO_FREE_SLOT = 8
ERR_DUPLICATE_KEY = 16
ERR_PROMOTION_COLUMN = 32
ERR_WORK_LIST_FULL = 64   # only with a work-list plan; no counterpart in the reference

ERROR_NAMES = {
    ERR_CONTINUATION_PREFILL: "a prompt arrived split across steps",
    ERR_SLOT_LOST: "a row with history matched no slot",
    ERR_STALE_SLOT_HISTORY: "a matched slot's length does not continue",
    ERR_NO_FREE_SLOT: "a row needing a slot found none free",
    ERR_DUPLICATE_KEY: "two live rows share a physical block",
    ERR_PROMOTION_COLUMN: "a promotion column is past the block table",
    ERR_WORK_LIST_FULL: "the list of decode pieces outgrew its capacity",
}


@dataclass(frozen=True)
class ControlOutputs:
    """Views into the control plane's scratch, valid until the next step (device only)."""

    row_to_slot: torch.Tensor
    token_to_slot: torch.Tensor
    seqused_fp4: torch.Tensor
    seqused_residual: torch.Tensor
    promotion_source_tokens: torch.Tensor   # full slot-table width
    promotion_pages: torch.Tensor           # full slot-table width, -1 = nothing to seal
    error_code: torch.Tensor


@dataclass(frozen=True)
class WorkListPlan:
    """What the step's balanced-split decode calls will be given, so that the control step can
    build their list of pieces in its own launch (an extension; the reference has neither the
    balanced split nor a list): the first ``decode_rows`` rows of the batch, a page table
    ``max_pages`` columns wide, pieces of ``target_pages`` pages, ``heads_q`` query heads and the
    ``workspace`` (uint8, ``balanced_workspace_bytes`` long) the calls share.  The calls then pass
    ``balance_reuse=True`` in every layer."""

    decode_rows: int
    max_pages: int
    target_pages: int
    heads_q: int
    workspace: torch.Tensor


class ControlPlaneError(RuntimeError):
    """An invariant the slot table reported through ``error_code``."""


class ControlPlane:
    """Slot table and per-step scratch of one engine, allocated once at the high-water mark."""

    def __init__(self, *, max_num_seqs: int, max_num_batched_tokens: int,
                 device: torch.device | str, page_size: int = PAGE_SIZE) -> None:
        if max_num_seqs < 1:
            raise ValueError(f"max_num_seqs must be positive, got {max_num_seqs}")
        if max_num_seqs > 128:
            raise ValueError(f"the slot table holds at most 128 slots, got {max_num_seqs}")
        if max_num_batched_tokens < max_num_seqs:
            raise ValueError(
                f"max_num_batched_tokens ({max_num_batched_tokens}) must cover "
                f"one token per row ({max_num_seqs})"
            )
        if page_size != PAGE_SIZE:
            raise ValueError("the page size is fixed at 128 tokens")
        self.num_slots = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.page_size = page_size
        self.device = torch.device(device)

        def slots(dtype, fill):
            return torch.full((self.num_slots,), fill, dtype=dtype, device=self.device)

        self.slot_keys = slots(torch.int32, FREE_KEY)
        self.slot_last_seq = slots(torch.int32, -1)
        self.slot_last_seen = slots(torch.int64, -1)
        self.step = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.row_to_slot = slots(torch.int32, INACTIVE_ROW)
        self.seqused_fp4 = slots(torch.int32, 0)
        self.seqused_residual = slots(torch.int32, 0)
        self.promotion_source_tokens = slots(torch.int32, 0)
        self.promotion_pages = slots(torch.int32, INACTIVE_ROW)
        self.error_code = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.token_to_slot = torch.full((max_num_batched_tokens,), INACTIVE_ROW, dtype=torch.int32,
                                        device=self.device)

    def reset(self) -> None:
        """Forget every slot.  Only valid when no request is in flight."""
        self.slot_keys.fill_(FREE_KEY)
        self.slot_last_seq.fill_(-1)
        self.slot_last_seen.fill_(-1)
        self.step.zero_()
        self.error_code.zero_()

    def raise_for_errors(self) -> None:
        """Read the sticky error word (a host synchronisation) and raise if anything is set."""
        code = int(self.error_code.item())
        if not code:
            return
        named = [text for bit, text in ERROR_NAMES.items() if code & bit]
        unknown = code & ~sum(ERROR_NAMES)
        if unknown:
            named.append(f"unrecognized flags {unknown:#x}")
        raise ControlPlaneError(
            f"the slot control plane reported error_code {code}: " + "; ".join(named)
        )

    def prepare(self, *, block_table: torch.Tensor, seq_lens: torch.Tensor,
                query_start_loc: torch.Tensor, num_reqs: int,
                num_actual_tokens: int, work_list: WorkListPlan | None = None) -> ControlOutputs:
        """Advance the slot table by one step; ``seq_lens`` already counts this step's tokens.
        With ``work_list`` the same launch also lists the pieces of the step's decode rows."""
        if block_table.ndim != 2:
            raise ValueError(f"block_table must be 2-D, got {block_table.ndim}-D")
        if num_reqs > self.num_slots:
            raise ValueError(f"{num_reqs} rows exceeds the {self.num_slots} tail slots")
        if num_actual_tokens > self.max_num_batched_tokens:
            raise ValueError(
                f"{num_actual_tokens} tokens exceeds the "
                f"{self.max_num_batched_tokens} the scratch was sized for"
            )
        for tensor, name in ((block_table, "block_table"), (seq_lens, "seq_lens"),
                             (query_start_loc, "query_start_loc")):
            if tensor.dtype is not torch.int32 or tensor.device != self.device:
                raise ValueError(f"{name} must be INT32 on {self.device}")
        if block_table.stride(1) != 1 and block_table.shape[1] > 1:
            raise ValueError("block_table rows must be contiguous")
        common = (
            block_table.data_ptr(), block_table.stride(0), block_table.shape[1],
            seq_lens.data_ptr(), query_start_loc.data_ptr(), self.slot_keys.data_ptr(),
            self.slot_last_seq.data_ptr(), self.slot_last_seen.data_ptr(), self.step.data_ptr(),
            self.row_to_slot.data_ptr(), self.token_to_slot.data_ptr(),
            self.seqused_fp4.data_ptr(), self.seqused_residual.data_ptr(),
            self.promotion_source_tokens.data_ptr(), self.promotion_pages.data_ptr(),
            self.error_code.data_ptr(), num_reqs, num_actual_tokens, self.num_slots)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            if work_list is None:
                _lib.check(_lib.load().nvfp4_control_step(*common, stream))
            else:
                space = work_list.workspace
                if space.dtype is not torch.uint8 or space.device != self.device or not space.is_contiguous():
                    raise ValueError(f"the work list's workspace must be contiguous UINT8 on {self.device}")
                _lib.check(_lib.load().nvfp4_control_step_balanced(
                    *common, work_list.decode_rows, work_list.max_pages, work_list.target_pages,
                    work_list.heads_q, space.data_ptr(), space.numel(), stream))
        return ControlOutputs(
            row_to_slot=self.row_to_slot[:num_reqs],
            token_to_slot=self.token_to_slot[:num_actual_tokens],
            seqused_fp4=self.seqused_fp4[:num_reqs],
            seqused_residual=self.seqused_residual[:num_reqs],
            promotion_source_tokens=self.promotion_source_tokens,
            promotion_pages=self.promotion_pages,
            error_code=self.error_code,
        )
