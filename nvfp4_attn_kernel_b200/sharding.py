"""Sharding of the decode path over the GPUs of one node (one process per GPU).

Three ways, as the path allows:

* rows (sequences) to GPUs and KV heads to GPUs need nothing from this module
  beyond :func:`kv_head_slice`: the work units are independent, no collective.
* KV page ranges to GPUs (long contexts): rank r owns logical pages
  ``page_range(n, r, world)`` of every row and the BF16 tail goes with rank 0.
  Each rank runs the decode in partial mode on its own pages and the partials
  ``(normalised O fp32, natural-log LSE)`` are merged by LSE weight.
  :class:`PageRangeGroup` does the exchange in one of four ways: ``"fused"`` (the
  decode kernel itself pushes and merges every (row, KV head) tile as soon as the
  tile's last split is done: one launch per rank and step), ``"push"`` (one
  launch per rank that folds the rank's local splits, stores the result into every
  peer's inbox in symmetric memory, and merges out of its own inbox once the peers'
  stores for the same (head, row) have arrived), ``"peer"`` (announce, bounded wait,
  merge with loads from the peers' buffers) or ``"nccl"`` (all-gather, then the local
  merge kernel).

The reference project has no multi-GPU code; the page-range rule and the partial
format are those of its intra-GPU split path
(``src/nvfp4_decode_kernel/_fa4/block_info.py:46-54``,
``fp4_decode_kernel.py:159,5186-5196``).
"""

from __future__ import annotations

import os

import torch

from . import _lib

PAGE = 128
HEAD_DIM = 128


def page_range(n_pages: int, part: int, parts: int) -> tuple[int, int]:
    """Logical pages ``[first, last)`` of a row of ``n_pages`` owned by ``part`` of ``parts``."""
    per = -(-n_pages // parts) if n_pages > 0 else 0
    return min(part * per, n_pages), min((part + 1) * per, n_pages)


def kv_head_slice(rank: int, world: int, heads_q: int, heads_kv: int) -> tuple[slice, slice]:
    """Query-head and KV-head slices of a tensor-parallel rank (KV head h -> rank h*world/Hkv)."""
    if heads_kv % world:
        raise ValueError(f"{heads_kv} KV heads do not divide over {world} ranks")
    per_kv = heads_kv // world
    group = heads_q // heads_kv
    return (slice(rank * per_kv * group, (rank + 1) * per_kv * group),
            slice(rank * per_kv, (rank + 1) * per_kv))


def local_page_table(page_table: torch.Tensor, seqused_fp4: torch.Tensor, rank: int, world: int):
    """A rank's view of the block table under the page-range split.

    Returns ``(local_table [rows, ceil(max_pages/world)], local_seqused_fp4 [rows])``; column j
    of the local table is global column ``first(row) + j``.  Pure tensor arithmetic on the
    table's device: nothing is read back to the host.
    """
    rows, max_pages = page_table.shape
    n = (seqused_fp4 // PAGE).to(torch.int64)
    per = (n + world - 1) // world
    first = torch.minimum(rank * per, n)
    last = torch.minimum((rank + 1) * per, n)
    width = max(1, -(-max_pages // world))
    cols = first[:, None] + torch.arange(width, device=page_table.device)[None, :]
    live = cols < last[:, None]
    gathered = torch.gather(page_table, 1, cols.clamp(max=max_pages - 1))
    local = torch.where(live, gathered, torch.full_like(gathered, -1)).to(torch.int32)
    return local.contiguous(), ((last - first) * PAGE).to(torch.int32)


class PageRangeGroup:
    """Exchange + merge of per-rank partial results for the KV page-range split.

    ``exchange="fused"``: as "push", but done by the decode kernel for each (row, KV head)
    tile as it completes (``nvfp4_decode_exchange``); needs ``heads_kv``, the tensor-core
    kernel and at most 8 query heads per KV head.  ``exchange="push"``: every rank owns an inbox in symmetric memory; ``merge`` is ONE kernel
    launch per rank (``nvfp4_push_merge``) that also folds the rank's local splits, and nothing
    is loaded over NVLink.  ``exchange="peer"``: partials live in symmetric memory that every
    rank of the group has mapped; ``merge`` is one launch per rank (``nvfp4_peer_merge``) that
    loads from the peers.  In both, two copies of the exchanged data alternate per call so that
    a fast rank cannot overwrite what a slow rank is still reading.  ``exchange="nccl"``:
    partials are all-gathered, then merged locally.
    """

    def __init__(self, group, rows: int, heads_q: int, device: torch.device, exchange: str = "peer",
                 heads_kv: int | None = None):
        import torch.distributed as dist

        if exchange not in ("fused", "push", "peer", "nccl"):
            raise ValueError("exchange must be 'fused', 'push', 'peer' or 'nccl'")
        if exchange == "fused" and not heads_kv:
            raise ValueError("the fused exchange counts arrivals per (row, KV head): pass heads_kv")
        if exchange == "fused" and heads_q // heads_kv > 8:
            raise ValueError("the fused exchange serves at most 8 query heads per KV head; "
                             "use exchange='push' for 16 and 32")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.rows, self.heads_q, self.device, self.exchange = rows, heads_q, device, exchange
        self.epoch = 0
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._epoch_state = torch.zeros(2, dtype=torch.int32, device=device)  # device-resident epoch
        self._o_elems = rows * heads_q * HEAD_DIM
        self._lse_elems = rows * heads_q
        per_copy = self._o_elems + self._lse_elems
        if exchange in ("push", "fused"):
            if exchange == "fused":
                self._tile_counters = torch.zeros(rows * heads_kv, dtype=torch.int32, device=device)
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm

            inbox = int(_lib.load().nvfp4_push_merge_inbox_floats(self.world, rows, heads_q))
            flag_words = self.world * rows * heads_q
            self._buf = symm.empty(inbox + flag_words, dtype=torch.float32, device=device)
            self._buf.zero_()
            torch.cuda.synchronize(device)
            self._hdl = symm.rendezvous(self._buf, group)
            bases = [int(p) for p in self._hdl.buffer_ptrs]
            self._inboxes = torch.tensor(bases, dtype=torch.int64, device=device)
            self._flags = torch.tensor([b + 4 * inbox for b in bases], dtype=torch.int64, device=device)
            # this rank's own partial never crosses NVLink: a plain local buffer
            self._own = torch.zeros(per_copy, dtype=torch.float32, device=device)
            dist.barrier(group)
        elif exchange == "peer":
            # plain peer loads only; no switch-side (multi-destination) objects are needed or used
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm

            flag_words = 64
            self._buf = symm.empty(2 * per_copy + flag_words, dtype=torch.float32, device=device)
            self._buf.zero_()
            torch.cuda.synchronize(device)
            self._hdl = symm.rendezvous(self._buf, group)
            bases = [int(p) for p in self._hdl.buffer_ptrs]
            self._ptr_tables = []
            for copy in range(2):
                o = [b + 4 * copy * per_copy for b in bases]
                lse = [b + 4 * (copy * per_copy + self._o_elems) for b in bases]
                self._ptr_tables.append((
                    torch.tensor(o, dtype=torch.int64, device=device),
                    torch.tensor(lse, dtype=torch.int64, device=device),
                ))
            self._flags = torch.tensor([b + 4 * 2 * per_copy for b in bases], dtype=torch.int64,
                                       device=device)
            dist.barrier(group)
        else:
            self._buf = torch.zeros(per_copy, dtype=torch.float32, device=device)
            self._gathered = torch.empty(self.world * per_copy, dtype=torch.float32, device=device)

    def local_split_buffers(self, splits: int):
        """fp32 scratch for ``splits`` local partials of a rank's own page range (allocated once
        per split count): ``([S, rows, 1, Hq, 128], [S, rows, Hq, 1])``."""
        cache = self.__dict__.setdefault("_local", {})
        if splits not in cache:
            cache[splits] = (
                torch.empty(splits, self.rows, 1, self.heads_q, HEAD_DIM, dtype=torch.float32,
                            device=self.device),
                torch.empty(splits, self.rows, self.heads_q, 1, dtype=torch.float32,
                            device=self.device),
            )
        return cache[splits]

    def fold_local_splits(self, splits: int) -> None:
        """Merge the local partials by LSE weight into this rank's partial for the NEXT
        ``merge`` call (normalised fp32 O and its LSE: the same form, one level up)."""
        o_loc, lse_loc = self.local_split_buffers(splits)
        o, lse = self.partial_buffers()
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().nvfp4_lse_merge(
                o_loc.data_ptr(), o_loc.stride(0), lse_loc.data_ptr(), lse_loc.stride(0), splits,
                self.rows, self.heads_q, o.data_ptr(), 1, None, lse.data_ptr(),
                torch.cuda.current_stream(self.device).cuda_stream))

    def partial_buffers(self):
        """(o_partial [1, rows, 1, Hq, 128], lse_partial [1, rows, Hq, 1]) for the NEXT merge call."""
        copy = (self.epoch + 1) & 1 if self.exchange == "peer" else 0
        per_copy = self._o_elems + self._lse_elems
        base = copy * per_copy
        buf = self._own if self.exchange in ("push", "fused") else self._buf
        o = buf[base:base + self._o_elems].view(1, self.rows, 1, self.heads_q, HEAD_DIM)
        lse = buf[base + self._o_elems:base + per_copy].view(1, self.rows, self.heads_q, 1)
        return o, lse

    def exchange_args(self, out: torch.Tensor):
        """The exchange block for ``nvfp4_decode_exchange`` writing the merged rows to ``out``;
        counts as this step's merge (the epoch advances)."""
        if self.exchange != "fused":
            raise ValueError("exchange_args belongs to exchange='fused'")
        if out.dtype not in (torch.bfloat16, torch.float32) or not out.is_contiguous() or \
                tuple(out.shape) != (self.rows, self.heads_q, HEAD_DIM):
            raise ValueError("out must be contiguous BF16/FP32 with shape [rows, heads_q, 128]")
        self.epoch += 1
        x = _lib.ExchangeArgs()
        x.inbox_ptrs = self._inboxes.data_ptr()
        x.flag_ptrs = self._flags.data_ptr()
        x.epoch_state = self._epoch_state.data_ptr()
        x.tile_counters = self._tile_counters.data_ptr()
        x.out = out.data_ptr()
        x.out_is_f32 = 1 if out.dtype is torch.float32 else 0
        x.rank, x.world = self.rank, self.world
        return x

    def merge(self, out: torch.Tensor, local_splits: int = 1) -> torch.Tensor:
        """Merge every rank's partial (written into ``partial_buffers()``) into ``out``.  With
        ``exchange="push"`` and ``local_splits`` > 1 the rank's partials are taken from
        ``local_split_buffers(local_splits)`` and folded inside the same launch."""
        if out.dtype not in (torch.bfloat16, torch.float32) or not out.is_contiguous() or \
                tuple(out.shape) != (self.rows, self.heads_q, HEAD_DIM):
            raise ValueError("out must be contiguous BF16/FP32 with shape [rows, heads_q, 128]")
        lib = _lib.load()
        stream = torch.cuda.current_stream(self.device).cuda_stream
        f32 = 1 if out.dtype is torch.float32 else 0
        if self.exchange == "fused":
            raise ValueError("with exchange='fused' the decode launch merges; there is no separate merge")
        self.epoch += 1
        if self.exchange == "push":
            o_loc, lse_loc = (self.partial_buffers() if local_splits <= 1
                              else self.local_split_buffers(local_splits))
            with torch.cuda.device(self.device):
                _lib.check(lib.nvfp4_push_merge(
                    o_loc.data_ptr(), o_loc.stride(0), lse_loc.data_ptr(), lse_loc.stride(0),
                    max(1, local_splits), self._inboxes.data_ptr(), self._flags.data_ptr(), self.rank,
                    self.world, self.epoch, self._epoch_state.data_ptr(), self.rows, self.heads_q,
                    out.data_ptr(), f32, self.status.data_ptr(), stream))
        elif self.exchange == "peer":
            o_tab, lse_tab = self._ptr_tables[self.epoch & 1]
            with torch.cuda.device(self.device):
                _lib.check(lib.nvfp4_peer_merge(
                    o_tab.data_ptr(), lse_tab.data_ptr(), self._flags.data_ptr(), self.rank,
                    self.world, self.epoch, self._epoch_state.data_ptr(), self.rows, self.heads_q,
                    out.data_ptr(), f32, self.status.data_ptr(), stream))
        else:
            import torch.distributed as dist

            # A step with NCCL's all-gather between this library's hand-launched kernels did not
            # finish when it was captured into one CUDA graph on two GPUs (the same step finishes
            # with plain launches).  Until that is understood the combination is refused here
            # rather than left to stall a serving process that captures its decode step.
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError(
                    "PageRangeGroup(exchange='nccl') cannot be captured into a CUDA graph: launch it "
                    "with plain launches, or use exchange='fused', 'push' or 'peer', which capture")
            dist.all_gather_into_tensor(self._gathered, self._buf, group=self.group)
            per_copy = self._o_elems + self._lse_elems
            with torch.cuda.device(self.device):
                _lib.check(lib.nvfp4_lse_merge(
                    self._gathered.data_ptr(), per_copy,
                    self._gathered.data_ptr() + 4 * self._o_elems, per_copy, self.world, self.rows,
                    self.heads_q, out.data_ptr(), f32, None, None, stream))
        return out


def decode_page_range(ranges: PageRangeGroup, query: torch.Tensor, key_pages_fp4, key_scales,
                      value_pages_fp4, value_scales, local_table: torch.Tensor,
                      local_seqused_fp4: torch.Tensor, *, out: torch.Tensor, softmax_scale=None,
                      residual_key_pages_bf16=None, residual_value_pages_bf16=None,
                      residual_page_ids=None, seqused_residual=None,
                      trusted_metadata: bool = True, local_splits: int = 1) -> torch.Tensor:
    """One decode step under the page-range split: local partial decode, exchange, merge.

    Every rank passes the SAME query rows, its own pages and its local table
    (:func:`local_page_table`); the residual arguments are given on rank 0 only.
    ``local_splits`` > 1 cuts a rank's own page range once more (few rows over a long context
    would otherwise leave most SMs idle); the local partials are merged on the rank first.
    """
    from .nvfp4_decode_kernel import _decode

    rows, heads_q, head_dim = query.shape
    heads_kv = key_pages_fp4.shape[2]
    if softmax_scale is None:
        softmax_scale = head_dim ** -0.5
    partials = ranges.partial_buffers() if local_splits <= 1 else ranges.local_split_buffers(local_splits)
    fused = ranges.exchange == "fused"
    # the decode kernel quantises the BF16 query itself: one launch
    _decode.decode_fp4(
        query_fp4=None, query_scales=None, query_padded_bf16=None, query_bf16=query,
        key_pages_fp4=key_pages_fp4, key_scales=key_scales, value_pages_fp4=value_pages_fp4,
        value_scales=value_scales, fp4_page_table=local_table, seqused_fp4=local_seqused_fp4,
        residual_key_pages_bf16=residual_key_pages_bf16,
        residual_value_pages_bf16=residual_value_pages_bf16, residual_page_ids=residual_page_ids,
        seqused_residual=seqused_residual, softmax_scale=softmax_scale,
        trusted_metadata=trusted_metadata, num_splits=max(1, local_splits), _partials=partials,
        _exchange=ranges.exchange_args(out) if fused else None)
    if fused:
        return out
    if ranges.exchange == "push":
        return ranges.merge(out, local_splits)   # folds the local splits in the same launch
    if local_splits > 1:
        ranges.fold_local_splits(local_splits)
    return ranges.merge(out)
