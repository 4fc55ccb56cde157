"""GPU state that one model's NVFP4 attention layers share for their whole lifetime: the BF16
tail of every layer, the carved views of each layer's block array, the query scratch, the
key-shift vector and its measurement, and the layer-order check.

Counterpart of the reference project's ``src/nvfp4_vllm/runtime.py`` (``load_key_shift`` :39-86,
``LayerRuntime`` :89-337).  Everything is allocated once, in the first forward pass (vLLM's
profile run), so the KV cache is sized around it and no decode step allocates.
"""

from __future__ import annotations

import os

import torch

from ..nvfp4_decode_kernel import RESIDUAL_ROW_TILE
from . import layout

PAGE_SIZE = 128
# Path of a safetensors file with one tensor ``key_shift`` [layers, kv_heads, head_dim].
KEY_SHIFT_ENV = "NVFP4_KEY_SHIFT"


# How a decode step's rows are cut into pieces of pages (the balanced split, not in the reference):
# "auto" (default) - piece length from the step's shape, see piece_pages; "0" - never, rows stay
# whole as in the reference; a positive number - pieces of that many pages.
BALANCE_PAGES_ENV = "NVFP4_BALANCE_PAGES"


def piece_pages(rows: int, heads_kv: int, columns: int, sms: int, setting: str | None = None) -> int:
    """Pages per piece for a decode step of ``rows`` rows whose page table is ``columns`` wide, or
    0 to leave the rows whole.

    The host knows the step's shape, not its lengths, so "auto" plans for full rows: pieces of
    1.5 times an even share of ``rows * columns * heads_kv`` page walks over the ``2 * sms``
    resident CTAs, at least 16 pages.  A batch that fills the GPU with whole rows (32 rows x 8 KV
    heads x 32 pages on 148 SMs: share 28, piece 42 > 32 columns) is left alone; one or a few long
    rows (1 row x 8 heads x 256 pages: piece 16, 128 CTAs instead of 8) are cut.  The list of
    pieces itself follows the lengths on the device, so short rows still get one piece.
    """
    from ..nvfp4_decode_kernel._decode import balance_pages_heuristic

    if setting is None:
        setting = os.environ.get(BALANCE_PAGES_ENV, "auto")
    setting = setting.strip().lower() or "auto"
    if setting == "auto":
        piece = balance_pages_heuristic(rows * columns, heads_kv, sms=sms)
    else:
        piece = int(setting)
        if piece < 0:
            raise ValueError(f"{BALANCE_PAGES_ENV} must be 'auto', 0 or a positive page count, got {setting!r}")
    return piece if 0 < piece < columns else 0


def load_key_shift(num_layers: int, num_kv_heads: int, head_dim: int, device, dtype):
    """The per-channel constant subtracted from post-RoPE K on its way into the cache, or None.

    Scores become ``q.k - q.mu`` and ``q.mu`` is the same for every key of a query, so softmax
    is unchanged as long as EVERY stored key is shifted; the constant only shrinks the block
    scales.  Held in the cache's dtype so the subtraction is a single BF16 operation.
    """
    path = os.environ.get(KEY_SHIFT_ENV)
    if not path:
        return None
    from safetensors.torch import load_file

    tensors = load_file(path)
    if "key_shift" not in tensors:
        raise ValueError(f"{path} has no 'key_shift' tensor, found {sorted(tensors)}")
    shift = tensors["key_shift"]
    expected = (num_layers, num_kv_heads, head_dim)
    if tuple(shift.shape) != expected:
        raise ValueError(
            f"{path} holds a key_shift of {tuple(shift.shape)}, this model needs {expected}"
        )
    return shift.to(device=device, dtype=dtype).contiguous()


class LayerRuntime:
    """Tail buffers, cache views and query scratch of one model."""

    def __init__(self, *, num_layers: int, num_slots: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, device, max_pages: int = 0) -> None:
        self.num_layers = num_layers
        self.num_slots = num_slots
        self.num_heads = num_heads
        self.sm_count = (torch.cuda.get_device_properties(device).multi_processor_count
                         if torch.device(device).type == "cuda" else 148)
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.key_shift_enabled = True
        self.key_shift_sum: torch.Tensor | None = None   # set only while measuring
        self.key_shift_tokens = 0

        # zeroed, because attention may read a whole tail page and masked positions must be finite
        shape = (num_layers, num_slots, PAGE_SIZE, num_kv_heads, head_dim)
        self.tail_key = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        self.tail_value = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        self.key_shift = load_key_shift(num_layers, num_kv_heads, head_dim, device,
                                        self.tail_key.dtype)
        # the same storage as one run of tokens: layer l, slot s starts at (l*slots + s)*128
        self.tail_key_tokens = self.tail_key.view(-1, num_kv_heads, head_dim)
        self.tail_value_tokens = self.tail_value.view(-1, num_kv_heads, head_dim)

        # zeroed once and never again (the contract fp4_decode states for caller-owned scratch)
        self.query_padded = torch.zeros(num_slots, RESIDUAL_ROW_TILE, num_heads, head_dim,
                                        dtype=torch.bfloat16, device=device)
        self.query_fp4 = torch.zeros(num_slots, 1, num_heads, head_dim // 2, dtype=torch.uint8,
                                     device=device)
        self.query_scales = torch.zeros(num_slots, 1, num_heads, head_dim // 64, 32, 4, 4,
                                        dtype=torch.uint8, device=device)
        self._views: dict[int, tuple[torch.Tensor, ...]] = {}
        self._by_layer: dict[int, tuple[torch.Tensor, ...]] = {}
        self._bases: torch.Tensor | None = None
        self._expected_layer = 0
        self._balance_workspace: torch.Tensor | None = None
        self._work_list_key: tuple | None = None
        if max_pages > 0:
            self.reserve_balance_workspace(max_pages)

    def reserve_balance_workspace(self, max_pages: int, limit_bytes: int = 256 << 20) -> int:
        """Allocate, once, the scratch of the largest decode step that ``piece_pages`` would cut:
        any row count up to the slot count and any page-table width up to the model's longest
        context (a step's width follows its longest row, and the need is not monotone in it: the
        piece length is rounded up from the width).  Called with the other allocations of the
        first forward pass, so the KV cache is sized around it and no decode step allocates.
        Returns the bytes reserved (0 when nothing would be cut, or when the worst case is larger
        than ``limit_bytes``: steps then leave their rows whole)."""
        worst = self.balance_need_worst(max_pages)
        if not 0 < worst <= limit_bytes:
            return 0
        self._balance_workspace = torch.empty(worst, dtype=torch.uint8, device=self.tail_key.device)
        return worst

    def balance_need_worst(self, max_pages: int) -> int:
        """The largest ``balance_need`` over every step shape the policy can meet."""
        worst = 0
        for rows in range(1, self.num_slots + 1):
            for columns in range(1, max_pages + 1):
                piece = piece_pages(rows, self.num_kv_heads, columns, self.sm_count)
                if piece:
                    worst = max(worst, self.balance_need(rows, self.num_heads, columns, piece))
        return worst

    @staticmethod
    def balance_need(rows: int, heads_q: int, columns: int, piece: int) -> int:
        """Bytes of scratch a step of this shape needs when cut into pieces of ``piece`` pages:
        the arithmetic of ``nvfp4_decode_balanced_workspace_bytes`` (partial outputs and LSEs of
        every possible piece, the list of pieces, two ints per row; each part rounded up to 16)."""
        capacity = 2 * rows + rows * columns // piece
        up16 = lambda n: (n + 15) & ~15   # noqa: E731
        return (up16(capacity * heads_q * 128 * 4) + up16(capacity * heads_q * 4) + up16(capacity * 16)
                + 2 * up16(rows * 4) + up16(rows * heads_q * 4))

    def balance_workspace(self, rows: int, heads_q: int, columns: int, balance_pages: int):
        """Scratch for a decode with a split count per row, or None when the reserved scratch is
        too small for this step (it then runs with whole rows).  A buffer that was handed out is
        never released or replaced: a captured CUDA graph holds its address."""
        need = self.balance_need(rows, heads_q, columns, balance_pages)
        held = self._balance_workspace
        if held is None:
            # nothing was reserved (a runtime built without a model length): allocate once, for
            # the largest shape this table width allows, and keep it for good
            held = torch.empty(max(need, self.balance_need_worst(columns)), dtype=torch.uint8,
                               device=self.tail_key.device)
            self._balance_workspace = held
        return held if held.numel() >= need else None

    def work_list_reusable(self, key: tuple) -> bool:
        """Layers of one step share the list of pieces that the step's first cut layer built.
        ``key`` names the step and its shape (lengths tensor, rows, columns, piece, scratch): True
        if a list for exactly that is in the scratch already, else the caller builds it and the
        key is remembered."""
        if self._work_list_key == key:
            return True
        self._work_list_key = key
        return False

    @property
    def tail_bytes(self) -> int:
        return 2 * self.tail_key.numel() * self.tail_key.element_size()

    @property
    def active_key_shift(self) -> torch.Tensor | None:
        """What the write path should subtract, or None to store K as it is."""
        return self.key_shift if self.key_shift_enabled else None

    def set_key_shift_enabled(self, enabled: bool) -> None:
        """Turn the shift on or off; only valid between requests (cached keys keep the setting
        they were written under)."""
        if enabled and self.key_shift is None:
            raise ValueError(
                "no shift has been loaded or measured, so there is nothing to enable"
            )
        self.key_shift_enabled = enabled

    def begin_key_shift_measurement(self) -> None:
        """Measure the K mean instead of removing it, until told to stop."""
        self.key_shift = None
        self.key_shift_sum = torch.zeros(self.num_layers, self.num_kv_heads, self.head_dim,
                                         dtype=torch.float64, device=self.tail_key.device)
        self.key_shift_tokens = 0

    def finish_key_shift_measurement(self) -> torch.Tensor:
        """Freeze what was measured (fp64 mean, rounded once to the cache dtype) and apply it."""
        if self.key_shift_sum is None or self.key_shift_tokens == 0:
            raise ValueError(
                "no tokens were measured, so there is no mean to subtract; "
                "begin_key_shift_measurement must precede a forward pass"
            )
        self.key_shift = (self.key_shift_sum / self.key_shift_tokens).to(self.tail_key.dtype)
        self.key_shift_enabled = True
        self.key_shift_sum = None
        self.key_shift_tokens = 0
        return self.key_shift

    def views(self, layer_index: int, kv_cache: torch.Tensor) -> tuple[torch.Tensor, ...]:
        """The four NVFP4 regions of one layer's block array (cached by the array's address)."""
        key = kv_cache.data_ptr()
        carved = self._views.get(key)
        if carved is None:
            carved = layout.carve(kv_cache, self.num_kv_heads, self.head_dim)
            self._views[key] = carved
        if self._by_layer.get(layer_index) is not carved:
            self._by_layer[layer_index] = carved
            self._bases = None
        return carved

    @property
    def destination_bases(self) -> torch.Tensor:
        """int64 ``[4, layers]``: where each layer's K packed, K scales, V packed, V scales start."""
        if self._bases is None:
            missing = [i for i in range(self.num_layers) if i not in self._by_layer]
            if missing:
                raise ValueError(
                    f"layers {missing} have not written their KV cache, so "
                    "promotion has no address to send their pages to"
                )
            self._bases = torch.tensor(
                [[self._by_layer[layer][region].data_ptr() for layer in range(self.num_layers)]
                 for region in range(4)],
                dtype=torch.int64, device=self.tail_key.device)
        return self._bases

    def layer_regions(self, layer_index: int) -> tuple[torch.Tensor, ...]:
        return self._by_layer[layer_index]

    def expect_layer(self, layer_index: int) -> None:
        """Refuse a step whose layers do not run in index order (the flush fires after the
        highest index and must come after every layer wrote its share of the boundary token)."""
        if layer_index != self._expected_layer:
            expected = self._expected_layer
            self._expected_layer = (layer_index + 1) % self.num_layers
            raise ValueError(
                f"layer {layer_index} ran where layer {expected} was expected; "
                "promotion assumes layers run in index order"
            )
        self._expected_layer = (layer_index + 1) % self.num_layers
