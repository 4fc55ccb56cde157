"""Host side of the paged NVFP4 decode: contract checks and the launch.

Mirrors ``decode_fp4`` / ``decode_fp4_split`` / ``split_k_heuristic`` of the
reference project (``src/nvfp4_decode_kernel/_decode.py:28-86,532-1171``): the
same tensor contracts are enforced with the same complaints, then the work is
handed to ``nvfp4_decode`` of the C ABI on torch's current stream.  With
``trusted_metadata=True`` nothing is read back from the device.
"""

from __future__ import annotations

import math

import torch

from .. import _lib

PAGE_SIZE = 128
HEAD_DIM = 128

# NVFP4_IMPL_* of the C ABI; tests flip this to compare the two decode kernels.
DEFAULT_IMPL = _lib.IMPL_AUTO


def split_k_heuristic(rows: int, heads_kv: int, max_pages_per_row: int, *, sms: int) -> int:
    """Pick a power-of-two split count for a pure-FP4 decode by predicted makespan.

    Model: one CTA per (row, KV head, split); a launch takes
    ``ceil(ctas / sms)`` scheduling rounds and each round costs the pages one CTA
    walks plus a fixed pipeline fill of 8 page-times.  A split is accepted only
    if it beats the unsplit makespan by more than 20 %, and among equals the
    smallest count wins.  ``max_pages_per_row`` is the page table's width, not
    the device-side lengths, so callers should size the table to the batch.
    """
    if rows < 1 or heads_kv < 1 or max_pages_per_row < 2 or sms < 1:
        return 1
    tiles = rows * heads_kv
    fill = 8

    def cost(splits: int) -> int:
        return math.ceil(tiles * splits / sms) * (math.ceil(max_pages_per_row / splits) + fill)

    best, best_cost = 1, None
    for splits in (2, 4, 8, 16, 32):
        if 2 * splits > max_pages_per_row:
            break
        c = cost(splits)
        if best_cost is None or c < best_cost:
            best, best_cost = splits, c
    if best_cost is None or best_cost * 6 >= cost(1) * 5:
        return 1
    return best


def balance_pages_heuristic(total_pages: int, heads_kv: int, *, sms: int, floor: int = 16) -> int:
    """Piece length, in pages, for ``balance_pages`` from what the host knows of a ragged batch.

    Two CTAs are resident per SM, so ``2 * sms`` pieces run at a time; a piece of about 1.5 times
    an even share (``total_pages * heads_kv / (2 * sms)``) measured best on a batch of 32 rows with
    lengths log-uniform in [128, 32768] (pieces of 24 / 32 / 48 / 64 pages: 85 / 80 / 74 / 75 us
    per serving step with an even share of 31): shorter pieces pay the fixed cost of a CTA more
    often, longer ones leave the end of the launch to a few long walks.  Never below ``floor``.
    """
    if total_pages < 1 or heads_kv < 1 or sms < 1:
        return floor
    share = total_pages * heads_kv / (2 * sms)
    return max(floor, math.ceil(1.5 * share))


def wide_piece_pages(page_counts, heads_kv: int, *, sms: int, floor: int = 4, tail_pieces: int = 0) -> int:
    """Piece length, in pages, that cuts rows of ``page_counts`` FP4 pages into at most ``sms``
    pieces per KV head set - one busy CTA per SM, the launch shape of the kernel's wide form
    (``wide_form=True``) - from lengths the caller knows on the host.  The smallest such length,
    never below ``floor``.  ``tail_pieces``: rows that hold a BF16 tail; the balanced split gives
    each of them a piece of its own, which takes an SM as well."""
    counts = [int(n) for n in page_counts if int(n) > 0]
    if not counts or heads_kv < 1 or sms < heads_kv:
        return floor
    budget = sms // heads_kv - max(0, int(tail_pieces))
    if budget < 1:
        return max(floor, max(counts))
    lo, hi = floor, max(floor, max(counts))
    if sum(-(-n // lo) for n in counts) <= budget:
        return lo
    while lo < hi:          # smallest T with sum(ceil(n / T)) <= budget
        mid = (lo + hi) // 2
        if sum(-(-n // mid) for n in counts) <= budget:
            hi = mid
        else:
            lo = mid + 1
    return lo


def wide_form_fits(page_counts, heads_kv: int, piece_pages: int, *, sms: int, tail_pieces: int = 0) -> bool:
    """Whether rows of ``page_counts`` FP4 pages cut into pieces of ``piece_pages`` pages (0: whole
    rows), plus ``tail_pieces`` tail pieces, make at most one CTA per SM - the case the kernel's
    wide form (``wide_form=True``) is built for.  Host arithmetic on lengths the caller knows."""
    pieces = sum(-(-int(n) // piece_pages) if piece_pages > 0 else 1 for n in page_counts if int(n) > 0)
    return heads_kv >= 1 and (pieces + max(0, int(tail_pieces))) * heads_kv <= sms


def _need_cuda(tensor: torch.Tensor, name: str, device: torch.device) -> None:
    if not tensor.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if tensor.device != device:
        raise ValueError(f"{name} must be on {device}, got {tensor.device}")


def _scale_bytes(scales: torch.Tensor, name: str) -> torch.Tensor:
    if scales.dtype is torch.uint8:
        return scales
    if scales.dtype is torch.float8_e4m3fn:
        return scales.view(torch.uint8)
    raise ValueError(f"{name} must contain E4M3 scale-factor bytes")


def _page_pitch_bytes(pages: torch.Tensor, name: str) -> int:
    """Dense below the page axis, free (>= dense, 16-byte aligned) page stride."""
    itemsize = pages.element_size()
    dense = 1
    for axis in range(pages.ndim - 1, 0, -1):
        if pages.stride(axis) != dense:
            raise ValueError(
                f"{name} must be densely packed within a page; axis {axis} has "
                f"stride {pages.stride(axis)}, expected {dense}"
            )
        dense *= pages.shape[axis]
    pitch = pages.stride(0)
    if pitch < dense or (pitch * itemsize) % 16:
        raise ValueError(
            f"{name} needs a page stride of at least {dense} elements, "
            f"aligned to 16 bytes, got {pitch}"
        )
    return pitch * itemsize


def _scale_pitch_bytes(scales: torch.Tensor, name: str) -> int:
    _, _, _, rest_m, _, rest_k, heads = scales.shape
    head_stride = rest_m * rest_k * 512
    pitch = scales.stride(0)
    if scales.stride() != (pitch, 16, 4, rest_k * 512, 1, 512, head_stride):
        raise ValueError(f"{name} must use the scale layout returned by the K/V quantizer")
    if pitch < heads * head_stride or pitch % 512:
        raise ValueError(
            f"{name} needs a page stride of at least {heads * head_stride} bytes, "
            f"aligned to 512, got {pitch}"
        )
    return pitch


def _any(condition: torch.Tensor, message: str) -> None:
    if bool(torch.any(condition).item()):
        raise ValueError(message)


def balanced_workspace_bytes(rows: int, heads_q: int, max_pages: int, balance_pages: int) -> int:
    """Bytes of workspace a ``balance_pages`` decode of this shape needs."""
    return int(_lib.load().nvfp4_decode_balanced_workspace_bytes(rows, heads_q, max_pages, balance_pages))


def persistent_workspace(rows: int, heads_q: int, heads_kv: int, device) -> torch.Tensor | None:
    """Zero-filled scratch for ``decode_fp4(persistent_workspace=...)`` on ``device`` for up to
    ``rows`` rows, or None when the persistent launch does not take the shape.  Allocate it once
    (outside any graph capture) and pass it to every call; calls that share it must not overlap."""
    with torch.cuda.device(device):
        lib = _lib.load()
        if not lib.nvfp4_decode_persistent_supported(rows, heads_q, heads_kv):
            return None
        need = int(lib.nvfp4_decode_persistent_workspace_bytes(rows, heads_q, heads_kv))
    return torch.zeros(need, dtype=torch.uint8, device=device)


def decode_fp4(
    *,
    query_fp4: torch.Tensor | None,
    query_scales: torch.Tensor | None,
    query_padded_bf16: torch.Tensor | None,
    query_bf16: torch.Tensor | None = None,
    key_pages_fp4: torch.Tensor,
    key_scales: torch.Tensor,
    value_pages_fp4: torch.Tensor,
    value_scales: torch.Tensor,
    fp4_page_table: torch.Tensor,
    seqused_fp4: torch.Tensor,
    residual_key_pages_bf16: torch.Tensor | None = None,
    residual_value_pages_bf16: torch.Tensor | None = None,
    residual_page_ids: torch.Tensor | None = None,
    seqused_residual: torch.Tensor | None = None,
    has_bf16: torch.Tensor | None = None,
    softmax_scale: float,
    out: torch.Tensor | None = None,
    out_indices: torch.Tensor | None = None,
    trusted_metadata: bool = False,
    validate_only: bool = False,
    num_splits: int = 1,
    status: torch.Tensor | None = None,
    _partials: tuple[torch.Tensor, torch.Tensor] | None = None,
    _exchange=None,
    programmatic_launch: bool = False,
    _plan_sink: list | None = None,
    append_key: torch.Tensor | None = None,
    append_value: torch.Tensor | None = None,
    key_shift: torch.Tensor | None = None,
    balance_pages: int | None = None,
    workspace: torch.Tensor | None = None,
    reuse_work_list: bool = False,
    persistent_workspace: torch.Tensor | None = None,
    wide_form: bool = False,
    merge_in_launch: bool = False,
) -> torch.Tensor | None:
    """Validate every tensor contract and launch the decode on the current stream.

    ``wide_form`` (a hint): the caller expects at most one busy CTA per SM (rows x KV heads x
    pieces at or below the SM count); see ``NVFP4_DECODE_WIDE_FORM``.

    ``persistent_workspace`` (an extension; from :func:`persistent_workspace`, zero-filled once):
    run the step as ONE persistent launch of two CTAs per SM that share the step's page tiles
    equally, whatever the rows' lengths (``NVFP4_DECODE_PERSISTENT`` of the C ABI).

    ``balance_pages`` (an extension): cut every row into pieces of about that many FP4 pages,
    each row by its own length, instead of one ``num_splits`` for the whole batch; ``workspace``
    (uint8, ``balanced_workspace_bytes`` long) may be passed to keep the call free of
    allocations.  ``reuse_work_list``: ``workspace`` still holds the list of pieces of an earlier
    call with the same lengths and shapes (the layers of one model step), so it is not rebuilt.

    ``query_padded_bf16`` (``[rows, 128, heads_q, 128]``, row 0 of each tile live)
    carries the BF16 query that meets the BF16 residual page.

    ``append_key`` / ``append_value`` (BF16 ``[rows, heads_kv, 128]``, the step's own token of
    every row) fuse the tail append of one-token rows into the launch: the token is stored at
    position ``seqused_residual - 1`` of the row's residual page (``key_shift``, BF16
    ``[heads_kv, 128]``, subtracted from the key first) and the residual caches are written.

    With ``query_fp4`` and ``query_scales`` both None and ``query_bf16`` (BF16
    ``[rows, heads_q, 128]``, unit stride along the channels) given, the decode kernel
    quantises the query itself with the query quantiser's arithmetic: one launch instead of
    two, no scratch, and the same ``query_bf16`` meets the residual page.
    """
    if not torch.cuda.is_available():
        raise RuntimeError("decode_fp4 requires CUDA")
    if not math.isfinite(softmax_scale) or softmax_scale <= 0.0:
        raise ValueError("softmax_scale must be finite and positive")
    fused_query = query_fp4 is None and query_scales is None
    fp4_dtype = torch.float4_e2m1fn_x2
    if fused_query:
        if query_bf16 is None:
            raise ValueError("give query_fp4 + query_scales, or query_bf16 to quantise in the kernel")
        if (
            query_bf16.dtype is not torch.bfloat16
            or query_bf16.ndim != 3
            or query_bf16.shape[0] < 1
            or query_bf16.shape[2] != HEAD_DIM
            or query_bf16.stride(2) != 1
            or query_bf16.stride(0) % 8
            or query_bf16.stride(1) % 8
            or query_bf16.data_ptr() % 16
        ):
            raise ValueError(
                "query_bf16 must be BF16 [rows, heads_q, 128] with unit channel stride and "
                "16-byte aligned rows"
            )
        if query_padded_bf16 is not None:
            raise ValueError("query_padded_bf16 belongs to the pre-quantised query path")
        device = query_bf16.device
        _need_cuda(query_bf16, "query_bf16", device)
        rows, heads_q, _ = query_bf16.shape
    else:
        if query_fp4 is None or query_scales is None:
            raise ValueError("query_fp4 and query_scales must be provided together")
        if query_bf16 is not None:
            raise ValueError("query_bf16 is only read when the kernel quantises the query")
        if query_fp4.ndim != 4:
            raise ValueError("query_fp4 must have shape [rows, 1, heads_q, 64]")
        device = query_fp4.device
        _need_cuda(query_fp4, "query_fp4", device)
        if query_fp4.dtype is not fp4_dtype or not query_fp4.is_contiguous():
            raise ValueError("query_fp4 must be contiguous packed E2M1 FP4")
        rows, query_len, heads_q, packed_dim = query_fp4.shape
        if rows < 1 or query_len != 1 or packed_dim * 2 != HEAD_DIM:
            raise ValueError("query_fp4 must have shape [rows, 1, heads_q, 64]")
    if torch.cuda.get_device_capability(device)[0] != 10:
        raise RuntimeError("decode_fp4 requires an SM100 CUDA device")

    for tensor, name in (
        (key_pages_fp4, "key_pages_fp4"),
        (value_pages_fp4, "value_pages_fp4"),
        *(() if fused_query else ((query_scales, "query_scales"),)),
        (key_scales, "key_scales"),
        (value_scales, "value_scales"),
        (fp4_page_table, "fp4_page_table"),
        (seqused_fp4, "seqused_fp4"),
    ):
        _need_cuda(tensor, name, device)

    packed_types = (torch.uint8, fp4_dtype)
    if (
        key_pages_fp4.dtype not in packed_types
        or key_pages_fp4.ndim != 4
        or key_pages_fp4.shape[1] != PAGE_SIZE
        or key_pages_fp4.shape[3] * 2 != HEAD_DIM
    ):
        raise ValueError("key_pages_fp4 must be packed FP4 with shape [pages, 128, heads_kv, 64]")
    page_count, _, heads_kv, _ = key_pages_fp4.shape
    if value_pages_fp4.dtype not in packed_types or tuple(value_pages_fp4.shape) != (
        page_count, heads_kv, HEAD_DIM, PAGE_SIZE // 2,
    ):
        raise ValueError("value_pages_fp4 must be packed FP4 with shape [pages, heads_kv, 128, 64]")
    k_pitch = _page_pitch_bytes(key_pages_fp4, "key_pages_fp4")
    v_pitch = _page_pitch_bytes(value_pages_fp4, "value_pages_fp4")
    if heads_kv < 1 or heads_q % heads_kv:
        raise ValueError("heads_q must be divisible by heads_kv")
    group = heads_q // heads_kv
    # (the reference takes only ratios that divide 128, _decode.py:617-622: its MMA packs
    # tokens x heads into 128 rows.  Here the heads are the N side of the product, so every ratio
    # up to 8 fits the N = 8 tile; 16 and 32 have tiles of their own.)
    if not (1 <= group <= 8 or group in (16, 32)):
        raise ValueError("the query-heads-per-KV-head ratio must be 1 to 8, 16 or 32")

    want_q_sf = (32, 4, 1, 4, 2, heads_kv, rows)
    want_page_sf = (page_count, 32, 4, 1, 4, 2, heads_kv)
    if not fused_query:
        if tuple(query_scales.shape) != want_q_sf:
            raise ValueError(f"query_scales must have shape {want_q_sf}")
        if query_scales.stride() != (16, 4, heads_q * 1024, 1, 512, 1024, heads_q * 1024):
            raise ValueError("query_scales must use the layout returned by quantize_query")
    if tuple(key_scales.shape) != want_page_sf:
        raise ValueError(f"key_scales must have shape {want_page_sf}")
    if tuple(value_scales.shape) != want_page_sf:
        raise ValueError(f"value_scales must have shape {want_page_sf}")
    key_scales = _scale_bytes(key_scales, "key_scales")
    value_scales = _scale_bytes(value_scales, "value_scales")
    if not fused_query:
        query_scales = _scale_bytes(query_scales, "query_scales")
        if query_scales.storage_offset() != 0:
            raise ValueError("query_scales must start at storage offset zero")
    k_sf_pitch = _scale_pitch_bytes(key_scales, "key_scales")
    v_sf_pitch = _scale_pitch_bytes(value_scales, "value_scales")

    if (
        fp4_page_table.dtype is not torch.int32
        or fp4_page_table.ndim != 2
        or fp4_page_table.shape[0] != rows
        or (fp4_page_table.shape[1] > 1 and fp4_page_table.stride(-1) != 1)
    ):
        raise ValueError("fp4_page_table must be row-major INT32 with shape [rows, max_pages]")
    if (
        seqused_fp4.dtype is not torch.int32
        or tuple(seqused_fp4.shape) != (rows,)
        or not seqused_fp4.is_contiguous()
    ):
        raise ValueError("seqused_fp4 must be contiguous INT32 with shape [rows]")
    max_tokens = fp4_page_table.shape[1] * PAGE_SIZE
    if not trusted_metadata:
        _any(
            (seqused_fp4 < 0) | (seqused_fp4 > max_tokens) | (seqused_fp4 % PAGE_SIZE != 0),
            f"seqused_fp4 values must be page-aligned and in [0, {max_tokens}]",
        )

    residual = (residual_key_pages_bf16, residual_value_pages_bf16, residual_page_ids,
                seqused_residual)
    has_residual = any(item is not None for item in residual)
    if has_residual and not all(item is not None for item in residual):
        raise ValueError(
            "residual_key_pages_bf16, residual_value_pages_bf16, "
            "residual_page_ids, and seqused_residual must be provided together"
        )
    if has_residual:
        # A pre-quantised query may come without its BF16 copy (the reference refuses that,
        # _decode.py:703-707): the tail then meets the dequantised NVFP4 query, whose values
        # (E2M1 x E4M3: six significant bits) are exact in BF16.
        if not fused_query and query_padded_bf16 is not None:
            _need_cuda(query_padded_bf16, "query_padded_bf16", device)
            want_padded = (rows, PAGE_SIZE, heads_q, HEAD_DIM)
            if (
                query_padded_bf16.dtype is not torch.bfloat16
                or tuple(query_padded_bf16.shape) != want_padded
                or not query_padded_bf16.is_contiguous()
            ):
                raise ValueError(
                    f"query_padded_bf16 must be contiguous BF16 with shape {want_padded}"
                )
        for tensor, name in (
            (residual_key_pages_bf16, "residual_key_pages_bf16"),
            (residual_value_pages_bf16, "residual_value_pages_bf16"),
            (residual_page_ids, "residual_page_ids"),
            (seqused_residual, "seqused_residual"),
        ):
            _need_cuda(tensor, name, device)
        if residual_key_pages_bf16.ndim != 4:
            raise ValueError(
                "residual_key_pages_bf16 must be contiguous BF16 with "
                "shape [pages, 128, heads_kv, 128]"
            )
        residual_pages = residual_key_pages_bf16.shape[0]
        want_residual = (residual_pages, PAGE_SIZE, heads_kv, HEAD_DIM)
        if (
            residual_key_pages_bf16.dtype is not torch.bfloat16
            or tuple(residual_key_pages_bf16.shape) != want_residual
            or not residual_key_pages_bf16.is_contiguous()
        ):
            raise ValueError(
                "residual_key_pages_bf16 must be contiguous BF16 with "
                "shape [pages, 128, heads_kv, 128]"
            )
        if (
            residual_value_pages_bf16.dtype is not torch.bfloat16
            or tuple(residual_value_pages_bf16.shape) != want_residual
            or not residual_value_pages_bf16.is_contiguous()
        ):
            raise ValueError("residual_value_pages_bf16 must match the residual K cache")
        for tensor, name in ((residual_page_ids, "residual_page_ids"),
                             (seqused_residual, "seqused_residual")):
            if (
                tensor.dtype is not torch.int32
                or tuple(tensor.shape) != (rows,)
                or not tensor.is_contiguous()
            ):
                raise ValueError(f"{name} must be contiguous INT32 with shape [rows]")
        if not trusted_metadata:
            _any(
                (residual_page_ids < 0) | (residual_page_ids >= residual_pages),
                "residual_page_ids contains an out-of-range physical page ID",
            )
            _any(
                (seqused_residual < 0) | (seqused_residual > PAGE_SIZE),
                "seqused_residual values must be in [0, 128]",
            )
        if has_bf16 is not None:
            _need_cuda(has_bf16, "has_bf16", device)
            if (
                has_bf16.dtype is not torch.bool
                or tuple(has_bf16.shape) != (rows,)
                or not has_bf16.is_contiguous()
            ):
                raise ValueError("has_bf16 must be contiguous BOOL with shape [rows]")
            if not trusted_metadata:
                _any(has_bf16 != (seqused_residual > 0),
                     "has_bf16 must agree with seqused_residual > 0")
    elif has_bf16 is not None:
        raise ValueError("has_bf16 requires the BF16 residual cache arguments")

    if out is None and out_indices is not None:
        raise ValueError("out_indices needs the out it indexes into")
    if out is not None:
        _need_cuda(out, "out", device)
        if (
            out.dtype is not torch.bfloat16
            or out.ndim != 3
            or tuple(out.shape[1:]) != (heads_q, HEAD_DIM)
            or not out.is_contiguous()
        ):
            raise ValueError("out must be contiguous BF16 with shape [output_rows, heads_q, 128]")
        if out_indices is None:
            if out.shape[0] < rows:
                raise ValueError(
                    f"out needs at least {rows} rows when no out_indices say "
                    f"where they go, found {out.shape[0]}"
                )
        else:
            _need_cuda(out_indices, "out_indices", device)
            if (
                out_indices.dtype is not torch.int32
                or tuple(out_indices.shape) != (rows,)
                or not out_indices.is_contiguous()
            ):
                raise ValueError("out_indices must be contiguous INT32 with shape [rows]")
            if not trusted_metadata:
                _any((out_indices < 0) | (out_indices >= out.shape[0]),
                     "out_indices contains an out-of-range output row")
    if status is not None and (
        status.dtype is not torch.int32 or status.numel() != 1 or status.device != device
    ):
        raise ValueError("status must be a one-element INT32 tensor on the query's device")
    if (append_key is None) != (append_value is None):
        raise ValueError("append_key and append_value must be provided together")
    if append_key is not None:
        if not has_residual:
            raise ValueError("the fused tail append needs the BF16 residual cache arguments")
        for tensor, name in ((append_key, "append_key"), (append_value, "append_value")):
            _need_cuda(tensor, name, device)
            if (
                tensor.dtype is not torch.bfloat16
                or tuple(tensor.shape) != (rows, heads_kv, HEAD_DIM)
                or tensor.stride(2) != 1
                or tensor.stride(1) != HEAD_DIM
                or tensor.stride(0) % 8
                or tensor.data_ptr() % 16
            ):
                raise ValueError(
                    f"{name} must be BF16 [rows, heads_kv, 128] with contiguous tokens' heads and "
                    "16-byte aligned rows"
                )
        if key_shift is not None:
            _need_cuda(key_shift, "key_shift", device)
            if (
                key_shift.dtype is not torch.bfloat16
                or tuple(key_shift.shape) != (heads_kv, HEAD_DIM)
                or not key_shift.is_contiguous()
            ):
                raise ValueError("key_shift must be contiguous BF16 with shape [heads_kv, 128]")
    elif key_shift is not None:
        raise ValueError("key_shift is only read together with append_key / append_value")

    if validate_only:
        return None

    if out is None and _partials is None:
        out = torch.empty(rows, heads_q, HEAD_DIM, dtype=torch.bfloat16, device=device)
    if balance_pages is not None and persistent_workspace is not None:
        raise ValueError("balance_pages and persistent_workspace are two ways to cut the step; give one")
    if balance_pages is not None:
        if not isinstance(balance_pages, int) or balance_pages < 1:
            raise ValueError(f"balance_pages must be a positive integer, got {balance_pages!r}")
        if num_splits != 1 or _partials is not None or out_indices is not None or _exchange is not None:
            raise ValueError("balance_pages replaces num_splits; it takes neither partial buffers, "
                             "out_indices nor the cross-GPU exchange")
        if programmatic_launch:
            raise ValueError("balance_pages cannot be combined with programmatic_launch")
        need = balanced_workspace_bytes(rows, heads_q, fp4_page_table.shape[1], balance_pages)
        if reuse_work_list and workspace is None:
            raise ValueError("reuse_work_list needs the workspace of the call that built the list")
        if workspace is None:
            workspace = torch.empty(need, dtype=torch.uint8, device=device)
        elif (workspace.dtype is not torch.uint8 or workspace.device != device or workspace.numel() < need
              or not workspace.is_contiguous() or workspace.data_ptr() % 16):
            raise ValueError(f"workspace must be contiguous 16-byte aligned uint8 of at least {need} bytes")
    elif workspace is not None or reuse_work_list:
        raise ValueError("workspace and reuse_work_list are only taken together with balance_pages")
    elif persistent_workspace is not None:
        if num_splits != 1 or _partials is not None or _exchange is not None:
            raise ValueError("the persistent launch writes the final rows: no num_splits, partial "
                             "buffers or cross-GPU exchange")
        with torch.cuda.device(device):
            need = int(_lib.load().nvfp4_decode_persistent_workspace_bytes(rows, heads_q, heads_kv))
        if (persistent_workspace.dtype is not torch.uint8 or persistent_workspace.device != device
                or persistent_workspace.numel() < need or not persistent_workspace.is_contiguous()
                or persistent_workspace.data_ptr() % 16):
            raise ValueError(f"persistent_workspace must be contiguous 16-byte aligned uint8 of at least {need} bytes")
        workspace = persistent_workspace
    elif num_splits > 1 and _partials is None:
        need = _lib.load().nvfp4_decode_workspace_bytes(rows, heads_q, num_splits)
        workspace = torch.empty(need, dtype=torch.uint8, device=device)

    args = _lib.DecodeArgs()
    if fused_query:
        args.q_bf16 = query_bf16.data_ptr()
        args.q_bf16_row_stride = query_bf16.stride(0)
        args.q_bf16_head_stride = query_bf16.stride(1)
    else:
        args.q_fp4 = query_fp4.data_ptr()
        args.q_sf = query_scales.data_ptr()
    if query_padded_bf16 is not None:
        args.q_bf16 = query_padded_bf16.data_ptr()
        args.q_bf16_row_stride = query_padded_bf16.stride(0)
        args.q_bf16_head_stride = query_padded_bf16.stride(2)
    args.k_packed = key_pages_fp4.data_ptr()
    args.k_pitch = k_pitch
    args.k_sf = key_scales.data_ptr()
    args.k_sf_pitch = k_sf_pitch
    args.v_packed = value_pages_fp4.data_ptr()
    args.v_pitch = v_pitch
    args.v_sf = value_scales.data_ptr()
    args.v_sf_pitch = v_sf_pitch
    args.num_pages = page_count
    args.page_table = fp4_page_table.data_ptr()
    args.page_table_row_stride = fp4_page_table.stride(0) if rows > 1 else fp4_page_table.shape[1]
    args.max_pages = fp4_page_table.shape[1]
    args.seqused_fp4 = seqused_fp4.data_ptr()
    if has_residual:
        args.tail_key = residual_key_pages_bf16.data_ptr()
        args.tail_value = residual_value_pages_bf16.data_ptr()
        args.tail_pages = residual_key_pages_bf16.shape[0]
        args.tail_ids = residual_page_ids.data_ptr()
        args.seqused_tail = seqused_residual.data_ptr()
    if out is not None:
        args.out = out.data_ptr()
    args.out_indices = _lib.ptr(out_indices)
    if _partials is not None:
        args.o_partial = _partials[0].data_ptr()
        args.lse_partial = _partials[1].data_ptr()
    args.rows = rows
    args.heads_q = heads_q
    args.heads_kv = heads_kv
    args.softmax_scale = softmax_scale
    args.num_splits = num_splits
    args.impl = DEFAULT_IMPL
    if workspace is not None:
        args.workspace = workspace.data_ptr()
        args.workspace_bytes = workspace.numel()
    args.status = _lib.ptr(status)
    if append_key is not None:
        args.append_key = append_key.data_ptr()
        args.append_value = append_value.data_ptr()
        args.append_key_token_stride = append_key.stride(0)
        args.append_value_token_stride = append_value.stride(0)
        args.key_shift = _lib.ptr(key_shift)
    if programmatic_launch:
        # CTAs may start while the previous kernel in the stream drains; pages, scales, table and
        # lengths must not be that kernel's output (query, tail and outputs may be)
        args.flags = _lib.DECODE_PROGRAMMATIC_LAUNCH
    if reuse_work_list:
        args.flags |= _lib.DECODE_REUSE_WORK_LIST
    if persistent_workspace is not None:
        args.flags |= _lib.DECODE_PERSISTENT
    if wide_form:
        args.flags |= _lib.DECODE_WIDE_FORM
    if merge_in_launch:   # balanced split only: the last piece of a row merges, no merge launch
        args.flags |= _lib.DECODE_MERGE_IN_LAUNCH
    if args.page_table_row_stride < args.max_pages:
        raise ValueError("fp4_page_table rows overlap")
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        if balance_pages is not None:
            _lib.check(_lib.load().nvfp4_decode_balanced(args, balance_pages, stream))
        elif _exchange is not None:   # an _lib.ExchangeArgs: decode and cross-GPU exchange in one launch
            _lib.check(_lib.load().nvfp4_decode_exchange(args, _exchange, stream))
        else:
            _lib.check(_lib.load().nvfp4_decode(args, stream))
    if _plan_sink is not None:
        # the filled argument block of a call that passed every check, for callers that repeat it
        _plan_sink.append((args, rows, heads_q, device))
    if out is None:
        return None
    return out if out_indices is not None else out[:rows]


def decode_fp4_split(
    *,
    query_fp4: torch.Tensor | None,
    query_scales: torch.Tensor | None,
    key_pages_fp4: torch.Tensor,
    key_scales: torch.Tensor,
    value_pages_fp4: torch.Tensor,
    value_scales: torch.Tensor,
    fp4_page_table: torch.Tensor,
    seqused_fp4: torch.Tensor,
    softmax_scale: float,
    num_splits: int,
    query_padded_bf16: torch.Tensor | None = None,
    query_bf16: torch.Tensor | None = None,
    residual_key_pages_bf16: torch.Tensor | None = None,
    residual_value_pages_bf16: torch.Tensor | None = None,
    residual_page_ids: torch.Tensor | None = None,
    seqused_residual: torch.Tensor | None = None,
    has_bf16: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    trusted_metadata: bool = False,
    return_partials: bool = False,
    append_key: torch.Tensor | None = None,
    append_value: torch.Tensor | None = None,
    key_shift: torch.Tensor | None = None,
    wide_form: bool = False,
):
    """Split-KV decode: split ``s`` owns pages ``[s*ceil(n/S), min((s+1)*ceil(n/S), n))``,
    the residual belongs to split 0; partials are merged by LSE weight.

    With ``return_partials=True`` the fp32 partials ``([S, rows, 1, heads, 128],
    [S, rows, heads, 1])`` are returned as well.
    """
    common = dict(
        query_fp4=query_fp4,
        query_scales=query_scales,
        query_padded_bf16=query_padded_bf16,
        query_bf16=query_bf16,
        key_pages_fp4=key_pages_fp4,
        key_scales=key_scales,
        value_pages_fp4=value_pages_fp4,
        value_scales=value_scales,
        fp4_page_table=fp4_page_table,
        seqused_fp4=seqused_fp4,
        residual_key_pages_bf16=residual_key_pages_bf16,
        residual_value_pages_bf16=residual_value_pages_bf16,
        residual_page_ids=residual_page_ids,
        seqused_residual=seqused_residual,
        has_bf16=has_bf16,
        softmax_scale=softmax_scale,
        out=out,
        trusted_metadata=trusted_metadata,
        append_key=append_key,      # the split that owns the residual (split 0) appends
        append_value=append_value,
        key_shift=key_shift,
        wide_form=wide_form,
    )
    if num_splits <= 1 and not return_partials:
        return decode_fp4(**common)
    if query_fp4 is not None:
        rows, _, heads_q, _ = query_fp4.shape
        device = query_fp4.device
    else:
        rows, heads_q, _ = query_bf16.shape
        device = query_bf16.device
    if out is None:
        out = torch.empty(rows, heads_q, HEAD_DIM, dtype=torch.bfloat16, device=device)
        common["out"] = out
    # Every slot is written by the kernel (an empty split stores O = 0, LSE = -inf),
    # so the workspace needs no fill.
    o_part = torch.empty(num_splits, rows, 1, heads_q, HEAD_DIM, dtype=torch.float32,
                         device=device)
    lse_part = torch.empty(num_splits, rows, heads_q, 1, dtype=torch.float32, device=device)
    result = decode_fp4(**common, num_splits=num_splits, _partials=(o_part, lse_part))
    if return_partials:
        return result, o_part, lse_part
    return result
