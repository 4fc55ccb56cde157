"""Shared builders for the GPU parity tests: move a seeded problem to the device,
quantise it with the library, and evaluate the numpy oracle on the library's own
dequantised bytes."""

from __future__ import annotations

import numpy as np
import torch

import nvfp4_oracle as O

PAGE = 128


def bf16_tensor(x: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(device).to(torch.bfloat16)


def to_np(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.bfloat16, torch.float16):
        t = t.float()
    if t.dtype in (torch.float8_e4m3fn, torch.float4_e2m1fn_x2):
        t = t.view(torch.uint8)
    return t.detach().cpu().numpy()


def scale_bytes(scales: torch.Tensor) -> np.ndarray:
    """[pages, Hkv*1024] bytes of a quantiser scale view (dense or pitched)."""
    pages = scales.shape[0]
    heads = scales.shape[-1]
    flat = scales.view(torch.uint8).as_strided((pages, heads * 1024), (scales.stride(0), 1),
                                               scales.storage_offset())
    return flat.cpu().numpy()


class Problem:
    """A decode problem resident on the GPU in the operator's own layouts."""

    def __init__(self, case: dict, device, key_shift=None):
        from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _quantize

        self.case = case
        self.device = device
        self.q = bf16_tensor(case["q"], device)
        self.k_pages = bf16_tensor(case["k_pages"], device)
        self.v_pages = bf16_tensor(case["v_pages"], device)
        self.page_table = torch.from_numpy(case["page_table"]).to(device)
        self.seqused_fp4 = torch.from_numpy(case["seqused_fp4"]).to(device)
        self.seqused_residual = torch.from_numpy(case["seqused_residual"]).to(device)
        self.residual_page_ids = torch.from_numpy(case["residual_page_ids"]).to(device)
        self.softmax_scale = case["softmax_scale"]
        self.k_fp4, self.k_sf = _quantize.quantize_key_pages(self.k_pages)
        self.v_fp4, self.v_sf = _quantize.quantize_value_pages(self.v_pages)
        self.heads_q = self.q.shape[1]
        self.heads_kv = self.k_pages.shape[2]

    def decode(self, **kw):
        from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import fp4_decode

        args = dict(
            query=self.q,
            key_pages_fp4=self.k_fp4,
            key_scales=self.k_sf,
            value_pages_fp4=self.v_fp4,
            value_scales=self.v_sf,
            fp4_page_table=self.page_table,
            seqused_fp4=self.seqused_fp4,
            residual_key_pages_bf16=self.k_pages,
            residual_value_pages_bf16=self.v_pages,
            residual_page_ids=self.residual_page_ids,
            seqused_residual=self.seqused_residual,
            softmax_scale=self.softmax_scale,
        )
        args.update(kw)
        return fp4_decode(**args)

    def decode_direct(self, **kw):
        """The host layer under ``fp4_decode`` (BF16 query quantised in the launch); takes
        ``status`` and the other arguments the operator's signature does not carry."""
        from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode

        args = dict(
            query_fp4=None, query_scales=None, query_padded_bf16=None, query_bf16=self.q,
            key_pages_fp4=self.k_fp4, key_scales=self.k_sf, value_pages_fp4=self.v_fp4,
            value_scales=self.v_sf, fp4_page_table=self.page_table, seqused_fp4=self.seqused_fp4,
            residual_key_pages_bf16=self.k_pages, residual_value_pages_bf16=self.v_pages,
            residual_page_ids=self.residual_page_ids, seqused_residual=self.seqused_residual,
            softmax_scale=self.softmax_scale,
        )
        args.update(kw)
        return _decode.decode_fp4(**args)

    def oracle_from_bytes(self, rows=None, splits: int = 1, dequantised_tail_query: bool = False):
        """Oracle fed with the library's dequantised Q/K/V bytes.  With ``splits`` > 1 the
        oracle runs once per page range (the tail goes with range 0) and the partials are
        merged by LSE weight, which is what the split path computes.
        ``dequantised_tail_query``: the tail meets the dequantised NVFP4 query instead of the
        BF16 one (a pre-quantised query passed without its BF16 copy)."""
        from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _quantize

        q_fp4, q_sf = _quantize.quantize_query(self.q, heads_kv=self.heads_kv)
        rows_n = self.q.shape[0]
        storage = q_sf.as_strided((rows_n, self.heads_q * 1024), (self.heads_q * 1024, 1))
        q_dq = O.dequantize_query(to_np(q_fp4), to_np(storage).reshape(rows_n, 1, self.heads_q, 2, 32, 4, 4),
                                  self.heads_kv)
        k_dq = O.dequantize_key_pages(to_np(self.k_fp4), scale_bytes(self.k_sf))
        v_dq = O.dequantize_value_pages(to_np(self.v_fp4), scale_bytes(self.v_sf))
        c = self.case
        sel = slice(None) if rows is None else rows
        common = dict(
            tail_key=c["k_pages"], tail_value=c["v_pages"], tail_ids=c["residual_page_ids"][sel],
            seqused_residual=c["seqused_residual"][sel], softmax_scale=c["softmax_scale"],
        )
        args = (q_dq[sel] if dequantised_tail_query else c["q"][sel], q_dq[sel], k_dq, v_dq,
                c["page_table"][sel], c["seqused_fp4"][sel])
        if splits == 1:
            return O.attention_from_dequantized(*args, **common)
        # an int means the split rule itself; a list gives (page_range function, owns_tail) pieces
        pieces = splits if isinstance(splits, list) else [
            ((lambda n, s=s: O.split_page_range(n, s, splits)), s == 0) for s in range(splits)]
        parts, lses = [], []
        for page_range, owns_tail in pieces:
            o, lse = O.attention_from_dequantized(
                *args, **common, page_range=page_range, owns_tail=owns_tail, return_lse=True)
            parts.append(o)
            lses.append(lse)
        return O.lse_merge(np.stack(parts), np.stack(lses))


def oracle_balanced(prob: "Problem", row: int, target_pages: int):
    """The oracle over the pieces the balanced split cuts ``row`` into: the tail alone (when the
    row holds one), then ceil(pages / target_pages) page ranges; merged by LSE weight."""
    c = prob.case
    pieces = O.balanced_pieces(c["seqused_fp4"][[row]], c["seqused_residual"][[row]], target_pages)[0]
    as_ranges = [((lambda n, first=first, last=last: (first, last)), owns_tail)
                 for first, last, owns_tail in pieces]
    return prob.oracle_from_bytes(rows=[row], splits=as_ranges)


def persistent_ctas(device) -> int:
    """CTAs of the persistent decode launch on this device: two per SM."""
    return 2 * torch.cuda.get_device_properties(device).multi_processor_count


def oracle_persistent(prob: "Problem", tiles=None, with_tail: bool = True):
    """The attention oracle over the pieces the persistent launch cuts this problem into, fed the
    library's own dequantised bytes; ``tiles`` restricts it to some (row, kvh) pairs."""
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _quantize

    c = prob.case
    rows_n = prob.q.shape[0]
    q_fp4, q_sf = _quantize.quantize_query(prob.q, heads_kv=prob.heads_kv)
    storage = q_sf.as_strided((rows_n, prob.heads_q * 1024), (prob.heads_q * 1024, 1))
    q_dq = O.dequantize_query(to_np(q_fp4), to_np(storage).reshape(rows_n, 1, prob.heads_q, 2, 32, 4, 4),
                              prob.heads_kv)
    k_dq = O.dequantize_key_pages(to_np(prob.k_fp4), scale_bytes(prob.k_sf))
    v_dq = O.dequantize_value_pages(to_np(prob.v_fp4), scale_bytes(prob.v_sf))
    tail = dict(tail_key=c["k_pages"], tail_value=c["v_pages"], tail_ids=c["residual_page_ids"],
                seqused_residual=c["seqused_residual"]) if with_tail else {}
    pieces = O.persistent_pieces(
        c["seqused_fp4"], c["seqused_residual"] if with_tail else None,
        c["residual_page_ids"] if with_tail else None, c["k_pages"].shape[0], prob.heads_kv,
        c["page_table"].shape[1], persistent_ctas(prob.device))
    return O.attention_in_pieces(pieces, c["q"], q_dq, k_dq, v_dq, c["page_table"], c["seqused_fp4"],
                                 softmax_scale=c["softmax_scale"], tiles=tiles, **tail), pieces


def interleave_vllm(k_fp4, k_sf, v_fp4, v_sf):
    """Repack dense regions into one [pages, block_bytes] cache and return the four
    carved views (page stride = block pitch), like one vLLM block per page."""
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel.quantize_kv_kernel import scale_view

    pages, _, heads, _ = k_fp4.shape
    kp = pages and k_fp4.reshape(pages, -1)
    ks = torch.from_numpy(scale_bytes(k_sf)).to(k_fp4.device)
    vp = v_fp4.reshape(pages, -1)
    vs = torch.from_numpy(scale_bytes(v_sf)).to(k_fp4.device)
    cache = torch.cat([kp, ks, vp, vs], dim=1).contiguous()
    pitch = cache.shape[1]
    o1 = kp.shape[1]
    o2 = o1 + ks.shape[1]
    o3 = o2 + vp.shape[1]
    flat = cache.view(-1)
    k_view = flat.as_strided((pages, PAGE, heads, 64), (pitch, heads * 64, 64, 1), 0)
    v_view = flat.as_strided((pages, heads, 128, 64), (pitch, 128 * 64, 64, 1), o2)
    ks_view = scale_view(flat, pages, heads, pitch, o1)
    vs_view = scale_view(flat, pages, heads, pitch, o3)
    return cache, k_view, ks_view, v_view, vs_view
