"""A scripted serving loop over the whole write + read path, on the GPU, against the oracle.

Per scheduler step: slot control plane -> page work table -> (per layer) tail reset, page
quantisation + tail append with the key shift, decode of the one-token rows -> tail flush after
the last layer.  The script mixes prompts and decodes, crosses page boundaries (so pages get
sealed from the tail), drops a request and reuses its slot.  Checked every step: decode output
against the oracle (2e-2) and, at the end, every sealed block byte-for-byte against the oracle's
quantisers.  This is the sequence the reference project's ``tests/test_nvfp4_vllm.py`` drives
through its backend (``src/nvfp4_vllm/impl.py:103-225``).
"""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import nvfp4_oracle as O
from helpers import bf16_tensor, to_np

pytestmark = pytest.mark.gpu

LAYERS, HEADS_Q, HEADS_KV, DIM = 2, 8, 2, 128
SLOTS, BLOCKS, COLUMNS = 3, 24, 5   # three slots: the fourth request must reuse one
TOL = 2e-2


class Request:
    def __init__(self, name, prompt, blocks):
        self.name, self.prompt, self.blocks = name, prompt, blocks
        self.length = 0
        self.keys = [np.zeros((0, HEADS_KV, DIM), np.float32) for _ in range(LAYERS)]
        self.values = [np.zeros((0, HEADS_KV, DIM), np.float32) for _ in range(LAYERS)]


def oracle_row(request, layer, query, shift, scale, piece=None):
    """Attention of one decode row over the request's whole history, as the cache holds it.
    With ``piece`` the row is cut into ceil(pages / piece) page ranges merged by LSE weight."""
    keys = O.bf16_round(request.keys[layer] - shift[None]) if shift is not None else request.keys[layer]
    values = request.values[layer]
    full = (request.length - 1) // 128
    k_pages = keys[: full * 128].reshape(full, 128, HEADS_KV, DIM)
    v_pages = values[: full * 128].reshape(full, 128, HEADS_KV, DIM)
    tail_k = np.zeros((1, 128, HEADS_KV, DIM), np.float32)
    tail_v = np.zeros_like(tail_k)
    rest = request.length - full * 128
    tail_k[0, :rest] = keys[full * 128:]
    tail_v[0, :rest] = values[full * 128:]
    if full:
        k_dq = O.dequantize_key_pages(*O.quantize_key_pages(k_pages))
        v_dq = O.dequantize_value_pages(*O.quantize_value_pages(v_pages))
    else:
        k_dq = np.zeros((1, 128, HEADS_KV, DIM), np.float32)
        v_dq = np.zeros_like(k_dq)
    q = query[None]
    q_dq = O.dequantize_query(*O.quantize_query(q, HEADS_KV), HEADS_KV)
    table = np.arange(max(full, 1), dtype=np.int32)[None]
    common = dict(tail_key=tail_k, tail_value=tail_v, tail_ids=np.array([0], np.int32),
                  seqused_residual=np.array([rest], np.int32), softmax_scale=scale)
    args = (q, q_dq, k_dq, v_dq, table, np.array([full * 128], np.int32))
    count = max(1, -(-full // piece)) if piece else 1
    if count == 1:
        return O.attention_from_dequantized(*args, **common)[0]
    parts, lses = [], []
    for s in range(count):
        o, lse = O.attention_from_dequantized(
            *args, **common, page_range=(lambda n, s=s: O.split_page_range(n, s, count)),
            owns_tail=s == 0, return_lse=True)
        parts.append(o)
        lses.append(lse)
    return O.lse_merge(np.stack(parts), np.stack(lses))[0]


@pytest.mark.parametrize("fuse_append,piece", [(False, None), (True, None), (True, 1), (False, 2)])
def test_serving_loop(cuda_device, fuse_append, piece):
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import fp4_decode
    from nvfp4_attn_kernel_b200.nvfp4_vllm import layout, promote
    from nvfp4_attn_kernel_b200.nvfp4_vllm.control import ControlPlane
    from nvfp4_attn_kernel_b200.nvfp4_vllm.runtime import LayerRuntime, piece_pages
    from nvfp4_attn_kernel_b200.nvfp4_vllm.write import (PageWorkTable, reset_new_request_tails,
                                                         write_kv)

    rng = np.random.default_rng(0xE61)
    dev = cuda_device
    scale = DIM ** -0.5
    plane = ControlPlane(max_num_seqs=SLOTS, max_num_batched_tokens=1024, device=dev)
    work = PageWorkTable(max_num_seqs=SLOTS, max_num_batched_tokens=1024, device=dev)
    runtime = LayerRuntime(num_layers=LAYERS, num_slots=SLOTS, num_heads=HEADS_Q,
                           num_kv_heads=HEADS_KV, head_dim=DIM, device=dev)
    scratch, built = [None], set()   # the cut steps' scratch and which (step, shape) lists it holds
    shift_np = O.bf16_round(rng.standard_normal((LAYERS, HEADS_KV, DIM)).astype(np.float32) * 2)
    runtime.key_shift = bf16_tensor(shift_np, dev)
    caches = [torch.zeros(BLOCKS, layout.page_bytes(HEADS_KV), dtype=torch.uint8, device=dev)
              for _ in range(LAYERS)]

    a = Request("a", 250, [3, 4, 5, 6, 7])
    b = Request("b", 128, [9, 10, 11, 12, 13])
    c = Request("c", 70, [14, 15, 16, 17, 18])
    d = Request("d", 300, [19, 20, 21, 22, 23])
    # who runs in each step, in batch order (one-token rows first, as vLLM reorders them)
    script = [[a, b], [a, b], [b, a], [a, b, c], [a, c, b], [a, c], [a, c], [c, a], [a, c, d],
              [d, a, c], [a, d]]
    checked = 0
    for step_index, batch in enumerate(script):
        query_lens = [r.prompt if r.length == 0 else 1 for r in batch]
        assert [n > 1 for n in query_lens] == sorted(n > 1 for n in query_lens)
        for r, n in zip(batch, query_lens):
            r.length += n
        tokens = sum(query_lens)
        starts = np.concatenate([[0], np.cumsum(query_lens)]).astype(np.int32)
        block_table = torch.tensor([r.blocks for r in batch], dtype=torch.int32, device=dev)
        seq_lens = torch.tensor([r.length for r in batch], dtype=torch.int32, device=dev)
        query_start_loc = torch.from_numpy(starts).to(dev)
        out = plane.prepare(block_table=block_table, seq_lens=seq_lens,
                            query_start_loc=query_start_loc, num_reqs=len(batch),
                            num_actual_tokens=tokens)
        sources, pages = work.build(query_start_loc=query_start_loc, seqused_fp4=out.seqused_fp4,
                                    row_to_slot=out.row_to_slot, block_table=block_table,
                                    num_reqs=len(batch), max_query_len=max(query_lens))
        decode_rows = sum(1 for n in query_lens if n == 1)
        columns = max(1, (max(r.length for r in batch) - 1) // 128)
        for layer in range(LAYERS):
            key = O.bf16_round(rng.standard_normal((tokens, HEADS_KV, DIM)).astype(np.float32) * 1.5
                               + shift_np[layer][None])
            value = O.bf16_round(rng.standard_normal((tokens, HEADS_KV, DIM)).astype(np.float32))
            query = O.bf16_round(rng.standard_normal((tokens, HEADS_Q, DIM)).astype(np.float32))
            for row, r in enumerate(batch):
                r.keys[layer] = np.concatenate([r.keys[layer], key[starts[row]:starts[row + 1]]])
                r.values[layer] = np.concatenate([r.values[layer], value[starts[row]:starts[row + 1]]])
            if layer == 0:
                reset_new_request_tails(tail_key=runtime.tail_key, tail_value=runtime.tail_value,
                                        query_start_loc=query_start_loc, seq_lens=seq_lens,
                                        row_to_slot=out.row_to_slot)
            runtime.expect_layer(layer)
            k_fp4, k_sf, v_fp4, v_sf = runtime.views(layer, caches[layer])
            # a step of one-token rows only may leave its tail copy to the decode launch
            fused = fuse_append and decode_rows == len(batch)
            key_dev, value_dev = bf16_tensor(key, dev), bf16_tensor(value, dev)
            extra = dict(append_key=key_dev, append_value=value_dev,
                         key_shift=runtime.active_key_shift[layer]) if fused else {}
            cut = piece_pages(decode_rows, HEADS_KV, columns, runtime.sm_count, str(piece or 0))
            assert cut == (piece if piece and columns > piece else 0)
            if cut:   # what the backend does with NVFP4_BALANCE_PAGES set to a page count
                need = runtime.balance_need(decode_rows, HEADS_Q, columns, piece)
                if scratch[0] is None or scratch[0].numel() < need:
                    scratch[0] = torch.empty(4 * need, dtype=torch.uint8, device=dev)
                    built.clear()
                list_key = (step_index, decode_rows, columns)
                extra.update(balance_pages=piece, balance_workspace=scratch[0], balance_reuse=list_key in built)
                built.add(list_key)
            if not fused:
                write_kv(key=key_dev, value=value_dev, key_pages_fp4=k_fp4,
                         key_scales=k_sf, value_pages_fp4=v_fp4, value_scales=v_sf,
                         tail_key=runtime.tail_key[layer], tail_value=runtime.tail_value[layer],
                         source_tokens=sources, destination_pages=pages,
                         query_start_loc=query_start_loc, seq_lens=seq_lens,
                         seqused_fp4=out.seqused_fp4, row_to_slot=out.row_to_slot,
                         num_actual_tokens=tokens, key_shift=runtime.active_key_shift[layer])
            if decode_rows:
                got = fp4_decode(
                    query=bf16_tensor(query[:decode_rows], dev), key_pages_fp4=k_fp4,
                    key_scales=k_sf, value_pages_fp4=v_fp4, value_scales=v_sf,
                    fp4_page_table=block_table[:decode_rows, :columns],
                    seqused_fp4=out.seqused_fp4[:decode_rows],
                    residual_key_pages_bf16=runtime.tail_key[layer],
                    residual_value_pages_bf16=runtime.tail_value[layer],
                    residual_page_ids=out.row_to_slot[:decode_rows],
                    seqused_residual=out.seqused_residual[:decode_rows], softmax_scale=scale,
                    trusted_metadata=True, query_padded_scratch=runtime.query_padded,
                    query_fp4_scratch=runtime.query_fp4, query_scales_scratch=runtime.query_scales, **extra)
                got = to_np(got)
                for row in range(decode_rows):
                    want = oracle_row(batch[row], layer, query[row], shift_np[layer], scale,
                                      piece if piece and columns > piece else None)
                    err = float(np.abs(got[row] - want).max())
                    assert err < TOL, (batch[row].name, batch[row].length, layer, err)
                    checked += 1
        promote.launch(SimpleNamespace(promotion_source_tokens=out.promotion_source_tokens,
                                       promotion_pages=out.promotion_pages), runtime)
    plane.raise_for_errors()
    assert checked >= 30

    # every sealed page of every request that is still running, byte for byte
    sealed = 0
    for r in (a, c, d):
        full = r.length // 128   # a page is sealed the step it fills
        if not full:
            continue
        for layer in range(LAYERS):
            keys = r.keys[layer][: full * 128].reshape(full, 128, HEADS_KV, DIM)
            values = r.values[layer][: full * 128].reshape(full, 128, HEADS_KV, DIM)
            want = O.assemble_vllm_blocks(*O.quantize_key_pages(keys, shift_np[layer]),
                                          *O.quantize_value_pages(values))
            got = to_np(caches[layer][torch.tensor(r.blocks[:full], device=dev)])
            assert np.array_equal(got, want), (r.name, layer)
            sealed += full
    assert sealed >= 2 * (2 + 0 + 2)
    # b left after filling exactly one page at its prompt and decoding past it
    want = O.assemble_vllm_blocks(*O.quantize_key_pages(b.keys[0][:128].reshape(1, 128, HEADS_KV, DIM),
                                                        shift_np[0]),
                                  *O.quantize_value_pages(b.values[0][:128].reshape(1, 128, HEADS_KV, DIM)))
    assert np.array_equal(to_np(caches[0][9:10]), want)
