"""Split decode for callers that cannot allocate.

Some users of this library - a serving engine that has given all free HBM to its KV cache, or
code that cannot afford the device synchronisation an allocation brings mid-step - must not call
cudaMalloc.  ``nvfp4_decode_split_static`` keeps the split partials in an array that belongs to
the library image instead.  This test drives it through the C ABI twice in a row and compares it
with the regular entry point given a caller-owned workspace.
"""

import ctypes

import numpy as np
import pytest
import torch

import inputs
from helpers import Problem, to_np

pytestmark = pytest.mark.gpu


def _args(L, prob, q_fp4, q_sf, padded, out, splits):
    a = L.DecodeArgs()
    a.q_fp4, a.q_sf = q_fp4.data_ptr(), q_sf.data_ptr()
    a.q_bf16, a.q_bf16_row_stride, a.q_bf16_head_stride = padded.data_ptr(), padded.stride(0), padded.stride(2)
    a.k_packed, a.k_pitch = prob.k_fp4.data_ptr(), prob.k_fp4.stride(0)
    a.k_sf, a.k_sf_pitch = prob.k_sf.data_ptr(), prob.k_sf.stride(0)
    a.v_packed, a.v_pitch = prob.v_fp4.data_ptr(), prob.v_fp4.stride(0)
    a.v_sf, a.v_sf_pitch = prob.v_sf.data_ptr(), prob.v_sf.stride(0)
    a.num_pages = prob.k_fp4.shape[0]
    a.page_table, a.page_table_row_stride = prob.page_table.data_ptr(), prob.page_table.stride(0)
    a.max_pages = prob.page_table.shape[1]
    a.seqused_fp4 = prob.seqused_fp4.data_ptr()
    a.tail_key, a.tail_value = prob.k_pages.data_ptr(), prob.v_pages.data_ptr()
    a.tail_pages = prob.k_pages.shape[0]
    a.tail_ids, a.seqused_tail = prob.residual_page_ids.data_ptr(), prob.seqused_residual.data_ptr()
    a.out = out.data_ptr()
    a.rows, a.heads_q, a.heads_kv = prob.q.shape[0], prob.heads_q, prob.heads_kv
    a.softmax_scale = prob.softmax_scale
    a.num_splits, a.impl = splits, L.IMPL_AUTO
    return a


def test_static_workspace_decode_matches_the_regular_entry_point(cuda_device):
    import nvfp4_attn_kernel_b200._lib as L
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _quantize

    lib = L.load()
    assert lib.nvfp4_static_workspace_bytes() == 8 << 20
    stream = torch.cuda.current_stream().cuda_stream
    for seed, lens in ((81, (128 * 7 + 5, 128 * 3, 64)), (82, (128 * 12, 128 * 2 + 100, 128 * 5 + 1))):
        prob = Problem(inputs.attention_case(seed, 3, 32, 8, lens, 1.0, 0.0), cuda_device)
        rows = 3
        q_fp4, q_sf = _quantize.quantize_query(prob.q, heads_kv=8)
        padded = torch.zeros(rows, 128, 32, 128, dtype=torch.bfloat16, device=cuda_device)
        padded[:, 0] = prob.q
        splits = 4
        want = torch.zeros(rows, 32, 128, dtype=torch.bfloat16, device=cuda_device)
        ws = torch.empty(lib.nvfp4_decode_workspace_bytes(rows, 32, splits), dtype=torch.uint8,
                         device=cuda_device)
        a = _args(L, prob, q_fp4, q_sf, padded, want, splits)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        L.check(lib.nvfp4_decode(ctypes.byref(a), stream))
        got = torch.full_like(want, 9.0)
        b = _args(L, prob, q_fp4, q_sf, padded, got, splits)
        # Set-up, as the header describes it: the first call on a device resolves the array's
        # address (the runtime loads the module that holds the array then); a NULL block does
        # just that and is refused.
        assert lib.nvfp4_decode_split_static(None, None) == L.ERR_INVALID
        assert b"null argument block" in lib.nvfp4_decode_split_static_error()
        # Two views of "no allocation" over two calls in a row: torch's caching allocator handed
        # out nothing, and the driver's count of free device memory (which also sees a cudaMalloc
        # made behind torch's back, and the module loader) did not move.
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(cuda_device)
        free_before, total_before = torch.cuda.mem_get_info(cuda_device)
        for _ in range(2):
            rc = lib.nvfp4_decode_split_static(ctypes.byref(b), stream)
            assert rc == 0, lib.nvfp4_decode_split_static_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(cuda_device) == before
        free_after, total_after = torch.cuda.mem_get_info(cuda_device)
        assert total_after == total_before
        assert free_after >= free_before, (free_before, free_after)
        # same kernels, same partials, same merge order: identical, and inside the parity bound
        assert torch.equal(got, want)
        assert np.abs(to_np(got) - prob.oracle_from_bytes(splits=splits)).max() <= 2e-2

    # a request beyond the built-in array is refused with both sizes in the message
    big = _args(L, prob, q_fp4, q_sf, padded, got, 1024)
    big.rows = 4096
    assert lib.nvfp4_decode_split_static(ctypes.byref(big), stream) == L.ERR_INVALID
    message = lib.nvfp4_decode_split_static_error().decode()
    assert "8388608" in message and "need" in message
    one = _args(L, prob, q_fp4, q_sf, padded, got, 1)
    assert lib.nvfp4_decode_split_static(ctypes.byref(one), stream) == L.ERR_INVALID
