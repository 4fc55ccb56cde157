"""GPU parity of the decode operator against the numpy oracle (tolerance: max-abs
2e-2 on BF16 outputs, the bound the project states for this path), the golden
vectors, and the operator's edge-case contract."""

import os

import numpy as np
import pytest
import torch

import inputs
import nvfp4_oracle as O
from helpers import Problem, bf16_tensor, interleave_vllm, to_np

pytestmark = pytest.mark.gpu

TOL = 2e-2          # max-abs vs the oracle fed the library's own dequantised bytes
# vs the golden output of the reference's oracle, which quantises Q/K/V from BF16 with its own
# tie rule (exact E2M1 midpoints go down, the hardware converter rounds them to even): 0.6 % of
# the quantised elements differ by one step, which moves single outputs by up to ~0.06 at
# N(0,1) inputs.  Informational bound; the parity bound is TOL above.
TOL_E2E = 1e-1
GOLD = os.path.join(os.path.dirname(__file__), "golden")

IMPLS = ["generic", "sm100"]


def _set_impl(name):
    import nvfp4_attn_kernel_b200._lib as L
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode

    _decode.DEFAULT_IMPL = {"generic": L.IMPL_GENERIC, "sm100": L.IMPL_SM100, "auto": L.IMPL_AUTO}[name]


@pytest.fixture(params=IMPLS)
def impl(request):
    _skip_if_unsupported(request.param, 8, 2)
    _set_impl(request.param)
    yield request.param
    _set_impl("auto")


def _case(name):
    if name == "config1":
        return inputs.config1(0)
    return inputs.attention_case(*inputs.SMALL_CASES[name])


def _skip_if_unsupported(impl, heads_q, heads_kv):
    import nvfp4_attn_kernel_b200._lib as L

    code = {"generic": L.IMPL_GENERIC, "sm100": L.IMPL_SM100}[impl]
    if not L.load().nvfp4_decode_impl_available(code, heads_q, heads_kv):
        pytest.skip(f"the {impl} kernel does not take {heads_q}/{heads_kv} heads")


@pytest.mark.parametrize("name", list(inputs.SMALL_CASES) + ["config1"])
def test_decode_matches_oracle(cuda_device, impl, name):
    case = _case(name)
    _skip_if_unsupported(impl, case["q"].shape[1], case["k_pages"].shape[2])
    prob = Problem(case, cuda_device)
    out = to_np(prob.decode())
    want = prob.oracle_from_bytes()
    assert np.isfinite(out).all()
    assert np.abs(out - want).max() <= TOL, np.abs(out - want).max()
    gold = np.load(os.path.join(GOLD, "attention.npz"))[name]
    assert np.abs(out - gold).max() <= TOL_E2E
    cos = (out * gold).sum() / np.sqrt((out * out).sum() * (gold * gold).sum())
    assert cos >= 0.99


def test_vllm_block_pitch_is_bit_identical(cuda_device, impl):
    prob = Problem(_case("gqa4_short"), cuda_device)
    dense = prob.decode()
    cache, kv, ksv, vv, vsv = interleave_vllm(prob.k_fp4, prob.k_sf, prob.v_fp4, prob.v_sf)
    assert cache.shape[1] == O.vllm_block_bytes(prob.heads_kv)
    paged = prob.decode(key_pages_fp4=kv, key_scales=ksv, value_pages_fp4=vv, value_scales=vsv)
    assert torch.equal(dense, paged)


def test_prequantised_query_equals_bf16_query(cuda_device, impl):
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _quantize, fp4_decode

    case = inputs.attention_case(41, 3, 8, 2, (256, 384, 128), 1.0, 0.0)
    case["seqused_fp4"] = np.array([256, 384, 128], dtype=np.int32)  # page-aligned, no tail
    prob = Problem(case, cuda_device)
    common = (prob.k_fp4, prob.k_sf, prob.v_fp4, prob.v_sf, prob.page_table, prob.seqused_fp4)
    a = fp4_decode(prob.q, *common)
    q_fp4, q_sf = _quantize.quantize_query(prob.q, heads_kv=2)
    b = fp4_decode(None, *common, query_fp4=q_fp4, query_scales=q_sf)
    assert torch.equal(a, b)


def test_prequantised_query_with_a_tail_and_no_bf16_copy(cuda_device, impl):
    """The reference refuses a pre-quantised query next to a BF16 residual unless the padded BF16
    query comes along (src/nvfp4_decode_kernel/_decode.py:703-707).  Here the call is served: the
    tail meets the dequantised NVFP4 query.  Checked against the oracle given that same query for
    the tail, whole rows and split; and it differs from the BF16-query result (the tail saw
    another query), within the quantisation error of the query."""
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _quantize, fp4_decode

    case = inputs.attention_case(44, 4, 8, 2, (128 * 3 + 100, 127, 128 * 5 + 1, 128 * 2), 1.0, 0.0)
    prob = Problem(case, cuda_device)
    q_fp4, q_sf = _quantize.quantize_query(prob.q, heads_kv=2)
    tail = dict(residual_key_pages_bf16=prob.k_pages, residual_value_pages_bf16=prob.v_pages,
                residual_page_ids=prob.residual_page_ids, seqused_residual=prob.seqused_residual)
    common = (prob.k_fp4, prob.k_sf, prob.v_fp4, prob.v_sf, prob.page_table, prob.seqused_fp4)
    for splits in (1, 2):
        got = to_np(fp4_decode(None, *common, query_fp4=q_fp4, query_scales=q_sf, num_splits=splits, **tail))
        want = prob.oracle_from_bytes(splits=splits, dequantised_tail_query=True)
        assert np.abs(got - want).max() <= TOL, splits
    with_bf16 = to_np(prob.decode())
    assert 0 < np.abs(got - with_bf16).max() <= 0.25


@pytest.mark.parametrize("heads", [(24, 8), (40, 8), (12, 2), (28, 4)])
def test_group_sizes_that_do_not_divide_128(cuda_device, impl, heads):
    """3, 5, 6 and 7 query heads per KV head (28/4 and 40/8 are shapes of published models).  The
    reference refuses them (src/nvfp4_decode_kernel/_decode.py:617-622: its product packs tokens x
    heads into 128 rows); here the heads are the N side of the product and any count up to 8 fits
    the N = 8 tile.  Whole rows, the uniform split and (tensor-core kernel) the balanced split with
    the tail's own piece, each against the oracle; the query quantised inside the launch equals
    the query quantiser's bytes fed back in."""
    from helpers import oracle_balanced
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _quantize, fp4_decode

    hq, hkv = heads
    _skip_if_unsupported(impl, hq, hkv)
    lengths = (128 * 4 + 77, 128 * 2, 90, 128 * 7 + 127)
    case = inputs.attention_case(500 + hq, len(lengths), hq, hkv, lengths, 1.0, 0.2)
    prob = Problem(case, cuda_device)
    whole = prob.decode()
    assert np.abs(to_np(whole) - prob.oracle_from_bytes()).max() <= TOL
    assert np.abs(to_np(prob.decode(num_splits=4)) - prob.oracle_from_bytes(splits=4)).max() <= TOL
    if impl == "sm100":
        out = to_np(prob.decode(balance_pages=2))
        for row in range(len(lengths)):
            assert np.abs(out[row] - oracle_balanced(prob, row, 2)[0]).max() <= TOL, row
    q_fp4, q_sf = _quantize.quantize_query(prob.q, heads_kv=hkv)
    padded = torch.zeros(len(lengths), 128, hq, 128, dtype=torch.bfloat16, device=cuda_device)
    padded[:, 0] = prob.q
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode

    two_launch = prob.decode_direct(query_fp4=q_fp4, query_scales=q_sf, query_padded_bf16=padded, query_bf16=None)
    assert torch.equal(whole, two_launch)


def test_rows_without_keys_and_padding_rows(cuda_device, impl):
    """CUDA-graph padding rows arrive with both lengths 0 and a tail id of -1; they
    must write zeros, fault nothing and leave live rows bit-identical."""
    case = inputs.attention_case(43, 4, 8, 2, (300, 1, 129, 256), 1.0, 0.0)
    prob = Problem(case, cuda_device)
    base = prob.decode()
    fp4 = prob.seqused_fp4.clone()
    res = prob.seqused_residual.clone()
    ids = prob.residual_page_ids.clone()
    fp4[1], res[1], ids[1] = 0, 0, -1
    table = prob.page_table.clone()
    table[1] = -1  # nothing of a dead row may be dereferenced
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode, _quantize

    out = prob.decode(fp4_page_table=table, seqused_fp4=fp4, seqused_residual=res,
                      residual_page_ids=ids, trusted_metadata=True)
    assert torch.equal(out[[0, 2, 3]], base[[0, 2, 3]])
    assert not out[1].any()
    # zero-length residual contributes exactly nothing: row 3 with its tail cut to 0
    res2 = prob.seqused_residual.clone()
    res2[3] = 0
    out2 = to_np(prob.decode(seqused_residual=res2))
    want = prob.oracle_from_bytes()
    c2 = dict(case)
    c2["seqused_residual"] = to_np(res2)
    prob2 = Problem(c2, cuda_device)
    assert np.abs(out2 - prob2.oracle_from_bytes()).max() <= TOL
    del status, _decode, _quantize, want


def test_poisoned_unused_table_columns_are_never_read(cuda_device, impl):
    case = inputs.attention_case(45, 2, 8, 2, (200, 600), 1.0, 0.0)
    prob = Problem(case, cuda_device)
    base = prob.decode()
    table = prob.page_table.clone()
    used = (prob.seqused_fp4 // 128).tolist()
    for r, n in enumerate(used):
        table[r, n:] = 0x7FFFFFF0
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode, _quantize

    q_fp4, q_sf = _quantize.quantize_query(prob.q, heads_kv=2)
    padded = torch.zeros(2, 128, 8, 128, dtype=torch.bfloat16, device=cuda_device)
    padded[:, 0] = prob.q
    out = _decode.decode_fp4(
        query_fp4=q_fp4, query_scales=q_sf, query_padded_bf16=padded,
        key_pages_fp4=prob.k_fp4, key_scales=prob.k_sf, value_pages_fp4=prob.v_fp4,
        value_scales=prob.v_sf, fp4_page_table=table, seqused_fp4=prob.seqused_fp4,
        residual_key_pages_bf16=prob.k_pages, residual_value_pages_bf16=prob.v_pages,
        residual_page_ids=prob.residual_page_ids, seqused_residual=prob.seqused_residual,
        softmax_scale=prob.softmax_scale, trusted_metadata=True, status=status)
    assert torch.equal(out, base)
    assert int(status.item()) == 0
    # a bad id INSIDE the used range is skipped and reported, never dereferenced
    table[1, 0] = 0x7FFFFFF0
    _decode.decode_fp4(
        query_fp4=q_fp4, query_scales=q_sf, query_padded_bf16=padded,
        key_pages_fp4=prob.k_fp4, key_scales=prob.k_sf, value_pages_fp4=prob.v_fp4,
        value_scales=prob.v_sf, fp4_page_table=table, seqused_fp4=prob.seqused_fp4,
        residual_key_pages_bf16=prob.k_pages, residual_value_pages_bf16=prob.v_pages,
        residual_page_ids=prob.residual_page_ids, seqused_residual=prob.seqused_residual,
        softmax_scale=prob.softmax_scale, trusted_metadata=True, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & 1


def test_non_finite_bytes_past_the_tail_length_do_not_reach_the_output(cuda_device, impl):
    case = inputs.attention_case(47, 2, 8, 2, (200, 130), 1.0, 0.0)
    prob = Problem(case, cuda_device)
    base = prob.decode()
    k2, v2 = prob.k_pages.clone(), prob.v_pages.clone()
    for r in range(2):
        pid = int(case["residual_page_ids"][r])
        n = int(case["seqused_residual"][r])
        k2[pid, n:] = float("nan")
        v2[pid, n:] = float("inf")
    out = prob.decode(residual_key_pages_bf16=k2, residual_value_pages_bf16=v2)
    assert torch.equal(out, base)


def test_out_buffer_scatter_and_row_indices(cuda_device, impl):
    case = inputs.attention_case(49, 3, 8, 2, (72 + 256, 127, 384), 1.0, 0.0)
    prob = Problem(case, cuda_device)
    base = prob.decode()
    out = torch.full((6, 8, 128), 7.0, dtype=torch.bfloat16, device=cuda_device)
    got = prob.decode(out=out)
    assert got.data_ptr() == out.data_ptr() and tuple(got.shape) == (3, 8, 128)
    assert torch.equal(out[:3], base) and (out[3:] == 7.0).all()
    out.fill_(7.0)
    idx = torch.tensor([4, 1, 3], dtype=torch.int32, device=cuda_device)
    got = prob.decode(out=out, out_indices=idx)
    assert tuple(got.shape) == (6, 8, 128)
    assert torch.equal(out[[4, 1, 3]], base) and (out[[0, 2, 5]] == 7.0).all()
    # query_row_indices picks rows out of a wider query
    wide = torch.zeros(7, 8, 128, dtype=torch.bfloat16, device=cuda_device)
    wide[[5, 0, 2]] = prob.q
    rows = torch.tensor([5, 0, 2], dtype=torch.int32, device=cuda_device)
    assert torch.equal(prob.decode(query=wide, query_row_indices=rows), base)


@pytest.mark.parametrize("splits", [2, 4, 8])
def test_split_kv_matches_unsplit_and_oracle(cuda_device, impl, splits):
    case = inputs.attention_case(51, 3, 8, 2, (1024 + 17, 128 * 5, 60), 1.0, 0.0)
    prob = Problem(case, cuda_device)
    base = to_np(prob.decode())
    out = to_np(prob.decode(num_splits=splits))
    # a split quantises P against its own running maximum, so it is not bit-equal to the
    # unsplit walk; both stay inside the reference's own gate for this comparison
    assert np.abs(out - base).max() <= 5e-2
    # the oracle run split by split, merged by LSE weight
    want = prob.oracle_from_bytes(splits=splits)
    assert np.abs(out - want).max() <= TOL


def test_split_partials_and_merge_entry_points(cuda_device, impl):
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode, _quantize
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel.split_k_combine import flash_attn_combine

    case = inputs.attention_case(53, 2, 8, 2, (128 * 6, 128 * 2), 1.0, 0.0)
    case["seqused_fp4"] = np.array([768, 256], dtype=np.int32)
    prob = Problem(case, cuda_device)
    q_fp4, q_sf = _quantize.quantize_query(prob.q, heads_kv=2)
    out, o_part, lse_part = _decode.decode_fp4_split(
        query_fp4=q_fp4, query_scales=q_sf, key_pages_fp4=prob.k_fp4, key_scales=prob.k_sf,
        value_pages_fp4=prob.v_fp4, value_scales=prob.v_sf, fp4_page_table=prob.page_table,
        seqused_fp4=prob.seqused_fp4, softmax_scale=prob.softmax_scale, num_splits=4,
        return_partials=True)
    lse = to_np(lse_part)[..., 0]
    assert np.isneginf(lse[2:, 1]).all()          # row 1 has 2 pages: splits 2, 3 are empty
    assert np.isfinite(lse[:2, 1]).all()
    assert np.isfinite(lse[:3, 0]).all()          # row 0 has 6 pages, 2 per split: split 3 is empty
    assert np.isneginf(lse[3, 0]).all()
    assert not to_np(o_part)[2:, 1].any()
    merged, merged_lse = flash_attn_combine(o_part, lse_part.transpose(-1, -2), out_dtype=torch.bfloat16)
    assert torch.equal(merged[:, 0], out)
    want, want_lse = O.lse_merge(to_np(o_part)[:, :, 0], lse, return_lse=True)
    assert np.abs(to_np(merged)[:, 0] - want).max() <= 1e-2
    assert np.abs(to_np(merged_lse)[:, 0] - want_lse).max() <= 1e-4
    f32, _ = flash_attn_combine(o_part, lse_part.transpose(-1, -2), out_dtype=torch.float32,
                                return_lse=False)
    assert np.abs(to_np(f32)[:, 0] - want).max() <= 1e-5


def test_repeated_calls_are_bitwise_identical(cuda_device, impl):
    case = inputs.attention_case(55, 18, 8, 1, tuple([513] * 18), 1.0, 0.0)
    prob = Problem(case, cuda_device)
    first = prob.decode()
    first_split = prob.decode(num_splits=4)
    for _ in range(8):
        assert torch.equal(prob.decode(), first)
        assert torch.equal(prob.decode(num_splits=4), first_split)


def test_refusals(cuda_device):
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import fp4_decode

    case = inputs.attention_case(57, 2, 16, 1, (256, 256), 0.3, 0.0)
    case["seqused_fp4"] = np.array([256, 256], dtype=np.int32)
    prob = Problem(case, cuda_device)
    common = (prob.k_fp4, prob.k_sf, prob.v_fp4, prob.v_sf, prob.page_table, prob.seqused_fp4)
    for shape, dtype, complaint in (
        ((2, 16, 128), torch.float16, "out must be contiguous BF16"),
        ((1, 16, 128), torch.bfloat16, "out needs at least 2 rows"),
        ((2, 17, 128), torch.bfloat16, "out must be contiguous BF16"),
    ):
        for splits in (1, 2):
            with pytest.raises(ValueError, match=complaint):
                fp4_decode(prob.q, *common, out=torch.zeros(shape, dtype=dtype, device=cuda_device),
                           num_splits=splits)
    idx = torch.zeros(2, dtype=torch.int32, device=cuda_device)
    out = torch.zeros(2, 16, 128, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(ValueError, match="cannot be combined with out_indices"):
        fp4_decode(prob.q, *common, out=out, out_indices=idx, num_splits=2)
    with pytest.raises(ValueError, match="complete residual"):
        fp4_decode(prob.q, *common, residual_key_pages_bf16=prob.k_pages, num_splits=2)
    with pytest.raises(ValueError, match="must be provided together"):
        fp4_decode(prob.q, *common, residual_key_pages_bf16=prob.k_pages)
    bad = prob.seqused_fp4.clone()
    bad[0] = 100
    with pytest.raises(ValueError, match="page-aligned"):
        fp4_decode(prob.q, prob.k_fp4, prob.k_sf, prob.v_fp4, prob.v_sf, prob.page_table, bad)
    with pytest.raises(ValueError, match="query_scales_scratch"):
        fp4_decode(prob.q, *common,
                   query_scales_scratch=torch.zeros(2, 1, 16, 2, 32, 4, 3, dtype=torch.uint8,
                                                    device=cuda_device))
    with pytest.raises(ValueError, match="query_padded_scratch"):
        fp4_decode(prob.q, *common, residual_key_pages_bf16=prob.k_pages,
                   residual_value_pages_bf16=prob.v_pages, residual_page_ids=prob.residual_page_ids,
                   seqused_residual=prob.seqused_residual,
                   query_padded_scratch=torch.zeros(2, 64, 16, 128, dtype=torch.bfloat16,
                                                    device=cuda_device))
    with pytest.raises(ValueError, match="layout returned"):
        fp4_decode(prob.q, prob.k_fp4, prob.k_sf.permute(0, 2, 1, 3, 4, 5, 6).contiguous().permute(
            0, 2, 1, 3, 4, 5, 6), prob.v_fp4, prob.v_sf, prob.page_table, prob.seqused_fp4)


@pytest.mark.parametrize("heads", [(4, 4), (4, 2), (8, 2), (16, 2), (32, 2)])
def test_in_kernel_query_quantisation_is_bit_identical(cuda_device, impl, heads):
    """A BF16 query the kernel can read in place is quantised inside the decode launch; the
    result must equal the two-launch form (query quantiser, then decode) bit for bit, with a
    BF16 tail, with a query that is a strided slice of a wider projection, and when split."""
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _kernel

    heads_q, heads_kv = heads
    _skip_if_unsupported(impl, heads_q, heads_kv)
    case = inputs.attention_case(57, 3, heads_q, heads_kv, (300, 129, 640), 1.0, 0.0)
    prob = Problem(case, cuda_device)
    wide = torch.zeros(3, heads_q + 2 * heads_kv, 128, dtype=torch.bfloat16, device=cuda_device)
    wide[:, :heads_q] = prob.q
    sliced = wide[:, :heads_q]                       # row stride wider than heads_q * 128
    assert not sliced.is_contiguous()
    for kw in ({}, {"num_splits": 2}):
        fused = prob.decode(query=sliced, **kw)
        fused_dense = prob.decode(**kw)
        _kernel.FUSE_QUERY_QUANT = False
        try:
            two_launch = prob.decode(**kw)
        finally:
            _kernel.FUSE_QUERY_QUANT = True
        assert torch.equal(fused, two_launch)
        assert torch.equal(fused_dense, two_launch)


def test_refused_page_ids_are_masked_and_reported(cuda_device, impl):
    """A page id outside the cache (possible only with ``trusted_metadata``) is never turned
    into an address: the page contributes nothing, the rest of the row is exact, and the device
    status word reports it.  Rows are long enough for every ring slot to be reused."""
    import nvfp4_attn_kernel_b200._lib as L
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode

    case = inputs.attention_case(63, 3, 8, 2, (12 * 128, 9 * 128 + 40, 5 * 128), 1.0, 0.0)
    prob = Problem(case, cuda_device)
    table = case["page_table"].copy()
    pages = prob.k_fp4.shape[0]
    bad = {0: [3, 4, 10], 1: [0, 8], 2: [2]}           # logical pages whose ids are corrupted
    for row, cols in bad.items():
        for n, col in enumerate(cols):
            table[row, col] = pages + 7 if n % 2 == 0 else -3
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    got = _decode.decode_fp4(
        query_fp4=None, query_scales=None, query_padded_bf16=None, query_bf16=prob.q,
        key_pages_fp4=prob.k_fp4, key_scales=prob.k_sf, value_pages_fp4=prob.v_fp4,
        value_scales=prob.v_sf, fp4_page_table=torch.from_numpy(table).to(cuda_device),
        seqused_fp4=prob.seqused_fp4, residual_key_pages_bf16=prob.k_pages,
        residual_value_pages_bf16=prob.v_pages, residual_page_ids=prob.residual_page_ids,
        seqused_residual=prob.seqused_residual, softmax_scale=prob.softmax_scale,
        trusted_metadata=True, status=status)
    assert int(status.item()) & L.STATUS_BAD_PAGE_ID
    # the oracle sees the same rows with the corrupted pages taken out of the walk
    clean = dict(case)
    clean["page_table"] = case["page_table"].copy()
    clean["seqused_fp4"] = case["seqused_fp4"].copy()
    for row, cols in bad.items():
        n = int(case["seqused_fp4"][row]) // 128
        keep = [c for c in range(n) if c not in cols]
        clean["page_table"][row, :len(keep)] = case["page_table"][row, keep]
        clean["seqused_fp4"][row] = len(keep) * 128
    prob.case = clean
    want = prob.oracle_from_bytes()
    got = to_np(got)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= TOL, np.abs(got - want).max()


def test_programmatic_launch_chain_is_bit_identical(cuda_device):
    """Back-to-back decode launches with programmatic stream serialization (a launch's CTAs may
    start while the previous launch drains) give the bits of plain launches, also when each
    launch's query is produced by the kernel right before it."""
    import nvfp4_attn_kernel_b200._lib as L
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode

    if not L.load().nvfp4_decode_impl_available(L.IMPL_SM100, 8, 2):
        pytest.skip("needs the tensor-core kernel")
    case = inputs.attention_case(81, 6, 8, 2, (1500, 700, 128 * 20, 90, 128 * 7 + 5, 300), 1.0, 0.0)
    prob = Problem(case, cuda_device)

    def run(pdl):
        outs = []
        q = prob.q.clone()
        for step in range(6):
            out = _decode.decode_fp4(
                query_fp4=None, query_scales=None, query_padded_bf16=None, query_bf16=q,
                key_pages_fp4=prob.k_fp4, key_scales=prob.k_sf, value_pages_fp4=prob.v_fp4,
                value_scales=prob.v_sf, fp4_page_table=prob.page_table, seqused_fp4=prob.seqused_fp4,
                residual_key_pages_bf16=prob.k_pages, residual_value_pages_bf16=prob.v_pages,
                residual_page_ids=prob.residual_page_ids, seqused_residual=prob.seqused_residual,
                softmax_scale=prob.softmax_scale, trusted_metadata=True, programmatic_launch=pdl)
            outs.append(out)
            q = out * 3.0 + prob.q      # the next launch's query depends on this launch's output
        torch.cuda.synchronize()
        return outs

    plain, chained = run(False), run(True)
    for a, b in zip(plain, chained):
        assert torch.equal(a, b)


def test_repeated_trusted_calls_reuse_their_argument_block(cuda_device, impl):
    """A trusted call whose tensors have the address, dtype, shape and strides of an earlier one
    is launched from that call's argument block; anything that differs is validated afresh."""
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _kernel, fp4_decode

    prob = Problem(_case("gqa4_short"), cuda_device)
    _kernel._PLANS.clear()
    first = prob.decode(trusted_metadata=True)
    assert len(_kernel._PLANS) == 1
    again = prob.decode(trusted_metadata=True)
    assert len(_kernel._PLANS) == 1 and torch.equal(first, again) and again.data_ptr() != first.data_ptr()
    out = torch.zeros_like(first)
    into = prob.decode(trusted_metadata=True, out=out)
    assert len(_kernel._PLANS) == 2 and into.data_ptr() == out.data_ptr() and torch.equal(into, first)
    out.zero_()
    prob.decode(trusted_metadata=True, out=out)
    assert torch.equal(out, first)
    # untrusted calls are never cached, and a bad argument is still refused after a cached good one
    prob.decode()
    assert len(_kernel._PLANS) == 2
    with pytest.raises(ValueError):
        prob.decode(trusted_metadata=True, seqused_fp4=prob.seqused_fp4.to(torch.int64))
    _kernel.CACHE_CALL_PLANS = False
    try:
        assert torch.equal(prob.decode(trusted_metadata=True), first)
    finally:
        _kernel.CACHE_CALL_PLANS = True


@pytest.mark.parametrize("with_shift", [False, True])
def test_fused_tail_append_equals_append_then_decode(cuda_device, impl, with_shift):
    """One-token rows may hand their step's K/V to the decode launch: the tail pages and the
    output must come out bit-identical to the tail-append kernel followed by the plain call.
    Includes a row whose token fills its tail page, a row whose tail holds only that token and a
    padding row (empty tail, tail id -1) that must not be touched."""
    import nvfp4_attn_kernel_b200._lib as L
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import fp4_decode

    heads_q, heads_kv = 8, 2
    case = inputs.attention_case(91, 5, heads_q, heads_kv, (128 * 3 + 50, 128 * 2, 1, 128 * 5 + 128, 300), 1.0, 0.0)
    prob = Problem(case, cuda_device)
    rows = 5
    rng = np.random.default_rng(92)
    seq_tail = case["seqused_residual"].copy()
    seq_tail[4] = 0                                       # a padding row: no keys in the tail
    tail_ids = case["residual_page_ids"].copy()
    tail_ids[4] = -1
    seq_fp4 = case["seqused_fp4"].copy()
    seq_fp4[4] = 0
    key = bf16_tensor(rng.standard_normal((rows, heads_kv, 128)).astype(np.float32) + 1.5, cuda_device)
    value = bf16_tensor(rng.standard_normal((rows, heads_kv, 128)).astype(np.float32), cuda_device)
    shift = bf16_tensor(rng.standard_normal((heads_kv, 128)).astype(np.float32), cuda_device) if with_shift else None
    t = lambda a: torch.from_numpy(a).to(cuda_device)
    common = dict(fp4_page_table=prob.page_table, seqused_fp4=t(seq_fp4), residual_page_ids=t(tail_ids),
                  seqused_residual=t(seq_tail), softmax_scale=prob.softmax_scale, trusted_metadata=True)

    def run(fused):
        tail_k, tail_v = prob.k_pages.clone(), prob.v_pages.clone()
        extra = {}
        if fused:
            extra = dict(append_key=key, append_value=value, key_shift=shift)
        else:
            starts = torch.arange(rows + 1, dtype=torch.int32, device=cuda_device)
            seq_lens = t((seq_fp4 + seq_tail).astype(np.int32))
            L.check(L.load().nvfp4_tail_append(
                key.data_ptr(), value.data_ptr(), key.stride(0), value.stride(0), L.ptr(shift),
                tail_k.data_ptr(), tail_v.data_ptr(), tail_k.stride(0), starts.data_ptr(), seq_lens.data_ptr(),
                common["seqused_fp4"].data_ptr(), common["residual_page_ids"].data_ptr(), rows, rows, heads_kv,
                torch.cuda.current_stream().cuda_stream))
        out = fp4_decode(prob.q, prob.k_fp4, prob.k_sf, prob.v_fp4, prob.v_sf, **mode,
                         residual_key_pages_bf16=tail_k, residual_value_pages_bf16=tail_v, **common, **extra)
        torch.cuda.synchronize()
        return out, tail_k, tail_v

    # with splits, the split that owns the residual appends; with the balanced split, the tail's own piece
    modes = [dict(num_splits=1), dict(num_splits=2)] + ([dict(balance_pages=2)] if impl == "sm100" else [])
    for mode in modes:
        want, want_k, want_v = run(False)
        got, got_k, got_v = run(True)
        assert torch.equal(got_k, want_k) and torch.equal(got_v, want_v)
        assert not torch.equal(want_k, prob.k_pages)          # something was appended
        assert torch.equal(got, want)


@pytest.mark.parametrize("heads", [(32, 2), (32, 1)])
def test_wide_groups_run_on_the_tensor_core_kernel(cuda_device, heads):
    """Sixteen and thirty-two query heads per KV head take N = 16 / N = 32 products (the latter
    one page per hand-over): rows with and without a tail, a row shorter than a page, the split
    path, and agreement with the CUDA-core kernel."""
    import nvfp4_attn_kernel_b200._lib as L

    heads_q, heads_kv = heads
    if not L.load().nvfp4_decode_impl_available(L.IMPL_SM100, heads_q, heads_kv):
        pytest.skip("this build's tensor-core kernel does not take this group size")
    case = inputs.attention_case(97, 5, heads_q, heads_kv, (128 * 6 + 77, 128 * 3, 90, 128 * 11 + 1, 1500), 1.0, 0.0)
    prob = Problem(case, cuda_device)
    want = prob.oracle_from_bytes()
    try:
        _set_impl("sm100")
        out = to_np(prob.decode())
        split = to_np(prob.decode(num_splits=2))
        _set_impl("generic")
        generic = to_np(prob.decode())
    finally:
        _set_impl("auto")
    assert np.isfinite(out).all()
    assert np.abs(out - want).max() <= TOL, np.abs(out - want).max()
    assert np.abs(split - prob.oracle_from_bytes(splits=2)).max() <= TOL
    assert np.abs(out - generic).max() <= TOL


@pytest.mark.parametrize("target", [1, 3, 8])
def test_balanced_split_gives_every_row_its_own_split_count(cuda_device, target):
    """Row r is cut into ceil(pages_r / target) page ranges plus a piece for its tail alone: checked
    row by row against the oracle run over exactly those pieces."""
    from helpers import oracle_balanced

    _set_impl("auto")
    lengths = (1024 + 17, 128 * 5, 60, 128 * 13, 128, 128 * 2 + 127, 1)
    case = inputs.attention_case(61, len(lengths), 8, 2, lengths, 1.0, 0.0)
    prob = Problem(case, cuda_device)
    out = to_np(prob.decode(balance_pages=target))
    for row in range(len(lengths)):
        want = oracle_balanced(prob, row, target)
        assert np.abs(out[row] - want[0]).max() <= TOL, (row, target)
    # rows without a tail, cut into a power-of-two count: the very bytes of num_splits = that count
    even = inputs.attention_case(62, 3, 8, 2, (128 * 8, 128 * 8, 128 * 8), 1.0, 0.0)
    even["seqused_fp4"] = np.full(3, 128 * 8, dtype=np.int32)      # all eight pages quantised,
    even["seqused_residual"] = np.zeros(3, dtype=np.int32)         # nothing left in the tail
    prob = Problem(even, cuda_device)
    assert torch.equal(prob.decode(balance_pages=2), prob.decode(num_splits=4))


@pytest.mark.parametrize("heads", [(8, 8), (8, 4), (8, 2), (32, 8), (8, 1), (32, 2), (32, 1)])
def test_tail_piece_of_the_balanced_split(cuda_device, heads):
    """The tail's own piece (keys and values staged in shared memory by bulk copies) for every
    group size, tail lengths 1..127 and 128, rows with and without pages, with the step's token
    appended inside the launch: equal to appending first and then decoding, and inside the
    parity bound of the oracle over the same pieces."""
    from helpers import oracle_balanced

    _set_impl("auto")
    hq, hkv = heads
    lengths = (128 * 3 + 1, 127, 128 * 2 + 64, 128 * 6, 128 + 127, 33, 128 * 4 + 2)
    case = inputs.attention_case(640 + hq + hkv, len(lengths), hq, hkv, lengths, 1.0, 0.3)
    prob = Problem(case, cuda_device)
    out = to_np(prob.decode(balance_pages=2))
    assert np.isfinite(out).all()
    for row in range(len(lengths)):
        want = oracle_balanced(prob, row, 2)
        assert np.abs(out[row] - want[0]).max() <= TOL, (row, heads)
    # on request the pieces are merged inside the decode launch by whichever piece finishes last
    # instead of by the merge launch: the same bits, call after call
    own_launch = prob.decode_direct(balance_pages=2, trusted_metadata=True)
    in_launch = prob.decode_direct(balance_pages=2, trusted_metadata=True, merge_in_launch=True)
    assert torch.equal(in_launch, own_launch)
    assert np.array_equal(to_np(own_launch), out)
    for _ in range(3):
        assert torch.equal(prob.decode_direct(balance_pages=2, trusted_metadata=True, merge_in_launch=True), in_launch)


def test_balanced_split_workspace_graph_replay_and_refusals(cuda_device):
    from nvfp4_attn_kernel_b200 import _lib
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel._decode import balanced_workspace_bytes

    _set_impl("auto")
    lengths = (128 * 9 + 3, 128 * 2 + 90, 128 * 30)
    case = inputs.attention_case(63, len(lengths), 8, 2, lengths, 1.0, 0.0)
    prob = Problem(case, cuda_device)
    columns = prob.page_table.shape[1]
    need = balanced_workspace_bytes(3, 8, columns, 4)
    capacity = _lib.load().nvfp4_decode_balanced_capacity(3, columns, 4)
    assert capacity == 2 * 3 + 3 * columns // 4
    assert need >= capacity * 8 * 129 * 4 + capacity * 16 + 2 * 3 * 4
    # garbage in the workspace must not matter: every slot the merge reads is written by the call
    space = torch.randint(0, 256, (need,), dtype=torch.uint8, device=cuda_device)
    out = torch.empty(3, 8, 128, dtype=torch.bfloat16, device=cuda_device)
    first = prob.decode(balance_pages=4, balance_workspace=space, out=out, trusted_metadata=True).clone()
    want = to_np(first)
    from helpers import oracle_balanced

    for row in range(len(lengths)):
        ref = oracle_balanced(prob, row, 4)
        assert np.abs(want[row] - ref[0]).max() <= TOL
    # another layer of the same step: other query, same lengths - the list in the workspace is reused
    other = (prob.q.float() * -0.5 + 0.25).to(torch.bfloat16)
    fresh = prob.decode(query=other, balance_pages=4, trusted_metadata=True)
    space[: need // 2].random_(0, 256)   # the partials of the earlier call are garbage by now
    reused = prob.decode(query=other, balance_pages=4, balance_workspace=space, balance_reuse=True,
                         trusted_metadata=True)
    assert torch.equal(reused, fresh)
    with pytest.raises(ValueError, match="reuse_work_list"):
        prob.decode(balance_pages=4, balance_reuse=True)
    # the three launches replay from a CUDA graph after the lengths change on the device
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        prob.decode(balance_pages=4, balance_workspace=space, out=out, trusted_metadata=True)
    out.zero_()
    graph.replay()
    assert torch.equal(out, first)
    prob.seqused_fp4.copy_(torch.tensor([128 * 2, 128 * 1, 128 * 17], dtype=torch.int32))
    graph.replay()
    torch.cuda.synchronize()
    shorter = to_np(out)
    case2 = dict(case)
    case2["seqused_fp4"] = np.array([256, 128, 128 * 17], dtype=np.int32)
    prob.case = case2
    for row in range(3):
        ref = oracle_balanced(prob, row, 4)
        assert np.abs(shorter[row] - ref[0]).max() <= TOL
    with pytest.raises(ValueError, match="balance_pages"):
        prob.decode(balance_pages=4, num_splits=2)
    with pytest.raises(ValueError, match="balance_pages"):
        prob.decode(balance_pages=0)
    with pytest.raises(ValueError, match="workspace"):
        prob.decode(balance_pages=4, balance_workspace=space[: need - 16])
    with pytest.raises(ValueError, match="out_indices"):
        prob.decode(balance_pages=4, out=out,
                    out_indices=torch.arange(3, dtype=torch.int32, device=cuda_device))


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("splits", [1, 4])
def test_kv_head_shard_equals_the_same_heads_of_the_full_call(cuda_device, world, splits):
    """Tensor parallelism by KV head needs no exchange inside attention: the decode of a rank's
    ``sharding.kv_head_slice`` (its query heads, its narrower K/V pages and tails) gives, bit for
    bit, those heads of the 32/8 call.  The quantised bytes are per (token, head), so the rank's
    own quantisation of its slice is the same bytes as the slice of the full cache."""
    from nvfp4_attn_kernel_b200 import sharding

    rows, hq, hkv = 3, 32, 8
    case = inputs.attention_case(4100 + world, rows, hq, hkv, (128 * 9 + 17, 128 * 4, 77), 1.0, 0.5)
    full = Problem(case, cuda_device)
    kw = dict(num_splits=splits) if splits > 1 else {}
    want = full.decode(**kw)
    for rank in range(world):
        q_heads, kv_heads = sharding.kv_head_slice(rank, world, hq, hkv)
        local = dict(case)
        local["q"] = case["q"][:, q_heads]
        local["k_pages"] = case["k_pages"][:, :, kv_heads]
        local["v_pages"] = case["v_pages"][:, :, kv_heads]
        part = Problem(local, cuda_device)
        assert part.heads_q == hq // world and part.heads_kv == hkv // world
        assert torch.equal(part.k_fp4, full.k_fp4[:, :, kv_heads])
        got = part.decode(**kw)
        assert torch.equal(got, want[:, q_heads]), (world, rank)


def test_kv_head_shard_of_a_large_batch_matches_under_the_same_kernel_form(cuda_device):
    """A batch whose full launch exceeds one CTA per SM runs the kernel's narrow form while a
    rank's eighth of it fits the wide form.  The two forms add a row's pages in a different order
    (results agree to output rounding, not bit for bit), so the bit-for-bit statement about
    KV-head shards is made under one form: with the full call asked to take the wide form too,
    every shard equals its heads exactly; against the default (narrow) full call it stays within
    output rounding."""
    from nvfp4_attn_kernel_b200 import sharding

    rows, hq, hkv, world = 40, 32, 8, 8
    lens = [128 * (3 + i % 5) + (i * 13) % 128 for i in range(rows)]
    case = inputs.attention_case(4200, rows, hq, hkv, lens, 1.0, 0.0)
    full = Problem(case, cuda_device)
    narrow = full.decode_direct(trusted_metadata=True)
    wide = full.decode_direct(trusted_metadata=True, wide_form=True)
    assert (narrow.float() - wide.float()).abs().max().item() <= 2e-3
    for rank in (0, 3, 7):
        q_heads, kv_heads = sharding.kv_head_slice(rank, world, hq, hkv)
        local = dict(case)
        local["q"] = case["q"][:, q_heads]
        local["k_pages"] = case["k_pages"][:, :, kv_heads]
        local["v_pages"] = case["v_pages"][:, :, kv_heads]
        got = Problem(local, cuda_device).decode_direct(trusted_metadata=True)
        assert torch.equal(got, wide[:, q_heads]), rank
        assert (got.float() - narrow[:, q_heads].float()).abs().max().item() <= 2e-3


def test_host_io_step_copies_and_direct_form(cuda_device):
    """``host_io_step``: query from pinned host memory, rows to pinned host memory, one call into
    the library.  With the copy operations and without them (the kernel reads and writes the
    pinned buffers itself) the rows equal ``fp4_decode`` on the same query bit for bit; a tail,
    several query rows, repeated calls with a changing query; unpinned buffers are refused."""
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import fp4_decode, host_io_step

    _set_impl("auto")
    case = inputs.attention_case(77, 5, 32, 8, (128 * 6 + 9, 128 * 2, 100, 128 * 9 + 127, 128 * 4 + 1), 1.0, 0.0)
    prob = Problem(case, cuda_device)
    tails = dict(residual_key_pages_bf16=prob.k_pages, residual_value_pages_bf16=prob.v_pages,
                 residual_page_ids=prob.residual_page_ids, seqused_residual=prob.seqused_residual)
    q_dev = torch.empty_like(prob.q)
    out_dev = torch.zeros(5, 32, 128, dtype=torch.bfloat16, device=cuda_device)
    q_dev.copy_(prob.q)
    common = (prob.k_fp4, prob.k_sf, prob.v_fp4, prob.v_sf, prob.page_table, prob.seqused_fp4)
    for direct in (False, True):
        step = host_io_step(q_dev, *common, out=out_dev, direct=direct, **tails)
        for scale in (1.0, -0.5):
            query = (prob.q.float() * scale).to(torch.bfloat16)
            want = fp4_decode(query, *common, **tails)
            q_host = query.cpu().pin_memory()
            out_host = torch.zeros(5, 32, 128, dtype=torch.bfloat16).pin_memory()
            step(q_host, out_host)
            assert torch.equal(out_host.to(cuda_device), want), (direct, scale)
        with pytest.raises((ValueError, RuntimeError)):
            step(query.cpu(), out_host)          # not pinned
    # steps over the same device query / output buffers but different caches (two page pools of a
    # benchmark, two layers): each keeps its own cache, in whatever order they are built
    other = Problem(inputs.attention_case(78, 5, 32, 8, (128 * 3, 128 * 5 + 7, 128, 128 * 2 + 1, 60), 1.0, 0.0), cuda_device)
    other_common = (other.k_fp4, other.k_sf, other.v_fp4, other.v_sf, other.page_table, other.seqused_fp4)
    other_tails = dict(residual_key_pages_bf16=other.k_pages, residual_value_pages_bf16=other.v_pages,
                       residual_page_ids=other.residual_page_ids, seqused_residual=other.seqused_residual)
    built = [host_io_step(q_dev, *common, out=out_dev, **tails),
             host_io_step(q_dev, *other_common, out=out_dev, **other_tails),
             host_io_step(q_dev, *common, out=out_dev, direct=True, **tails),
             host_io_step(q_dev, *other_common, out=out_dev, direct=True, **other_tails)]
    q_host = prob.q.cpu().pin_memory()
    out_host = torch.zeros(5, 32, 128, dtype=torch.bfloat16).pin_memory()
    wants = [fp4_decode(prob.q, *common, **tails), fp4_decode(prob.q, *other_common, **other_tails)]
    assert not torch.equal(wants[0], wants[1])
    for i, step in enumerate(built):
        step(q_host, out_host)
        assert torch.equal(out_host.to(cuda_device), wants[i % 2]), i
