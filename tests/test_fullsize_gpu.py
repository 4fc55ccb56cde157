"""GPU tests at the benchmark's full size (32 sequences x 4096 context, 32/8 heads) through
size-independent properties, plus the oracle on sampled rows."""

import numpy as np
import pytest
import torch

import nvfp4_oracle as O
from helpers import to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def workload(cuda_device):
    import bench
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import fp4_decode

    pool = bench.build_pools(cuda_device)[0]
    gen = torch.Generator(device=cuda_device)
    gen.manual_seed(5)
    q = torch.randn(bench.ROWS, bench.HQ, bench.D, device=cuda_device, generator=gen).to(torch.bfloat16)
    seq = torch.full((bench.ROWS,), bench.CTX, dtype=torch.int32, device=cuda_device)

    def decode(table=None, k=None, ksf=None, v=None, vsf=None, query=None, **kw):
        return fp4_decode(q if query is None else query, pool["k"] if k is None else k,
                          pool["ksf"] if ksf is None else ksf, pool["v"] if v is None else v,
                          pool["vsf"] if vsf is None else vsf,
                          pool["table"] if table is None else table, seq, **kw)

    return dict(pool=pool, q=q, seq=seq, decode=decode, base=decode())


def test_sampled_rows_match_the_oracle(workload, cuda_device):
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _quantize

    pool, q = workload["pool"], workload["q"]
    rows = [0, 17, 31]
    table = pool["table"][rows].cpu().numpy()
    ids = np.unique(table)
    remap = {int(p): i for i, p in enumerate(ids)}
    sel = torch.from_numpy(ids).to(cuda_device).long()
    blocks = to_np(pool["cache"][sel])               # [n, 147456]: K packed | K scales | V packed | V scales
    o1, o2, o3 = 65536, 73728, 139264
    k_dq = O.dequantize_key_pages(blocks[:, :o1].reshape(-1, 128, 8, 64), blocks[:, o1:o2])
    v_dq = O.dequantize_value_pages(blocks[:, o2:o3].reshape(-1, 8, 128, 64), blocks[:, o3:])
    q_fp4, q_sf = _quantize.quantize_query(q[rows].contiguous(), heads_kv=8)
    storage = q_sf.as_strided((3, 32 * 1024), (32 * 1024, 1))
    q_dq = O.dequantize_query(to_np(q_fp4), to_np(storage).reshape(3, 1, 32, 2, 32, 4, 4), 8)
    local = np.vectorize(remap.get)(table).astype(np.int32)
    want = O.attention_from_dequantized(to_np(q[rows]), q_dq, k_dq, v_dq, local,
                                        np.full(3, 4096, dtype=np.int32), softmax_scale=128 ** -0.5)
    got = to_np(workload["base"][rows])
    assert np.abs(got - want).max() <= 2e-2


def test_physical_page_permutation_is_bit_identical(workload, cuda_device):
    pool = workload["pool"]
    pages = pool["cache"].shape[0]
    perm = torch.randperm(pages, device=cuda_device)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(pages, device=cuda_device)
    moved = pool["cache"][perm].contiguous()          # new block j holds old block perm[j]
    table = inv[pool["table"].long()].to(torch.int32)  # old id -> new id
    off = lambda t: t.data_ptr() - pool["cache"].data_ptr()
    flat = moved.view(-1)
    views = [flat.as_strided(t.shape, t.stride(), off(t)) for t in
             (pool["k"], pool["ksf"].view(torch.uint8), pool["v"], pool["vsf"].view(torch.uint8))]
    out = workload["decode"](table=table, k=views[0], ksf=views[1], v=views[2], vsf=views[3])
    assert torch.equal(out, workload["base"])


def test_equal_rows_give_equal_outputs_and_repeats_are_bitwise(workload):
    q2 = workload["q"].clone()
    q2[1] = q2[0]
    table = workload["pool"]["table"].clone()
    table[1] = table[0]
    out = workload["decode"](table=table, query=q2)
    assert torch.equal(out[0], out[1])
    assert torch.equal(workload["decode"](), workload["base"])


@pytest.mark.parametrize("splits", [2, 8])
def test_split_merge_is_consistent_at_full_size(workload, splits):
    out = to_np(workload["decode"](num_splits=splits))
    base = to_np(workload["base"])
    assert np.isfinite(out).all()
    # a split quantises P against its own running maximum; the reference's gate for
    # split vs unsplit is max-abs 5e-2
    assert np.abs(out - base).max() <= 5e-2
    cos = (out * base).sum() / np.sqrt((out * out).sum() * (base * base).sum())
    assert cos >= 0.99  # the reference's own gate for kernel-vs-oracle comparisons


def test_both_kernels_agree_at_full_size(workload):
    import nvfp4_attn_kernel_b200._lib as L
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode

    _decode.DEFAULT_IMPL = L.IMPL_GENERIC
    try:
        generic = to_np(workload["decode"]())
    finally:
        _decode.DEFAULT_IMPL = L.IMPL_AUTO
    assert np.abs(generic - to_np(workload["base"])).max() <= 1e-2
