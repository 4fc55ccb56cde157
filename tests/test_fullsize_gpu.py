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


def test_ragged_batch_with_tails_matches_the_oracle(cuda_device):
    """32 sequences with lengths log-uniform in [128, 32768] and tails uniform in [0, 127], block
    tables drawn from one shuffled pool, every row with a BF16 tail slot: sampled rows (the
    shortest, the longest and two in between) against the oracle fed the cache's own bytes, all
    rows for finiteness, and the split path against the unsplit one."""
    import bench
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _quantize, fp4_decode

    rng = np.random.default_rng(20)
    rows, hq, hkv = 32, 32, 8
    full = np.exp(rng.uniform(np.log(128), np.log(32768), rows)).astype(np.int64) // 128   # full pages per row
    tails = rng.integers(0, 128, rows).astype(np.int32)
    total = int(full.sum())
    pool = bench.build_pools(cuda_device, 1, -(-total // 128) * 128, 1)[0]   # whole quantiser chunks
    perm = rng.permutation(total)
    width = int(full.max())
    table = np.full((rows, width), -1, dtype=np.int32)     # unused columns hold an id nobody may read
    at = 0
    for r in range(rows):
        table[r, :full[r]] = perm[at:at + full[r]]
        at += full[r]
    gen = torch.Generator(device=cuda_device)
    gen.manual_seed(21)
    q = torch.randn(rows, hq, 128, device=cuda_device, generator=gen).to(torch.bfloat16)
    tail_k = torch.randn(rows, 128, hkv, 128, device=cuda_device, generator=gen).to(torch.bfloat16)
    tail_v = torch.randn(rows, 128, hkv, 128, device=cuda_device, generator=gen).to(torch.bfloat16)
    slots = torch.from_numpy(rng.permutation(rows).astype(np.int32)).to(cuda_device)
    seq_fp4 = torch.from_numpy((full * 128).astype(np.int32)).to(cuda_device)
    seq_tail = torch.from_numpy(tails).to(cuda_device)
    args = (q, pool["k"], pool["ksf"], pool["v"], pool["vsf"], torch.from_numpy(table).to(cuda_device), seq_fp4)
    kw = dict(residual_key_pages_bf16=tail_k, residual_value_pages_bf16=tail_v,
              residual_page_ids=slots, seqused_residual=seq_tail, trusted_metadata=True)
    out = fp4_decode(*args, **kw)
    got = to_np(out)
    assert np.isfinite(got).all()
    split = to_np(fp4_decode(*args, **kw, num_splits=4))
    assert np.abs(split - got).max() <= 5e-2

    order = np.argsort(full)
    sample = [int(order[0]), int(order[10]), int(order[21]), int(order[-1])]
    ids = np.unique(np.concatenate([table[r, :full[r]] for r in sample]))
    remap = {int(p): i for i, p in enumerate(ids)}
    blocks = to_np(pool["cache"][torch.from_numpy(ids).to(cuda_device).long()])
    o1, o2, o3 = 65536, 73728, 139264
    k_dq = O.dequantize_key_pages(blocks[:, :o1].reshape(-1, 128, 8, 64), blocks[:, o1:o2])
    v_dq = O.dequantize_value_pages(blocks[:, o2:o3].reshape(-1, 8, 128, 64), blocks[:, o3:])
    qs = q[sample].contiguous()
    q_fp4, q_sf = _quantize.quantize_query(qs, heads_kv=hkv)
    storage = q_sf.as_strided((len(sample), hq * 1024), (hq * 1024, 1))
    q_dq = O.dequantize_query(to_np(q_fp4), to_np(storage).reshape(len(sample), 1, hq, 2, 32, 4, 4), hkv)
    local = np.zeros((len(sample), width), dtype=np.int32)
    for i, r in enumerate(sample):
        local[i, :full[r]] = [remap[int(p)] for p in table[r, :full[r]]]
    want = O.attention_from_dequantized(
        to_np(qs), q_dq, k_dq, v_dq, local, (full[sample] * 128).astype(np.int32),
        tail_key=to_np(tail_k), tail_value=to_np(tail_v), tail_ids=to_np(slots)[sample],
        seqused_residual=tails[sample], softmax_scale=128 ** -0.5)
    assert np.abs(got[sample] - want).max() <= 2e-2
