"""CPU tests of the multi-GPU host logic: the page-range partition, the local block tables and
the exchange + merge arithmetic, run as two gloo ranks."""

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import inputs
import nvfp4_oracle as O
from nvfp4_attn_kernel_b200 import sharding


def test_page_range_matches_the_split_rule():
    for n in (0, 1, 2, 7, 32, 256, 257):
        for parts in (1, 2, 4, 8):
            got = [sharding.page_range(n, r, parts) for r in range(parts)]
            assert got == [O.split_page_range(n, r, parts) for r in range(parts)]
            covered = [p for a, b in got for p in range(a, b)]
            assert covered == list(range(n))


def test_kv_head_slices():
    q, kv = sharding.kv_head_slice(3, 8, 32, 8)
    assert (q.start, q.stop, kv.start, kv.stop) == (12, 16, 3, 4)
    q, kv = sharding.kv_head_slice(1, 2, 32, 8)
    assert (q.start, q.stop, kv.start, kv.stop) == (16, 32, 4, 8)
    with pytest.raises(ValueError, match="do not divide"):
        sharding.kv_head_slice(0, 3, 32, 8)


def test_local_page_table():
    table = torch.arange(40, dtype=torch.int32).reshape(4, 10) + 100
    seq = torch.tensor([10 * 128, 3 * 128, 0, 7 * 128], dtype=torch.int32)
    seen = [[] for _ in range(4)]
    for rank in range(4):
        local, lseq = sharding.local_page_table(table, seq, rank, 4)
        assert local.shape == (4, 3) and local.dtype == torch.int32
        for r in range(4):
            first, last = sharding.page_range(int(seq[r]) // 128, rank, 4)
            assert int(lseq[r]) == (last - first) * 128
            assert local[r, :last - first].tolist() == table[r, first:last].tolist()
            assert (local[r, last - first:] == -1).all()
            seen[r] += local[r, :last - first].tolist()
    for r in range(4):
        assert seen[r] == table[r, :int(seq[r]) // 128].tolist()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = inputs.attention_case(61, 2, 8, 2, (128 * 5 + 40, 128 * 2), 1.0, 0.0)
        q_dq = O.bf16_round(O.nvfp4_round_trip(case["q"]))
        k_dq = O.bf16_round(O.nvfp4_round_trip(case["k_pages"]))
        vt = np.ascontiguousarray(case["v_pages"].transpose(0, 2, 3, 1))
        v_dq = O.bf16_round(O.nvfp4_round_trip(vt)).transpose(0, 3, 1, 2)
        local, lseq = sharding.local_page_table(torch.from_numpy(case["page_table"]),
                                                torch.from_numpy(case["seqused_fp4"]), rank, world)
        tail = dict(tail_key=case["k_pages"], tail_value=case["v_pages"],
                    tail_ids=case["residual_page_ids"], seqused_residual=case["seqused_residual"])
        o, lse = O.attention_from_dequantized(
            case["q"], q_dq, k_dq, v_dq, local.numpy(), lseq.numpy(), softmax_scale=case["softmax_scale"],
            owns_tail=(rank == 0), return_lse=True, **tail)
        packed = torch.from_numpy(np.concatenate([o.reshape(-1), lse.reshape(-1)]))
        gathered = [torch.empty_like(packed) for _ in range(world)]
        dist.all_gather(gathered, packed)
        n_o = o.size
        parts = np.stack([g[:n_o].numpy().reshape(o.shape) for g in gathered])
        lses = np.stack([g[n_o:].numpy().reshape(lse.shape) for g in gathered])
        merged = O.lse_merge(parts, lses)
        if rank == 0:
            want_parts, want_lse = [], []
            for s in range(world):
                po, pl = O.attention_from_dequantized(
                    case["q"], q_dq, k_dq, v_dq, case["page_table"], case["seqused_fp4"],
                    softmax_scale=case["softmax_scale"], owns_tail=(s == 0), return_lse=True,
                    page_range=lambda n, s=s: O.split_page_range(n, s, world), **tail)
                want_parts.append(po)
                want_lse.append(pl)
            want = O.lse_merge(np.stack(want_parts), np.stack(want_lse))
            full = O.attention_from_dequantized(case["q"], q_dq, k_dq, v_dq, case["page_table"],
                                                case["seqused_fp4"], softmax_scale=case["softmax_scale"], **tail)
            result.put((float(np.abs(merged - want).max()), float(np.abs(merged - full).max())))
    finally:
        dist.destroy_process_group()


def test_fused_exchange_refuses_more_than_eight_heads_per_kv_head():
    """The exchange done by the decode kernel serves group sizes up to 8 (the kernel's 16- and
    32-head instantiations are built without it); the refusal comes before anything is set up."""
    cpu = torch.device("cpu")
    with pytest.raises(ValueError, match="at most 8 query heads per KV head"):
        sharding.PageRangeGroup(None, 4, 32, cpu, exchange="fused", heads_kv=2)
    with pytest.raises(ValueError, match="at most 8 query heads per KV head"):
        sharding.PageRangeGroup(None, 4, 32, cpu, exchange="fused", heads_kv=1)
    with pytest.raises(ValueError, match="pass heads_kv"):
        sharding.PageRangeGroup(None, 4, 32, cpu, exchange="fused")


def test_two_ranks_merge_to_the_split_oracle():
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    exact, vs_unsplit = result.get(timeout=10)
    assert exact == 0.0            # the ranks reproduce the single-process split oracle bit for bit
    assert vs_unsplit <= 2e-2      # and stay within the parity bound of the unsplit walk
