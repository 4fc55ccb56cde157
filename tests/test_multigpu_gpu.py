"""GPU tests of the cross-GPU page-range split.  The two-rank cases need two GPUs (they are
skipped on a single-GPU box); the expired-wait case runs on one GPU."""

import os
import socket
import time

import numpy as np
import pytest
import torch

import inputs
import nvfp4_oracle as O
from helpers import Problem, to_np

pytestmark = pytest.mark.gpu


def test_peer_merge_wait_expires_with_a_status_and_leaves_out_untouched(cuda_device):
    """Failure detection without a fault: rank 1 never announces, the wait gives up after its
    bound, the status word says so and the output buffer is not written."""
    import nvfp4_attn_kernel_b200._lib as L

    lib = L.load()
    rows, hq = 2, 8
    o = torch.zeros(2, rows, hq, 128, dtype=torch.float32, device=cuda_device)
    lse = torch.zeros(2, rows, hq, dtype=torch.float32, device=cuda_device)
    flags = torch.zeros(2, 2, dtype=torch.int32, device=cuda_device)  # [owner][announcer]
    tab = lambda t: torch.tensor([t[0].data_ptr(), t[1].data_ptr()], dtype=torch.int64, device=cuda_device)
    o_tab, lse_tab, flag_tab = tab(o), tab(lse), tab(flags)
    out = torch.full((rows, hq, 128), 3.0, dtype=torch.bfloat16, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    L.check(lib.nvfp4_peer_merge(o_tab.data_ptr(), lse_tab.data_ptr(), flag_tab.data_ptr(), 0, 2, 1,
                                 None, rows, hq, out.data_ptr(), 0, status.data_ptr(), stream))
    torch.cuda.synchronize()
    assert int(status.item()) & L.STATUS_WAIT_TIMEOUT
    assert (out == 3.0).all()
    assert int(flags[0, 0]) == 1 and int(flags[1, 0]) == 1 and int(flags[0, 1]) == 0
    # the context is still usable, and once the missing announcement is there the merge runs
    flags[0, 1] = 1
    status.zero_()
    L.check(lib.nvfp4_peer_merge(o_tab.data_ptr(), lse_tab.data_ptr(), flag_tab.data_ptr(), 0, 2, 1,
                                 None, rows, hq, out.data_ptr(), 0, status.data_ptr(), stream))
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and (out == 0.0).all()


def test_push_merge_wait_expires_then_completes(cuda_device):
    """The push exchange on one GPU with a peer that never pushes: the wait of every (head, row)
    gives up after its bound with a status, ``out`` stays untouched and this rank's own pushes and
    announcements have landed in the (stand-in) peer's inbox.  After the peer's data and flags are
    put there by hand the same call merges both partials."""
    import nvfp4_attn_kernel_b200._lib as L
    import nvfp4_oracle as O

    lib = L.load()
    rows, hq, world = 2, 8, 2
    pairs = rows * hq
    rng = np.random.default_rng(3)
    inbox_floats = int(lib.nvfp4_push_merge_inbox_floats(world, rows, hq))
    assert inbox_floats == 2 * world * pairs * 132
    inbox = [torch.zeros(inbox_floats, dtype=torch.float32, device=cuda_device) for _ in range(world)]
    flags = [torch.zeros(world * pairs, dtype=torch.int32, device=cuda_device) for _ in range(world)]
    table = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=cuda_device)
    inbox_tab, flag_tab = table(inbox), table(flags)
    splits = 3
    o_loc = torch.from_numpy(rng.standard_normal((splits, rows, hq, 128)).astype(np.float32)).to(cuda_device)
    lse_loc = torch.from_numpy(rng.standard_normal((splits, rows, hq)).astype(np.float32)).to(cuda_device)
    lse_loc[1, 0, 3] = float("-inf")
    out = torch.full((rows, hq, 128), 3.0, dtype=torch.bfloat16, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        L.check(lib.nvfp4_push_merge(o_loc.data_ptr(), o_loc.stride(0), lse_loc.data_ptr(), lse_loc.stride(0),
                                     splits, inbox_tab.data_ptr(), flag_tab.data_ptr(), 0, world, 1, None,
                                     rows, hq, out.data_ptr(), 0, status.data_ptr(), stream))
        torch.cuda.synchronize()

    call()
    assert int(status.item()) & L.STATUS_WAIT_TIMEOUT
    assert (out == 3.0).all()
    # rank 0's fold, as pushed into rank 1's inbox: copy 1 (epoch 1), source 0
    mine_o, mine_lse = O.lse_merge(to_np(o_loc), to_np(lse_loc), return_lse=True)
    slot = inbox[1].view(2, world, pairs, 132)[1, 0]
    assert np.allclose(to_np(slot[:, :128]).reshape(rows, hq, 128), mine_o, atol=1e-5)
    assert np.allclose(to_np(slot[:, 128]).reshape(rows, hq), mine_lse, atol=1e-5)
    assert (flags[1][:pairs] == 1).all() and (flags[1][pairs:] == 0).all()
    # now the peer's push arrives
    peer_o = rng.standard_normal((rows, hq, 128)).astype(np.float32)
    peer_lse = rng.standard_normal((rows, hq)).astype(np.float32)
    mine = inbox[0].view(2, world, pairs, 132)
    mine[1, 1, :, :128] = torch.from_numpy(peer_o.reshape(pairs, 128)).to(cuda_device)
    mine[1, 1, :, 128] = torch.from_numpy(peer_lse.reshape(pairs)).to(cuda_device)
    flags[0][pairs:] = 1
    status.zero_()
    call()
    assert int(status.item()) == 0
    want = O.lse_merge(np.stack([mine_o, peer_o]), np.stack([mine_lse, peer_lse]))
    assert np.abs(to_np(out) - want).max() <= 1e-2   # bf16 output


def test_fused_exchange_wait_expires_then_completes(cuda_device):
    """The exchange done by the decode kernel itself, on one GPU with a stand-in peer that never
    pushes: every tile's wait gives up after its bound, ``out`` stays untouched, and - the point of
    the arrival counting - the tile counters are back at zero and the device epoch has advanced, so
    the launch that follows (with the peer's push in place) merges both ranks' partials."""
    import nvfp4_attn_kernel_b200._lib as L

    lib = L.load()
    rows, hq, hkv, world, splits = 2, 32, 8, 2, 2
    pairs = rows * hq
    prob = Problem(inputs.attention_case(91, rows, hq, hkv, (128 * 6 + 3, 128 * 4), 1.0, 0.0), cuda_device)
    inbox_floats = int(lib.nvfp4_push_merge_inbox_floats(world, rows, hq))
    inbox = [torch.zeros(inbox_floats, dtype=torch.float32, device=cuda_device) for _ in range(world)]
    flags = [torch.zeros(world * pairs, dtype=torch.int32, device=cuda_device) for _ in range(world)]
    table = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=cuda_device)
    inbox_tab, flag_tab = table(inbox), table(flags)
    epoch_state = torch.zeros(2, dtype=torch.int32, device=cuda_device)
    counters = torch.zeros(rows * hkv, dtype=torch.int32, device=cuda_device)
    o_loc = torch.zeros(splits, rows, 1, hq, 128, dtype=torch.float32, device=cuda_device)
    lse_loc = torch.zeros(splits, rows, hq, 1, dtype=torch.float32, device=cuda_device)
    out = torch.full((rows, hq, 128), 3.0, dtype=torch.bfloat16, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    x = L.ExchangeArgs()
    x.inbox_ptrs, x.flag_ptrs = inbox_tab.data_ptr(), flag_tab.data_ptr()
    x.epoch_state, x.tile_counters = epoch_state.data_ptr(), counters.data_ptr()
    x.out, x.out_is_f32, x.rank, x.world = out.data_ptr(), 0, 0, world

    def call():
        prob.decode_direct(num_splits=splits, _partials=(o_loc, lse_loc), _exchange=x, status=status,
                           trusted_metadata=True)
        torch.cuda.synchronize()

    call()                                   # epoch 1: nobody answers
    assert int(status.item()) & L.STATUS_WAIT_TIMEOUT
    assert (out == 3.0).all()
    assert (counters == 0).all()
    assert epoch_state.tolist() == [1, 0]
    # this rank's fold of its two splits went to the stand-in peer's inbox, copy 1, source 0
    mine_o, mine_lse = O.lse_merge(to_np(o_loc).reshape(splits, rows, hq, 128),
                                   to_np(lse_loc).reshape(splits, rows, hq), return_lse=True)
    slot = inbox[1].view(2, world, pairs, 132)[1, 0]
    assert np.allclose(to_np(slot[:, :128]).reshape(rows, hq, 128), mine_o, atol=1e-5)
    assert (flags[1][:pairs] == 1).all()
    # epoch 2 (copy 0): the peer's push is there before the launch
    rng = np.random.default_rng(5)
    peer_o = rng.standard_normal((rows, hq, 128)).astype(np.float32)
    peer_lse = rng.standard_normal((rows, hq)).astype(np.float32) + mine_lse.mean()
    own = inbox[0].view(2, world, pairs, 132)
    own[0, 1, :, :128] = torch.from_numpy(peer_o.reshape(pairs, 128)).to(cuda_device)
    own[0, 1, :, 128] = torch.from_numpy(peer_lse.reshape(pairs)).to(cuda_device)
    flags[0][pairs:] = 2
    status.zero_()
    call()
    assert int(status.item()) == 0
    assert (counters == 0).all()
    assert epoch_state.tolist() == [2, 0]
    want = O.lse_merge(np.stack([mine_o, peer_o]), np.stack([mine_lse, peer_lse]))
    assert np.abs(to_np(out) - want).max() <= 1e-2   # bf16 output


def test_nccl_exchange_refuses_graph_capture(cuda_device):
    """The all-gather exchange is for plain launches only: under stream capture the merge raises
    before it enqueues anything, and the same group still works outside the capture."""
    import torch.distributed as dist

    from nvfp4_attn_kernel_b200 import sharding

    if dist.is_initialized():
        pytest.skip("a process group is already up in this process")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{_free_port()}", rank=0, world_size=1,
                            device_id=cuda_device)
    try:
        rows, hq = 2, 8
        grp = sharding.PageRangeGroup(dist.group.WORLD, rows, hq, cuda_device, exchange="nccl")
        o, lse = grp.partial_buffers()
        o.normal_()
        lse.normal_()
        out = torch.zeros(rows, hq, 128, dtype=torch.float32, device=cuda_device)
        grp.merge(out)                       # plain launch: one rank's partial is the result
        torch.cuda.synchronize()
        assert torch.equal(out, o.view(rows, hq, 128))
        side = torch.cuda.Stream(cuda_device)
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with pytest.raises(RuntimeError, match="cannot be captured"):
            with torch.cuda.graph(graph, stream=side):
                out.zero_()
                grp.merge(out)
        torch.cuda.synchronize()
        grp.merge(out)
        torch.cuda.synchronize()
        assert torch.equal(out, o.view(rows, hq, 128))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, exchange, result):
    import torch.distributed as dist

    from nvfp4_attn_kernel_b200 import sharding
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode, _quantize

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        case = inputs.attention_case(71, 4, 32, 8, (128 * 9 + 33, 128 * 4, 128 * 16 + 128, 77), 1.0, 0.0)
        prob = Problem(case, device)   # every rank holds the whole cache here; it only READS its range
        rows = 4
        grp = sharding.PageRangeGroup(dist.group.WORLD, rows, 32, device, exchange=exchange, heads_kv=8)
        local, lseq = sharding.local_page_table(prob.page_table, prob.seqused_fp4, rank, world)
        tail = {}
        if rank == 0:
            tail = dict(residual_key_pages_bf16=prob.k_pages, residual_value_pages_bf16=prob.v_pages,
                        residual_page_ids=prob.residual_page_ids, seqused_residual=prob.seqused_residual)
        out = torch.zeros(rows, 32, 128, dtype=torch.bfloat16, device=device)
        outs = []
        for step in range(3):   # three steps exercise the alternating partial copies and the epochs
            sharding.decode_page_range(grp, prob.q, prob.k_fp4, prob.k_sf, prob.v_fp4, prob.v_sf, local, lseq,
                                       out=out, softmax_scale=prob.softmax_scale, **tail)
            outs.append(out.clone())
        torch.cuda.synchronize()
        assert int(grp.status.item()) == 0
        # single-GPU split decode of the same problem: same partials, same merge order
        want = prob.decode(num_splits=world)
        same = all(torch.equal(o, want) for o in outs)
        err = float((outs[-1].float() - torch.from_numpy(prob.oracle_from_bytes(splits=world)).to(device)).abs().max())
        # the same with every rank's own range cut once more and folded on the rank first
        sharding.decode_page_range(grp, prob.q, prob.k_fp4, prob.k_sf, prob.v_fp4, prob.v_sf, local, lseq,
                                   out=out, softmax_scale=prob.softmax_scale, local_splits=2, **tail)
        torch.cuda.synchronize()
        assert int(grp.status.item()) == 0

        def nested(r, s):
            def page_range(n):
                first, last = O.split_page_range(n, r, world)
                lo, hi = O.split_page_range(last - first, s, 2)
                return first + lo, first + hi
            return page_range

        pieces = [(nested(r, s), r == 0 and s == 0) for r in range(world) for s in range(2)]
        want_nested = torch.from_numpy(prob.oracle_from_bytes(splits=pieces)).to(device)
        err = max(err, float((out.float() - want_nested).abs().max()))
        gathered = [None] * world
        dist.all_gather_object(gathered, (same, err))
        if rank == 0:
            result.put(gathered)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["fused", "push", "peer", "nccl"])
def test_page_range_split_over_two_gpus(cuda_device, exchange):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, exchange, result)) for r in range(2)]
    # A rank that fails or stalls must not outlive the test: every rank started here is ended
    # here, by the Process handle this test holds (never by a name pattern).
    try:
        for p in procs:
            p.start()
        deadline = time.monotonic() + 300
        for p in procs:
            p.join(max(1.0, deadline - time.monotonic()))
        codes = [p.exitcode for p in procs]
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(10)
            if p.is_alive():
                p.kill()
                p.join(10)
    assert codes == [0, 0], codes
    for same, err in result.get(timeout=10):
        assert same          # bit-identical to the one-GPU split path
        assert err <= 2e-2   # and within the parity bound of the split oracle
