"""GPU parity of the slot control plane and the page work table against the serial oracle,
under a scripted and a randomised scheduler simulation (integers: bit-exact)."""

import numpy as np
import pytest
import torch

import nvfp4_oracle as O

pytestmark = pytest.mark.gpu

SLOTS = 8
COLUMNS = 6


def _run(plane, table_rows, seq_lens, query_lens, device):
    from nvfp4_attn_kernel_b200.nvfp4_vllm.control import ControlPlane  # noqa: F401

    t = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    qsl = np.concatenate([[0], np.cumsum(query_lens)]).astype(np.int32)
    bt = t(table_rows)
    out = plane.prepare(block_table=bt, seq_lens=t(seq_lens), query_start_loc=t(qsl.tolist()),
                        num_reqs=len(seq_lens), num_actual_tokens=int(qsl[-1]))
    got = dict(
        row_to_slot=out.row_to_slot.tolist(), token_to_slot=out.token_to_slot.tolist(),
        seqused_fp4=out.seqused_fp4.tolist(), seqused_residual=out.seqused_residual.tolist(),
        promotion_source_tokens=out.promotion_source_tokens.tolist(),
        promotion_pages=out.promotion_pages.tolist(), error_code=int(out.error_code.item()))
    return got, bt, qsl


def _compare(got, want, rows):
    for name in ("row_to_slot", "seqused_fp4", "seqused_residual"):
        assert got[name] == want[name][:rows], name
    assert got["token_to_slot"] == want["token_to_slot"]
    assert got["promotion_source_tokens"][:rows] == want["promotion_source_tokens"][:rows]
    assert got["promotion_pages"][:rows] == want["promotion_pages"][:rows]
    assert got["error_code"] == want["error_code"]


def test_scripted_lifecycle(cuda_device):
    from nvfp4_attn_kernel_b200.nvfp4_vllm.control import ControlPlane, ControlPlaneError

    plane = ControlPlane(max_num_seqs=SLOTS, max_num_batched_tokens=4096, device=cuda_device)
    ref = O.SlotTable(SLOTS)
    rows = lambda *first: [[b] + [b * 10 + c for c in range(1, COLUMNS)] for b in first]
    steps = [
        (rows(5, 7), [300, 128], [300, 128]),          # two prompts, one exactly a page
        (rows(5, 7), [301, 129], [1, 1]),              # decode
        (rows(7, 5), [130, 302], [1, 1]),              # rows swapped by the batch condenser
        (rows(7), [131], [1]),                         # request 5 sits a step out
        (rows(7, 5, 9), [132, 303, 64], [1, 1, 64]),   # 5 returns, 9 arrives
        (rows(7, 5, 9, 0), [133, 304, 65, 77], [1, 1, 1, 1]),   # a dummy row over the null block
        (rows(7, 5, 9, 3), [134, 305, 66, 0], [1, 1, 1, 0]),    # a padding row with zero length
        (rows(9, 5), [256, 384], [190, 79]),           # lengths landing on page boundaries
    ]
    for table, seq, qlen in steps[:7]:
        got, _, _ = _run(plane, table, seq, qlen, cuda_device)
        want = ref.prepare(table, seq, qlen)
        _compare(got, want, len(seq))
    assert ref.errors == 0
    plane.raise_for_errors()
    # the last scripted step continues prompts across steps: flagged by both
    table, seq, qlen = steps[7]
    got, _, _ = _run(plane, table, seq, qlen, cuda_device)
    want = ref.prepare(table, seq, qlen)
    _compare(got, want, len(seq))
    assert got["error_code"] & O.SlotTable.E_CONT_PREFILL
    with pytest.raises(ControlPlaneError, match="split across steps"):
        plane.raise_for_errors()
    plane.reset()
    assert int(plane.error_code.item()) == 0 and (plane.slot_keys == -1).all()


@pytest.mark.parametrize("sit_out", [0.0, 0.1])
def test_randomised_scheduler(cuda_device, sit_out):
    """``sit_out`` > 0 lets a running request miss steps; its slot may then be handed to a
    newcomer, which both sides must flag identically (a served engine never does this: vLLM
    schedules every running request every step)."""
    from nvfp4_attn_kernel_b200.nvfp4_vllm.control import ControlPlane

    rng = np.random.default_rng(0xC7)
    plane = ControlPlane(max_num_seqs=SLOTS, max_num_batched_tokens=8192, device=cuda_device)
    ref = O.SlotTable(SLOTS)
    running = {}            # first block -> length
    next_block = 1
    for step in range(300):
        # finish some, admit some, leave some out of the batch
        for key in [k for k in running if rng.random() < 0.04]:
            del running[key]
        while len(running) < SLOTS and rng.random() < 0.3:
            running[next_block] = 0
            next_block += 1
        batch = [k for k in running if rng.random() >= sit_out]
        rng.shuffle(batch)
        if not batch:
            continue
        seq, qlen, table = [], [], []
        for key in batch:
            add = int(rng.integers(1, 400)) if running[key] == 0 else 1
            running[key] += add
            seq.append(running[key])
            qlen.append(add)
            table.append([key] + [1000 + key * COLUMNS + c for c in range(1, COLUMNS)])
        pad = int(rng.integers(0, 2))
        for _ in range(pad):   # CUDA-graph padding rows: zero length over a stale block id
            if len(seq) < SLOTS:
                seq.append(0); qlen.append(0); table.append([int(rng.integers(1, next_block + 1))] * COLUMNS)
        got, bt, qsl = _run(plane, table, seq, qlen, cuda_device)
        want = ref.prepare(table, seq, qlen)
        _compare(got, want, len(seq))
        # the work table of the same step
        from nvfp4_attn_kernel_b200.nvfp4_vllm.write import PageWorkTable

        wt = PageWorkTable(max_num_seqs=SLOTS, max_num_batched_tokens=8192, device=cuda_device)
        t = lambda v: torch.tensor(v, dtype=torch.int32, device=cuda_device)
        src, dst = wt.build(query_start_loc=t(qsl.tolist()), seqused_fp4=t(got["seqused_fp4"]),
                            row_to_slot=t(got["row_to_slot"]), block_table=bt, num_reqs=len(seq),
                            max_query_len=max(qlen))
        if max(qlen) <= 1:
            assert src.numel() == 0
        else:
            columns = min(max(qlen) // 128 + 1, wt.max_columns, COLUMNS)
            wsrc, wdst = O.work_table(qsl.tolist(), got["seqused_fp4"], got["row_to_slot"], table, columns)
            assert src.tolist() == wsrc and dst.tolist() == wdst
    assert int(plane.error_code.item()) == ref.errors
    if sit_out == 0.0:
        assert ref.errors == 0


def test_error_flags(cuda_device):
    from nvfp4_attn_kernel_b200.nvfp4_vllm.control import ControlPlane

    plane = ControlPlane(max_num_seqs=4, max_num_batched_tokens=512, device=cuda_device)
    ref = O.SlotTable(4)
    cases = [
        ([[5, 1], [5, 2]], [10, 20], [10, 20]),      # two live rows share a block
        ([[8, 1]], [50, ], [1]),                     # history but no slot
        ([[9, 1]], [256], [256]),                    # boundary page past a 2-column table is fine (column 1)
        ([[9, 1]], [384], [128]),                    # promotion column 2 is past the table
    ]
    for table, seq, qlen in cases:
        got, _, _ = _run(plane, table, seq, qlen, cuda_device)
        want = ref.prepare(table, seq, qlen)
        assert got["error_code"] == want["error_code"]
        assert got["row_to_slot"] == want["row_to_slot"]
    assert ref.errors & (O.SlotTable.E_DUP | O.SlotTable.E_SLOT_LOST | O.SlotTable.E_PROMO)
    with pytest.raises(ValueError, match="exceeds the 4 tail slots"):
        plane.prepare(block_table=torch.zeros(5, 2, dtype=torch.int32, device=cuda_device),
                      seq_lens=torch.zeros(5, dtype=torch.int32, device=cuda_device),
                      query_start_loc=torch.zeros(6, dtype=torch.int32, device=cuda_device),
                      num_reqs=5, num_actual_tokens=0)


def _list_regions(space, rows, heads_q, capacity):
    """(work [capacity, 4], row_offset [rows], row_count [rows]) of a balanced-split workspace:
    partial outputs, their LSEs, the list, the rows' first slots, the rows' piece counts, each
    region rounded up to 16 bytes."""
    up = lambda b: (b + 15) & ~15
    at = up(capacity * heads_q * 128 * 4) + up(capacity * heads_q * 4)
    work = space[at:at + capacity * 16].view(torch.int32).view(capacity, 4)
    at += up(capacity * 16)
    row_offset = space[at:at + rows * 4].view(torch.int32)
    at += up(rows * 4)
    row_count = space[at:at + rows * 4].view(torch.int32)
    return work.cpu().numpy(), row_offset.cpu().numpy(), row_count.cpu().numpy()


@pytest.mark.parametrize("target", [2, 5])
def test_control_step_builds_the_decode_work_list_in_its_own_launch(cuda_device, target):
    """The control step given a work-list plan leaves in the workspace the list the stand-alone
    builder makes from the same lengths (row by row: the tail piece, then the page pieces; rows
    ordered by size class), the oracle's pieces for every row, and a decode that reuses that list
    equals the decode that builds its own, bit for bit."""
    import inputs
    from helpers import Problem
    from nvfp4_attn_kernel_b200 import _lib
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel._decode import balanced_workspace_bytes
    from nvfp4_attn_kernel_b200.nvfp4_vllm.control import ControlPlane, WorkListPlan

    lengths = (128 * 9 + 3, 128 * 2 + 90, 128 * 30, 77, 128, 128 * 4 + 1)
    rows, hq, hkv = len(lengths), 8, 2
    case = inputs.attention_case(71, rows, hq, hkv, lengths, 1.0, 0.0)
    prob = Problem(case, cuda_device)
    columns = prob.page_table.shape[1]
    plane = ControlPlane(max_num_seqs=8, max_num_batched_tokens=8192, device=cuda_device)
    # the engine's block table: column 0 of a row keys its slot (any non-zero id)
    table = (prob.page_table + 1).contiguous()
    need = balanced_workspace_bytes(rows, hq, columns, target)
    space = torch.randint(0, 256, (need,), dtype=torch.uint8, device=cuda_device)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=cuda_device)
    out = plane.prepare(block_table=table, seq_lens=t(list(lengths)),
                        query_start_loc=t([0] + list(np.cumsum(lengths))), num_reqs=rows,
                        num_actual_tokens=int(sum(lengths)),
                        work_list=WorkListPlan(rows, columns, target, hq, space))
    torch.cuda.synchronize()
    assert int(out.error_code.item()) == 0
    assert out.seqused_fp4.tolist() == case["seqused_fp4"].tolist()
    assert out.seqused_residual.tolist() == case["seqused_residual"].tolist()
    capacity = int(_lib.load().nvfp4_decode_balanced_capacity(rows, columns, target))
    work, offset, count = _list_regions(space, rows, hq, capacity)
    pieces = O.balanced_pieces(case["seqused_fp4"], case["seqused_residual"], target)
    used = 0
    for row in range(rows):
        mine = work[offset[row]:offset[row] + count[row]]
        page_pieces = [p for p in pieces[row] if not p[2]]
        want = [[row, 0, 1, 1]] + [[row, s, len(page_pieces), 0] for s in range(len(page_pieces))]
        assert mine.tolist() == want, row
        used += count[row]
    assert (work[used:, 0] == -1).all() and (work[:used, 0] >= 0).all()
    # a decode that reuses the list = a decode that builds its own
    slots = out.row_to_slot[:rows]
    tails = dict(residual_page_ids=prob.residual_page_ids, seqused_residual=out.seqused_residual[:rows])
    reused = prob.decode(balance_pages=target, balance_workspace=space, balance_reuse=True,
                         seqused_fp4=out.seqused_fp4[:rows], trusted_metadata=True, **tails)
    fresh = prob.decode(balance_pages=target)
    assert slots.tolist() == list(range(rows))   # a fresh table hands out slots in row order
    assert torch.equal(reused, fresh)
