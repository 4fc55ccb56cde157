"""CPU tests of the C-ABI boundary: the shared library loads without a GPU,
exports every function the public header declares, and rejects bad arguments
before touching the device."""

import ctypes
import os
import re

import pytest

import nvfp4_attn_kernel_b200._lib as L

ROOT = os.path.dirname(os.path.dirname(__file__))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "nvfp4_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nvfp4_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = L.load()
    names = declared_functions()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/nvfp4_b200.h but not exported"
    assert set(names) == set(L.EXPORTS) | {n for n in names if n not in L.EXPORTS}
    assert set(L.EXPORTS) <= set(names)
    assert lib.nvfp4_version() >= 100


def test_struct_mirror_matches_header_field_order():
    text = open(os.path.join(ROOT, "include", "nvfp4_b200.h")).read()
    body = text[text.index("typedef struct nvfp4_decode_args {"):text.index("} nvfp4_decode_args;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"\b([a-z_0-9]+)\s*;", body)
    assert fields == [name for name, _ in L.DecodeArgs._fields_]


def test_workspace_size():
    lib = L.load()
    assert lib.nvfp4_decode_workspace_bytes(32, 32, 1) == 0
    assert lib.nvfp4_decode_workspace_bytes(4, 32, 8) == 8 * 4 * 32 * 129 * 4
    assert lib.nvfp4_decode_workspace_bytes(0, 32, 8) == 0


def test_balanced_split_sizes_and_refusals():
    """Host arithmetic of the balanced split: the capacity bounds the number of pieces of any
    batch, the workspace holds partials, list, the per-row ranges and the arrival counters, and the entry refuses what
    its header says it refuses - all before anything is launched."""
    import numpy as np

    import nvfp4_oracle as O

    lib = L.load()
    rng = np.random.default_rng(5)
    for _ in range(200):
        rows = int(rng.integers(1, 70))
        max_pages = int(rng.integers(0, 300))
        target = int(rng.integers(1, 80))
        capacity = lib.nvfp4_decode_balanced_capacity(rows, max_pages, target)
        assert capacity == O.balanced_capacity(rows, max_pages, target)
        lengths = rng.integers(0, max_pages + 1, rows) * 128
        assert int(O.balanced_split_counts(lengths, target).sum()) + rows <= capacity   # + a tail piece each
        full = np.full(rows, max_pages * 128)
        assert int(O.balanced_split_counts(full, target).sum()) + rows <= capacity
        heads_q = int(rng.choice([8, 32, 64]))
        need = lib.nvfp4_decode_balanced_workspace_bytes(rows, heads_q, max_pages, target)
        # partials and their LSEs, the list, first slot and piece count per row, arrival counters
        floor = capacity * heads_q * 129 * 4 + capacity * 16 + 2 * rows * 4 + rows * heads_q * 4
        assert floor <= need <= floor + 6 * 16
    assert lib.nvfp4_decode_balanced_capacity(0, 32, 8) == 0
    assert lib.nvfp4_decode_balanced_capacity(4, 32, 0) == 0
    assert lib.nvfp4_decode_balanced_workspace_bytes(4, 0, 32, 8) == 0

    assert lib.nvfp4_decode_balanced(None, 8, None) == L.ERR_INVALID
    args = L.DecodeArgs()
    args.rows, args.heads_q, args.heads_kv, args.softmax_scale, args.num_splits = 2, 32, 8, 0.1, 1
    assert lib.nvfp4_decode_balanced(ctypes.byref(args), 0, None) == L.ERR_INVALID
    assert "target_pages" in L.last_error()
    assert lib.nvfp4_decode_balanced(ctypes.byref(args), 8, None) == L.ERR_INVALID   # no out
    assert "num_splits = 1, out" in L.last_error()
    args.num_splits = 2
    assert lib.nvfp4_decode_balanced(ctypes.byref(args), 8, None) == L.ERR_INVALID
    # the reuse flag belongs to the balanced entry alone
    args.num_splits = 1
    args.flags = L.DECODE_REUSE_WORK_LIST
    args.q_bf16 = args.k_packed = args.k_sf = args.v_packed = args.v_sf = 1 << 20
    args.page_table = args.seqused_fp4 = args.out = 1 << 20
    args.k_pitch = args.v_pitch = 128 * 8 * 64
    args.k_sf_pitch = args.v_sf_pitch = 8 * 1024
    args.max_pages = args.page_table_row_stride = 4
    args.num_pages = 16
    args.q_bf16_row_stride, args.q_bf16_head_stride = 32 * 128, 128
    assert lib.nvfp4_decode(ctypes.byref(args), None) == L.ERR_INVALID
    assert "work list to reuse" in L.last_error()
    # and the balanced entry wants its workspace before it launches anything
    args.flags = 0
    assert lib.nvfp4_decode_balanced(ctypes.byref(args), 2, None) == L.ERR_INVALID
    assert "workspace" in L.last_error()


def test_argument_errors_are_reported_without_a_device():
    lib = L.load()
    assert lib.nvfp4_decode(None, None) == L.ERR_INVALID
    assert "null argument block" in L.last_error()
    assert lib.nvfp4_quantize_q(None, 0, 0, None, None, None, None, -1, 32, 8, None) == L.ERR_INVALID
    with pytest.raises(ValueError, match="non-negative"):
        L.check(L.ERR_INVALID)
    args = L.DecodeArgs()
    args.rows, args.heads_q, args.heads_kv = 1, 72, 8   # 9 query heads per KV head: refused
    assert lib.nvfp4_decode(ctypes.byref(args), None) == L.ERR_UNSUPPORTED
    args.heads_q = 32
    args.softmax_scale = 0.0
    assert lib.nvfp4_decode(ctypes.byref(args), None) == L.ERR_INVALID
    assert "softmax_scale" in L.last_error()
    args.softmax_scale = 0.1
    args.num_splits = 0
    assert lib.nvfp4_decode(ctypes.byref(args), None) == L.ERR_INVALID
    args.num_splits = 1
    assert lib.nvfp4_decode(ctypes.byref(args), None) == L.ERR_INVALID
    assert "required pointer" in L.last_error()
    # zero-sized work is a successful no-op
    assert lib.nvfp4_quantize_kv_pages(0, None, 0, None, None, 0, None, 0, None, None, None, None,
                                       0, 1, 0, 8, None) == 0
    assert lib.nvfp4_lse_merge(None, 0, None, 0, 1, 0, 32, None, 0, None, None, None) == 0


def test_host_side_checks_of_the_python_operator():
    import torch

    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import fp4_decode
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel._decode import split_k_heuristic

    with pytest.raises(ValueError, match="missing required decode arguments"):
        fp4_decode(torch.zeros(1, 32, 128, dtype=torch.bfloat16))
    z = torch.zeros(1)
    with pytest.raises(ValueError, match="positive power of two"):
        fp4_decode(z, z, z, z, z, z, z, num_splits=3)
    with pytest.raises(ValueError, match="either BF16 query"):
        fp4_decode(None, z, z, z, z, z, z)
    with pytest.raises(ValueError, match="must be provided together"):
        fp4_decode(None, z, z, z, z, z, z, query_fp4=z)
    with pytest.raises(ValueError, match="applies only to the BF16 query path"):
        fp4_decode(None, z, z, z, z, z, z, query_fp4=z, query_scales=z, query_row_indices=z)
    # the makespan model: 32 tiles on 148 SMs split, 256 tiles do not
    assert split_k_heuristic(4, 8, 256, sms=148) == 4
    assert split_k_heuristic(32, 8, 32, sms=148) == 1
    assert split_k_heuristic(1, 8, 1, sms=148) == 1
    assert split_k_heuristic(1, 1, 64, sms=148) == 32


def test_wide_piece_pages_fills_one_cta_per_sm():
    """The piece length for the kernel's wide form: the smallest one that cuts the rows into at
    most sms // heads_kv pieces, never below the floor."""
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel._decode import wide_piece_pages

    def pieces(counts, t):
        return sum(-(-n // t) for n in counts if n > 0)

    for counts, heads_kv, sms in (([32] * 16, 8, 148), ([257, 3, 0, 64, 1000], 8, 148), ([5], 1, 148),
                                  ([4096] * 4, 8, 148), ([7] * 300, 8, 148), ([100, 200], 2, 8)):
        t = wide_piece_pages(counts, heads_kv, sms=sms)
        budget = sms // heads_kv
        live = [n for n in counts if n > 0]
        assert t >= 4
        if pieces(live, max(max(live), 4)) <= budget:      # the budget can be met at all
            assert pieces(live, t) <= budget
            assert t == 4 or pieces(live, t - 1) > budget   # and no shorter piece meets it
    assert wide_piece_pages([], 8, sms=148) == 4
    assert wide_piece_pages([0, 0], 8, sms=148) == 4
    assert wide_piece_pages([50], 8, sms=4) == 4           # fewer SMs than KV heads: the floor
    assert wide_piece_pages([32] * 16, 8, sms=148, floor=2) == 32


def test_wide_form_fits_counts_pieces_and_tails():
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel._decode import wide_form_fits, wide_piece_pages

    assert wide_form_fits([32] * 16, 8, 0, sms=148)                 # 16 whole rows x 8 heads = 128 CTAs
    assert not wide_form_fits([32] * 16, 8, 16, sms=148)            # 32 pieces x 8 heads
    assert not wide_form_fits([32] * 16, 8, 0, sms=148, tail_pieces=16)
    assert wide_form_fits([68] * 32, 1, 22, sms=148)                # 32 x 4 = 128 pieces
    assert not wide_form_fits([68] * 32, 1, 22, sms=148, tail_pieces=32)
    assert wide_form_fits([60] * 32, 1, 22, sms=148, tail_pieces=32)   # 96 pieces + 32 tails
    # the wide piece length leaves room for the tails it is told about
    t = wide_piece_pages([68] * 32, 1, sms=148, tail_pieces=32)
    assert wide_form_fits([68] * 32, 1, t, sms=148, tail_pieces=32)
    assert not wide_form_fits([68] * 32, 1, t - 1, sms=148, tail_pieces=32)
    assert wide_piece_pages([50], 8, sms=148, tail_pieces=40) == 50   # no room at all: whole rows


def test_entry_points_added_beside_the_reference_refuse_bad_arguments_before_any_launch():
    """The entry points without a counterpart in the reference validate on the host, like the
    others: a refused call returns a code and a message and touches no device."""
    lib = L.load()
    # K-mean accumulation of the calibration
    assert lib.nvfp4_key_sum_accumulate(None, 1024, 0, 8, None, None) == 0            # nothing to do
    assert lib.nvfp4_key_sum_accumulate(None, 1024, 4, 8, None, None) == L.ERR_INVALID
    assert "null" in L.last_error()
    assert lib.nvfp4_key_sum_accumulate(16, 512, 4, 8, 64, None) == L.ERR_INVALID       # stride below a token
    assert "stride" in L.last_error()
    assert lib.nvfp4_key_sum_accumulate(16, 1024, -1, 8, 64, None) == L.ERR_INVALID
    # host-buffer decode
    assert lib.nvfp4_decode_host_io(None, None, 0, None, 0, None) == L.ERR_INVALID
    assert "null" in L.last_error()
    args = L.DecodeArgs()
    assert lib.nvfp4_decode_host_io(ctypes.byref(args), 16, 16, 16, 16, None) == L.ERR_INVALID
    assert "query buffer and out" in L.last_error()
    # control step that also lists the decode pieces: the list's arguments are checked after the
    # slot table's
    ptrs = [16] * 13
    base = [16, 8, 8] + ptrs
    assert lib.nvfp4_control_step_balanced(*base, 4, 4, 8, 0, 32, 8, 32, 16, 1 << 20, None) == L.ERR_INVALID   # decode_rows 0
    assert "decode_rows" in L.last_error()
    assert lib.nvfp4_control_step_balanced(*base, 4, 4, 8, 4, 32, 0, 32, 16, 1 << 20, None) == L.ERR_INVALID   # target_pages 0
    assert lib.nvfp4_control_step_balanced(*base, 4, 4, 8, 4, 32, 8, 32, 16, 64, None) == L.ERR_INVALID        # workspace too small
    assert "workspace" in L.last_error()
    assert lib.nvfp4_control_step_balanced(*base, 4, 4, 200, 4, 32, 8, 32, 16, 1 << 20, None) == L.ERR_INVALID  # too many slots
    assert "128 slots" in L.last_error()
    # flags that belong to one entry point are refused by the others
    args = L.DecodeArgs()
    args.rows, args.heads_q, args.heads_kv, args.softmax_scale, args.num_splits = 1, 32, 8, 0.1, 1
    for k in ("k_packed", "k_sf", "v_packed", "v_sf", "page_table", "seqused_fp4", "q_bf16", "out"):
        setattr(args, k, 4096)
    args.k_pitch = args.v_pitch = 128 * 8 * 64
    args.k_sf_pitch = args.v_sf_pitch = 8 * 1024
    args.num_pages, args.max_pages, args.page_table_row_stride = 4, 4, 4
    args.q_bf16_row_stride, args.q_bf16_head_stride = 32 * 128, 128
    args.flags = L.DECODE_MERGE_IN_LAUNCH
    assert lib.nvfp4_decode(ctypes.byref(args), None) == L.ERR_INVALID
    assert "balanced" in L.last_error()
    args.flags = 1 << 20
    assert lib.nvfp4_decode(ctypes.byref(args), None) == L.ERR_INVALID
    assert "unknown flag" in L.last_error()
