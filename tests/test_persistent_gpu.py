"""GPU parity of the persistent decode launch (``NVFP4_DECODE_PERSISTENT``): one launch whose
CTAs share the step's page tiles equally and merge the pieces of a cut tile.

A tile cut into pieces is, by the reference's definition of its split path
(``src/nvfp4_decode_kernel/_decode.py:982-1171``: every page range runs the whole pipeline on its
own, softmax probabilities quantised against the range's own running maximum, then an LSE merge),
the merge of the oracle run per piece; that is what the kernel is held to here (max-abs 2e-2), with
the schedule restated by ``nvfp4_oracle.persistent_pieces``.  The distance to the oracle over whole
rows is reported by the bench line; it is of the size of the probabilities' quantisation step.
"""

import numpy as np
import pytest
import torch

import inputs
import nvfp4_oracle as O
from helpers import Problem, bf16_tensor, oracle_persistent, persistent_ctas, to_np

pytestmark = pytest.mark.gpu

TOL = 2e-2


def _ws(prob, rows=None):
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode

    ws = _decode.persistent_workspace(rows or prob.q.shape[0], prob.heads_q, prob.heads_kv, prob.device)
    assert ws is not None
    return ws


def _launches(ws):
    """(launches counted on this workspace, CTAs that have left the running launch: 0 between launches)"""
    head = ws[:8].view(torch.int32).tolist()
    return head[0], head[1]


PERSISTENT_CASES = [n for n, c in inputs.SMALL_CASES.items() if c[2] // c[3] <= 8] + ["config1"]


@pytest.mark.parametrize("name", PERSISTENT_CASES)
def test_persistent_matches_the_piecewise_oracle(cuda_device, name):
    case = inputs.config1(0) if name == "config1" else inputs.attention_case(*inputs.SMALL_CASES[name])
    prob = Problem(case, cuda_device)
    ws = _ws(prob)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    got = to_np(prob.decode_direct(persistent_workspace=ws, status=status))
    want, pieces = oracle_persistent(prob)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= TOL
    assert int(status.item()) == 0
    assert _launches(ws) == (1, 0)                        # counted, ready for the next call
    # the launch really cut tiles (else this test would only repeat the one-tile kernel's)
    assert any(len(t) > 1 for t in pieces.values())


def test_persistent_ragged_batch_with_tails_padding_rows_and_scatter(cuda_device):
    """Rows from one token to 4000, a row on an exact page boundary, two padding rows (zero
    lengths, tail id -1) and a scattered output; the page table's unused columns are poisoned."""
    lens = (4000, 130, 1, 2500, 0, 777, 128, 0)
    case = inputs.attention_case(21, len(lens), 32, 8, lens, 1.0, 0.5)
    for r, n in enumerate(lens):
        if n == 0:
            case["residual_page_ids"][r] = -1
        used = int(case["seqused_fp4"][r]) // 128
        case["page_table"][r, used:] = -7
    prob = Problem(case, cuda_device)
    ws = _ws(prob)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    out = torch.full((12, 32, 128), 9.0, dtype=torch.bfloat16, device=cuda_device)
    idx = torch.tensor([3, 0, 11, 5, 7, 1, 8, 2], dtype=torch.int32, device=cuda_device)
    prob.decode_direct(persistent_workspace=ws, status=status, out=out, out_indices=idx, trusted_metadata=True)
    want, _ = oracle_persistent(prob)
    got = to_np(out)
    where = to_np(idx)
    assert np.abs(got[where] - want).max() <= TOL
    assert not got[where[4]].any() and not got[where[7]].any()      # padding rows give zero rows
    untouched = [r for r in range(12) if r not in set(where.tolist())]
    assert (got[untouched] == 9.0).all()
    assert int(status.item()) == 0
    assert _launches(ws) == (1, 0)


def test_persistent_repeats_bitwise_and_agrees_with_the_one_tile_kernel(cuda_device):
    case = inputs.attention_case(5, 9, 32, 8, (1500, 3000, 640, 2048, 129, 300, 4096, 1024, 2900), 1.0, 0.3)
    prob = Problem(case, cuda_device)
    ws = _ws(prob)
    first = to_np(prob.decode(persistent_workspace=ws))
    for _ in range(8):
        assert np.array_equal(to_np(prob.decode(persistent_workspace=ws)), first)
    whole = to_np(prob.decode())
    # both are NVFP4-P approximations of the same attention; they differ by the probabilities'
    # quantisation step where a tile was cut
    assert np.abs(first - whole).max() <= 6e-2


def test_persistent_prequantised_query_equals_bf16_query(cuda_device):
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _quantize, fp4_decode

    case = inputs.attention_case(8, 4, 32, 8, (2048, 1024, 3072, 512), 1.0, 0.0)
    case["seqused_residual"][:] = 0
    prob = Problem(case, cuda_device)
    ws = _ws(prob)
    common = dict(key_pages_fp4=prob.k_fp4, key_scales=prob.k_sf, value_pages_fp4=prob.v_fp4,
                  value_scales=prob.v_sf, fp4_page_table=prob.page_table, seqused_fp4=prob.seqused_fp4,
                  softmax_scale=prob.softmax_scale, persistent_workspace=ws)
    a = to_np(fp4_decode(prob.q, **common))
    q_fp4, q_sf = _quantize.quantize_query(prob.q, heads_kv=prob.heads_kv)
    b = to_np(fp4_decode(query_fp4=q_fp4, query_scales=q_sf, **common))
    assert np.array_equal(a, b)


def test_persistent_fused_append_equals_append_then_decode(cuda_device):
    """The step's own K/V token appended by the launch: tails and outputs bit-identical to the
    separate tail append followed by the same launch."""
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import fp4_decode

    lens = (700, 129, 1, 2049, 384)
    case = inputs.attention_case(31, len(lens), 16, 4, lens, 1.0, 0.4)
    prob = Problem(case, cuda_device)
    ws = _ws(prob)
    rng = np.random.default_rng(3)
    rows, hkv = len(lens), 4
    new_k = bf16_tensor(inputs.bf16(rng.standard_normal((rows, hkv, 128)).astype(np.float32)), cuda_device)
    new_v = bf16_tensor(inputs.bf16(rng.standard_normal((rows, hkv, 128)).astype(np.float32)), cuda_device)
    shift = bf16_tensor(inputs.bf16(rng.standard_normal((hkv, 128)).astype(np.float32) * 0.2), cuda_device)
    common = dict(key_pages_fp4=prob.k_fp4, key_scales=prob.k_sf, value_pages_fp4=prob.v_fp4,
                  value_scales=prob.v_sf, fp4_page_table=prob.page_table, seqused_fp4=prob.seqused_fp4,
                  residual_page_ids=prob.residual_page_ids, seqused_residual=prob.seqused_residual,
                  softmax_scale=prob.softmax_scale, persistent_workspace=ws)
    # separately: store the shifted token at position len - 1 of each row's residual page
    tk, tv = prob.k_pages.clone(), prob.v_pages.clone()
    pos = (prob.seqused_residual - 1).long()
    ids = prob.residual_page_ids.long()
    tk[ids, pos] = torch.sub(new_k, shift)
    tv[ids, pos] = new_v
    want = to_np(fp4_decode(prob.q, residual_key_pages_bf16=tk, residual_value_pages_bf16=tv, **common))
    fk, fv = prob.k_pages.clone(), prob.v_pages.clone()
    got = to_np(fp4_decode(prob.q, residual_key_pages_bf16=fk, residual_value_pages_bf16=fv,
                           append_key=new_k, append_value=new_v, key_shift=shift, **common))
    assert np.array_equal(got, want)
    assert torch.equal(fk, tk) and torch.equal(fv, tv)


def test_persistent_refuses_a_page_id_outside_the_cache(cuda_device):
    case = inputs.attention_case(41, 2, 8, 2, (640, 512), 1.0, 0.0)
    case["page_table"][1, 2] = 10_000
    prob = Problem(case, cuda_device)
    ws = _ws(prob)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    got = to_np(prob.decode_direct(persistent_workspace=ws, status=status, trusted_metadata=True))
    import nvfp4_attn_kernel_b200._lib as L

    assert int(status.item()) & L.STATUS_BAD_PAGE_ID
    assert np.isfinite(got).all()
    # the other row is untouched by the refusal
    clean = inputs.attention_case(41, 2, 8, 2, (640, 512), 1.0, 0.0)
    prob2 = Problem(clean, cuda_device)
    assert np.array_equal(to_np(prob2.decode(persistent_workspace=ws))[0], got[0])


def test_persistent_refusals(cuda_device):
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _decode

    case = inputs.attention_case(*inputs.SMALL_CASES["gqa4_short"])
    prob = Problem(case, cuda_device)
    ws = _ws(prob)
    with pytest.raises(ValueError, match="persistent"):
        prob.decode(persistent_workspace=ws, num_splits=2)
    with pytest.raises(ValueError, match="persistent_workspace must be"):
        prob.decode(persistent_workspace=ws[:64])
    # 16 query heads per KV head stay on the one-tile kernel
    assert _decode.persistent_workspace(1, 16, 1, cuda_device) is None


def test_persistent_headline_size_sampled_tiles(cuda_device):
    """32 sequences x 4096 context (the bench workload's shape): sampled tiles against the
    piecewise oracle, every row against the one-tile kernel."""
    rows, ctx = 32, 4096
    case = inputs.attention_case(77, rows, 32, 8, (ctx,) * rows, 1.0, 0.5)
    case["seqused_fp4"][:] = ctx          # pure NVFP4 pages, no tail
    case["seqused_residual"][:] = 0
    prob = Problem(case, cuda_device)
    ws = _ws(prob)
    got = to_np(prob.decode(persistent_workspace=ws))
    tiles = {(0, 0), (7, 3), (19, 5), (31, 7)}
    want, pieces = oracle_persistent(prob, tiles=tiles)
    assert max(len(t) for t in pieces.values()) >= 2
    for r, h in tiles:
        hs = slice(4 * h, 4 * h + 4)
        assert np.abs(got[r, hs] - want[r, hs]).max() <= TOL
    assert np.abs(got - to_np(prob.decode())).max() <= 6e-2
    assert _launches(ws)[1] == 0
