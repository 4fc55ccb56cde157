"""CPU tests: the numpy oracle against the golden vectors produced by the
reference's own torch code, and its byte converters against NVIDIA's host
conversion routines and torch's float8 cast."""

import os
import subprocess

import numpy as np
import pytest
import torch

import inputs
import nvfp4_oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")
ROOT = os.path.dirname(os.path.dirname(__file__))


def test_value_round_trip_matches_reference_golden():
    g = np.load(os.path.join(GOLD, "values_kat.npz"))
    x = inputs.value_kat()
    assert np.array_equal(O.nvfp4_round_trip(x), g["round_trip"])
    assert np.array_equal(O.round_e2m1_ties_down(x), g["round_e2m1"])
    assert np.array_equal(O.nvfp4_round_trip(np.ascontiguousarray(x[:64].T)), g["round_trip_t"])


def test_package_value_model_matches_reference_golden():
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import reference

    g = np.load(os.path.join(GOLD, "values_kat.npz"))
    x = torch.from_numpy(inputs.value_kat())
    assert np.array_equal(reference.nvfp4_round_trip(x).numpy(), g["round_trip"])
    assert np.array_equal(reference.round_e2m1(x).numpy(), g["round_e2m1"])
    with pytest.raises(ValueError, match="divisible by group"):
        reference.nvfp4_round_trip(torch.zeros(3, 10))
    with pytest.raises(ValueError, match="must be positive"):
        reference.nvfp4_round_trip(torch.zeros(3, 16), group=0)


@pytest.mark.parametrize("name", list(inputs.SMALL_CASES) + ["config1"])
def test_attention_oracle_matches_reference_golden(name):
    g = np.load(os.path.join(GOLD, "attention.npz"))
    if name == "config1":
        c = inputs.config1(0)
    else:
        c = inputs.attention_case(*inputs.SMALL_CASES[name])
    out = O.reference_decode(c["q"], c["k_pages"], c["v_pages"], c["page_table"], c["seqused_k"],
                             c["residual_page_ids"], c["seqused_residual"], c["softmax_scale"])
    # fp32 re-association only (numpy einsum vs torch einsum)
    assert np.abs(out - g[name]).max() <= 5e-5


def test_online_softmax_matches_reference_golden():
    g = np.load(os.path.join(GOLD, "online_softmax.npz"))
    rng = np.random.default_rng(21)
    scores = rng.standard_normal((1, 4, 1, 384)).astype(np.float32) * 2.0
    scores[..., 300:] = -np.inf
    v = inputs.bf16(rng.standard_normal((1, 384, 4, 128)).astype(np.float32))
    res = np.zeros(384, dtype=bool)
    res[256:300] = True
    out = O.online_softmax_pv(scores[0, :, 0, :], v[0], res)
    assert np.abs(out - g["out"]).max() <= 1e-5


def _probe_values():
    rng = np.random.default_rng(1)
    return np.concatenate([
        rng.standard_normal(100000).astype(np.float32)
        * np.exp(rng.uniform(-12, 8, 100000)).astype(np.float32),
        np.arange(0, 8, 1 / 64, dtype=np.float32),
        -np.arange(0, 8, 1 / 64, dtype=np.float32),
        np.arange(0, 600, 0.5, dtype=np.float32),
        np.ldexp(np.arange(0, 64, dtype=np.float32), -12),
        np.array([0.0, -0.0, 448, 464, 465, 1e9, -1e9, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10],
                 dtype=np.float32),
    ])


def test_converters_match_cuda_host_headers(tmp_path):
    binary = os.path.join(ROOT, "oracle", "_build", "cvt_check")
    made = subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], capture_output=True, text=True)
    if made.returncode or not os.path.exists(binary):
        pytest.skip("g++ / CUDA headers unavailable: " + made.stderr[-200:])
    x = _probe_values()
    fin, fout = tmp_path / "x.f32", tmp_path / "y.u8"
    x.tofile(fin)
    subprocess.check_call([binary, str(fin), str(fout)])
    y = np.fromfile(fout, dtype=np.uint8).reshape(-1, 2)
    assert np.array_equal(O.e4m3_encode(x), y[:, 0])
    assert np.array_equal(O.e2m1_encode(x), y[:, 1] & 0xF)


def test_e4m3_matches_torch_cast():
    x = _probe_values()
    x = x[np.abs(x) <= 448]
    t8 = torch.from_numpy(x).to(torch.float8_e4m3fn)
    assert np.array_equal(O.e4m3_encode(x), t8.view(torch.uint8).numpy())
    codes = np.arange(256, dtype=np.uint8)
    ref = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    mine = O.e4m3_decode(codes)
    ok = ~np.isnan(ref)
    assert np.array_equal(mine[ok], ref[ok]) and np.isnan(mine[~ok]).all()


def test_byte_quantiser_differs_from_value_oracle_only_on_ties():
    """Kernel arithmetic (ties to even, multiply by 1/6, reciprocal) vs the value
    oracle (ties toward zero, divide): every differing element is an exact tie."""
    rng = np.random.default_rng(5)
    x = inputs.bf16(rng.standard_normal((256, 128)).astype(np.float32))
    nib, sb = O.quantize_groups(x)
    mine = O.dequantize_groups(nib, sb)
    theirs = O.nvfp4_round_trip(x)
    diff = mine != theirs
    frac = diff.mean()
    assert 0.001 < frac < 0.02
    s = np.repeat(O.e4m3_decode(sb), 16, axis=-1)
    ratio = np.abs(x[diff].astype(np.float64) / s[diff].astype(np.float64))
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    assert np.all(np.min(np.abs(ratio[:, None] - mids[None]), axis=1) == 0.0)
    # idempotence: both round trips leave dequantised values unchanged
    n2, s2 = O.quantize_groups(mine)
    assert np.array_equal(O.dequantize_groups(n2, s2), mine)
    assert np.array_equal(O.nvfp4_round_trip(mine), mine)


def test_layout_round_trips():
    rng = np.random.default_rng(3)
    k = inputs.bf16(rng.standard_normal((3, 128, 2, 128)).astype(np.float32))
    kp, ks = O.quantize_key_pages(k)
    vp, vs = O.quantize_value_pages(k)
    assert kp.shape == (3, 128, 2, 64) and ks.shape == (3, 2048)
    assert vp.shape == (3, 2, 128, 64) and vs.shape == (3, 2048)
    k_dq = O.dequantize_key_pages(kp, ks)
    nib, sb = O.quantize_groups(k)
    assert np.array_equal(k_dq, O.dequantize_groups(nib, sb))
    v_dq = O.dequantize_value_pages(vp, vs)
    vt = np.ascontiguousarray(k.transpose(0, 2, 3, 1))
    nib, sb = O.quantize_groups(vt)
    assert np.array_equal(v_dq, O.dequantize_groups(nib, sb).transpose(0, 3, 1, 2))
    q = inputs.bf16(rng.standard_normal((5, 8, 128)).astype(np.float32) * 3)
    qp, qs = O.quantize_query(q, 2)
    nib, sb = O.quantize_groups(q)
    assert np.array_equal(O.dequantize_query(qp, qs, 2), O.dequantize_groups(nib, sb))
    # only G of the 128 slots of each KV head block are written
    flat = qs.reshape(5, 8, 1024)
    assert np.count_nonzero(flat[:, 2:]) == 0
    assert O.vllm_block_bytes(8) == 147456


def test_split_rule_and_merge():
    fp4, res = O.split_lengths([1, 127, 128, 129, 255, 256, 257, 1000])
    assert fp4.tolist() == [0, 0, 0, 128, 128, 128, 256, 896]
    assert res.tolist() == [1, 127, 128, 1, 127, 128, 1, 104]
    assert [O.split_page_range(7, s, 4) for s in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 7)]
    assert [O.split_page_range(1, s, 4) for s in range(4)] == [(0, 1), (1, 1), (1, 1), (1, 1)]
    # merging split partials reproduces the unsplit softmax-weighted sum
    rng = np.random.default_rng(9)
    scores = rng.standard_normal((4, 512)).astype(np.float32)
    v = rng.standard_normal((512, 16)).astype(np.float32)
    full = (np.exp(scores - scores.max(1, keepdims=True)) @ v) / np.exp(
        scores - scores.max(1, keepdims=True)).sum(1, keepdims=True)
    parts, lses = [], []
    for s in range(4):
        sl = slice(s * 128, (s + 1) * 128)
        e = np.exp(scores[:, sl] - scores[:, sl].max(1, keepdims=True))
        parts.append((e @ v[sl]) / e.sum(1, keepdims=True))
        lses.append(scores[:, sl].max(1) + np.log(e.sum(1)))
    parts.append(np.full_like(parts[0], np.nan))  # an empty split may hold anything
    lses.append(np.full(4, -np.inf, dtype=np.float32))
    merged = O.lse_merge(np.stack(parts)[:, None], np.stack(lses)[:, None])
    assert np.abs(merged[0] - full).max() < 1e-5
    none = O.lse_merge(np.zeros((2, 1, 4, 16)), np.full((2, 1, 4), -np.inf))
    assert np.all(none == 0)
