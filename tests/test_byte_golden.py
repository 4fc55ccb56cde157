"""Quantised bytes against a fixture this repository's code did not produce.

``tests/golden/quant_bytes.npz`` was written on a B200 by ``tests/golden/make_byte_golden.py``:
FlashInfer ``fp4_quantize`` (global scale 1, swizzled scales) called as the reference's test aid
calls it, and the reference's own CuTeDSL quantiser kernels, on seeded inputs that the
generator module rebuilds here.  The numpy byte oracle must equal the fixture bit for bit (CPU);
the library must equal it bit for bit (GPU, through the C ABI).
"""

import os

import numpy as np
import pytest

import make_byte_golden as G
import nvfp4_oracle as O

FIXTURE = os.path.join(os.path.dirname(os.path.abspath(G.__file__)), "quant_bytes.npz")


@pytest.fixture(scope="module")
def golden():
    assert os.path.exists(FIXTURE), "tests/golden/quant_bytes.npz is missing"
    return np.load(FIXTURE)


def _producers(golden):
    """Prefixes of the producers the fixture holds bytes from."""
    have = [p for p, key in (("fi", "flashinfer_error"), ("ref", "reference_error")) if str(golden[key]) == ""]
    assert have, "the fixture holds bytes of neither producer"
    return have


def _query_storage(view7: np.ndarray) -> np.ndarray:
    """(32, 4, 1, 4, 2, heads_kv, rows) scale view -> the bytes of every (row, KV head) block in
    storage order [rows, heads_kv, 2, 32, 4, 4]."""
    return np.ascontiguousarray(view7[:, :, 0].transpose(5, 4, 3, 0, 1, 2))


def _oracle_query(rows):
    packed, storage = O.quantize_query(G.query_input(rows), G.Q_HEADS)   # heads_kv = heads
    return packed, storage.reshape(rows, G.Q_HEADS, 2, 32, 4, 4)


@pytest.mark.parametrize("rows", G.Q_ROWS)
def test_oracle_query_bytes_equal_the_fixture(golden, rows):
    packed, storage = _oracle_query(rows)
    for prod in _producers(golden):
        assert np.array_equal(packed, golden[f"{prod}_q{rows}_fp4"]), prod
        assert np.array_equal(storage, _query_storage(golden[f"{prod}_q{rows}_sf"])), prod


def _oracle_pages(heads):
    win = G.windows(G.token_input(heads))
    return O.quantize_key_pages(win), O.quantize_value_pages(win)


def _sf_bytes(a: np.ndarray) -> np.ndarray:
    """[pages, 32, 4, 1, 4, 2, heads] scale array (logical order) -> [pages, heads * 1024] bytes."""
    pages, heads = a.shape[0], a.shape[-1]
    # logical index (r32, r4, 0, g4, atom, h) sits at byte h*1024 + atom*512 + r32*16 + r4*4 + g4
    return np.ascontiguousarray(a[:, :, :, 0].transpose(0, 5, 4, 1, 2, 3)).reshape(pages, heads * 1024)


def _check_pages(golden, heads, got, tag):
    (kp, ks), (vp, vs) = got
    order = np.argsort(np.array(G.DESTINATIONS))   # page p of an indexed destination holds window order[p]
    full = heads == G.KV_HEADS_FULL
    for name, arr, indexed in (("k", (kp, ks), False), ("v", (vp, vs), False),
                               ("k", (kp, ks), True), ("v", (vp, vs), True)):
        packed, sf = arr
        if indexed:
            packed, sf = packed[order], sf[order]
        key = f"ref_{name}{heads}" + ("_into" if indexed else "")
        for part, mine in (("packed", packed), ("sf", sf)):
            if full:
                want = golden[f"{key}_{part}"]
                want = _sf_bytes(want) if part == "sf" else want
                assert np.array_equal(mine.reshape(want.shape), want), f"{tag} {key}_{part}"
        if indexed:
            assert bool(golden[f"{key}_canaries_intact"])


@pytest.mark.parametrize("heads", [G.KV_HEADS_FULL])
def test_oracle_page_bytes_equal_the_reference_kernels(golden, heads):
    if str(golden["reference_error"]):
        pytest.skip("the reference's quantiser kernels did not run where the fixture was made: "
                    + str(golden["reference_error"])[-200:])
    _check_pages(golden, heads, _oracle_pages(heads), "oracle")


def test_reference_digests_of_the_eight_head_case(golden):
    """For 8 KV heads the fixture holds SHA-256 digests of the reference's outputs."""
    if str(golden["reference_error"]):
        pytest.skip("no reference bytes in the fixture")
    (kp, ks), (vp, vs) = _oracle_pages(G.KV_HEADS_DIGEST)
    heads = G.KV_HEADS_DIGEST

    def to_logical(sf):   # byte h*1024 + atom*512 + r32*16 + r4*4 + g4 -> [page, r32, r4, 0, g4, atom, h]
        b = sf.reshape(-1, heads, 2, 32, 4, 4)            # [page, h, atom, r32, r4, g4]
        return np.ascontiguousarray(b.transpose(0, 3, 4, 5, 2, 1)[:, :, :, None])
    for name, packed, sf in (("k", kp, ks), ("v", vp, vs)):
        assert np.array_equal(G.digest(packed), golden[f"ref_{name}{heads}_packed_sha256"])
        assert np.array_equal(G.digest(to_logical(sf)), golden[f"ref_{name}{heads}_sf_sha256"])


# ---------------------------------------------------------------------------- GPU


@pytest.mark.gpu
@pytest.mark.parametrize("rows", G.Q_ROWS)
def test_library_query_bytes_equal_the_fixture(golden, cuda_device, rows):
    from helpers import bf16_tensor, to_np
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel._quantize import quantize_query

    fp4, sf = quantize_query(bf16_tensor(G.query_input(rows), cuda_device))
    for prod in _producers(golden):
        assert np.array_equal(to_np(fp4), golden[f"{prod}_q{rows}_fp4"]), prod
        assert np.array_equal(to_np(sf.contiguous()), golden[f"{prod}_q{rows}_sf"]), prod


@pytest.mark.gpu
def test_library_page_bytes_equal_the_reference_kernels(golden, cuda_device):
    import torch
    from helpers import bf16_tensor, scale_bytes, to_np
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import quantize_kv_kernel as qkv

    if str(golden["reference_error"]):
        pytest.skip("no reference bytes in the fixture")
    heads = G.KV_HEADS_FULL
    tok = G.token_input(heads)
    win = bf16_tensor(G.windows(tok), cuda_device)
    kp, ks = qkv.quantize_key_pages(win)
    vp, vs = qkv.quantize_value_pages(win)
    _check_pages(golden, heads, ((to_np(kp), scale_bytes(ks)), (to_np(vp), scale_bytes(vs))), "library dense")
    # the indexed entry points, pages 100 KiB apart
    pitch = 100 * 1024
    t = bf16_tensor(tok, cuda_device)
    starts = torch.tensor(G.STARTS, dtype=torch.int32, device=cuda_device)
    dests = torch.tensor(G.DESTINATIONS, dtype=torch.int32, device=cuda_device)
    n = len(G.STARTS)
    for name, fn, shape, strides in (
        ("k", qkv.quantize_key_tokens_into, (128, heads, 64), (heads * 64, 64, 1)),
        ("v", qkv.quantize_value_tokens_into, (heads, 128, 64), (128 * 64, 64, 1)),
    ):
        pbuf = torch.full((n, pitch), 0xA5, dtype=torch.uint8, device=cuda_device)
        sbuf = torch.full((n, pitch), 0xA5, dtype=torch.uint8, device=cuda_device)
        packed = pbuf.as_strided((n,) + shape, (pitch,) + strides, 0)
        scales = sbuf.as_strided((n, 32, 4, 1, 4, 2, heads), (pitch, 16, 4, 1024, 1, 512, 1024), 0)
        fn(t, packed, scales, starts, dests)
        assert np.array_equal(to_np(packed), golden[f"ref_{name}{heads}_into_packed"])
        assert np.array_equal(to_np(scales.contiguous()), golden[f"ref_{name}{heads}_into_sf"])
