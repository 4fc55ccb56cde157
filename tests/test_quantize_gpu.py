"""GPU parity: quantiser bytes (Q, K, V) and the write path (tail append / reset /
flush) against the numpy oracle, bit for bit, through the C ABI."""

import numpy as np
import pytest
import torch

import inputs
import nvfp4_oracle as O
from helpers import bf16_tensor, scale_bytes, to_np

pytestmark = pytest.mark.gpu


def _qmods():
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import _quantize, quantize_kv_kernel

    return _quantize, quantize_kv_kernel


def _storage(q_sf, rows, heads):
    return to_np(q_sf.as_strided((rows, heads * 1024), (heads * 1024, 1))).reshape(
        rows, 1, heads, 2, 32, 4, 4)


@pytest.mark.parametrize("rows", [1, 7, 8, 32])
@pytest.mark.parametrize("heads,heads_kv", [(32, 8), (16, 16), (16, 1)])
def test_query_bytes(cuda_device, rows, heads, heads_kv):
    _quantize, _ = _qmods()
    rng = np.random.default_rng(0x5200 + rows)
    q = inputs.bf16(rng.standard_normal((rows, heads, 128)).astype(np.float32) * 3.0)
    fp4, sf = _quantize.quantize_query(bf16_tensor(q, cuda_device), heads_kv=heads_kv)
    assert fp4.dtype is torch.float4_e2m1fn_x2 and tuple(fp4.shape) == (rows, 1, heads, 64)
    assert tuple(sf.shape) == (32, 4, 1, 4, 2, heads_kv, rows)
    assert sf.stride() == (16, 4, heads * 1024, 1, 512, 1024, heads * 1024)
    want_p, want_s = O.quantize_query(q, heads_kv)
    assert np.array_equal(to_np(fp4), want_p)
    assert np.array_equal(_storage(sf, rows, heads), want_s)


def test_query_indexed_strided_padded_and_scratch(cuda_device):
    _quantize, _ = _qmods()
    rng = np.random.default_rng(77)
    full = inputs.bf16(rng.standard_normal((9, 32, 256)).astype(np.float32))
    t = bf16_tensor(full, cuda_device)[:, :, :128]  # row/head strides wider than dense
    idx = torch.tensor([4, 1, 3], dtype=torch.int32, device=cuda_device)
    padded = torch.zeros(5, 128, 32, 128, dtype=torch.bfloat16, device=cuda_device)
    fp4_s = torch.full((5, 1, 32, 64), 0xA5, dtype=torch.uint8, device=cuda_device)
    sf_s = torch.zeros(5, 1, 32, 2, 32, 4, 4, dtype=torch.uint8, device=cuda_device)
    fp4, sf = _quantize.quantize_query(t, row_indices=idx, query_padded_out=padded, heads_kv=8,
                                       query_fp4_scratch=fp4_s, query_scales_scratch=sf_s)
    src = full[[4, 1, 3], :, :128]
    want_p, want_s = O.quantize_query(src, 8)
    assert np.array_equal(to_np(fp4), want_p)
    assert np.array_equal(_storage(sf, 3, 32), want_s)
    assert fp4.data_ptr() == fp4_s.data_ptr()
    assert (fp4_s[3:] == 0xA5).all()  # rows past the batch untouched
    p = to_np(padded)
    assert np.array_equal(p[:3, 0], src)
    assert not p[:, 1:].any() and not p[3:].any()


def _pages(seed, pages, heads, offset=0.0):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((pages, 128, heads, 128)).astype(np.float32)
    if offset:
        x = x + rng.standard_normal((heads, 128)).astype(np.float32)[None, None] * offset
    return inputs.bf16(x)


@pytest.mark.parametrize("heads", [1, 2, 8])
def test_dense_page_bytes(cuda_device, heads):
    _, qkv = _qmods()
    x = _pages(3 + heads, 5, heads)
    x[0, :16, 0, :16] = 0.0  # a zero group: scale 0, nibbles 0
    t = bf16_tensor(x, cuda_device)
    kp, ks = qkv.quantize_key_pages(t)
    vp, vs = qkv.quantize_value_pages(t)
    assert ks.dtype is torch.float8_e4m3fn and tuple(ks.shape) == (5, 32, 4, 1, 4, 2, heads)
    assert ks.stride() == (heads * 1024, 16, 4, 1024, 1, 512, 1024)
    wkp, wks = O.quantize_key_pages(x)
    wvp, wvs = O.quantize_value_pages(x)
    assert np.array_equal(to_np(kp), wkp) and np.array_equal(scale_bytes(ks), wks)
    assert np.array_equal(to_np(vp), wvp) and np.array_equal(scale_bytes(vs), wvs)


def test_key_shift_is_one_bf16_subtract(cuda_device):
    _, qkv = _qmods()
    x = _pages(21, 3, 8, offset=2.0)
    mu = inputs.bf16(x.reshape(-1, 8, 128).astype(np.float64).mean(0).astype(np.float32))
    kp, ks = qkv.quantize_key_pages(bf16_tensor(x, cuda_device), key_shift=bf16_tensor(mu, cuda_device))
    wkp, wks = O.quantize_key_pages(x, mu)
    assert np.array_equal(to_np(kp), wkp) and np.array_equal(scale_bytes(ks), wks)
    # same bytes as subtracting in torch first (what the reference's write path does)
    pre = torch.sub(bf16_tensor(x, cuda_device), bf16_tensor(mu, cuda_device))
    kp2, ks2 = qkv.quantize_key_pages(pre)
    assert torch.equal(kp, kp2) and torch.equal(ks.view(torch.uint8), ks2.view(torch.uint8))


def test_indexed_pitched_destinations_with_canaries(cuda_device):
    """Unaligned source windows, scattered destinations, a 100 KiB page pitch, a
    skipped item: equal to the dense quantiser byte for byte, canaries intact."""
    _, qkv = _qmods()
    heads = 2
    rng = np.random.default_rng(0xC0FFEE)
    tokens = inputs.bf16(rng.standard_normal((1200, heads, 128)).astype(np.float32))
    t = bf16_tensor(tokens, cuda_device)
    starts = [0, 37, 1000, 128, 511, 64]
    dests = [4, 1, 0, 3, 2, -1]
    pitch = 100 * 1024
    pages = 6
    for which in ("k", "v"):
        buf = torch.full((pages * pitch,), 0xA5, dtype=torch.uint8, device=cuda_device)
        inner = (128, heads, 64) if which == "k" else (heads, 128, 64)
        packed = buf.as_strided((pages,) + inner, (pitch, inner[1] * 64, 64, 1), 0)
        sf = qkv.scale_view(buf, pages, heads, pitch, 128 * heads * 64)
        fn = qkv.quantize_key_tokens_into if which == "k" else qkv.quantize_value_tokens_into
        fn(t, packed, sf, torch.tensor(starts, dtype=torch.int32, device=cuda_device),
           torch.tensor(dests, dtype=torch.int32, device=cuda_device))
        host = buf.cpu().numpy().reshape(pages, pitch)
        quant = O.quantize_key_pages if which == "k" else O.quantize_value_pages
        used = 128 * heads * 64 + heads * 1024
        for s, d in zip(starts, dests):
            if d < 0:
                continue
            wp, ws = quant(tokens[s:s + 128][None])
            assert np.array_equal(host[d, :128 * heads * 64], wp.reshape(-1)), (which, s, d)
            assert np.array_equal(host[d, 128 * heads * 64:used], ws.reshape(-1)), (which, s, d)
        assert (host[:, used:] == 0xA5).all()
        assert (host[5] == 0xA5).all()  # page 5 was nobody's destination


def test_per_layer_destination_bases_and_layer_check(cuda_device):
    _, qkv = _qmods()
    heads, layers, slots = 2, 3, 4
    rng = np.random.default_rng(5)
    src = inputs.bf16(rng.standard_normal((layers * slots * 128, heads, 128)).astype(np.float32))
    t = bf16_tensor(src, cuda_device)
    dst_p = [torch.zeros(6, 128, heads, 64, dtype=torch.uint8, device=cuda_device) for _ in range(layers)]
    dst_s = [qkv.scale_view(torch.zeros(6 * heads * 1024, dtype=torch.uint8, device=cuda_device), 6, heads)
             for _ in range(layers)]
    table = torch.tensor([[p.data_ptr() for p in dst_p], [s.data_ptr() for s in dst_s]],
                         dtype=torch.int64, device=cuda_device)
    starts = torch.tensor([128, 384], dtype=torch.int32, device=cuda_device)  # slots 1, 3
    dests = torch.tensor([5, 2], dtype=torch.int32, device=cuda_device)
    qkv.quantize_key_tokens_into(t, dst_p[0], dst_s[0], starts, dests, table)
    for layer in range(layers):
        for s, d in ((128, 5), (384, 2)):
            lo = layer * slots * 128 + s
            wp, ws = O.quantize_key_pages(src[lo:lo + 128][None])
            assert np.array_equal(to_np(dst_p[layer][d]), wp[0])
            assert np.array_equal(scale_bytes(dst_s[layer])[d], ws[0])
        assert not to_np(dst_p[layer][[0, 1, 3, 4]]).any()
    with pytest.raises(ValueError, match="does not divide"):
        qkv.quantize_key_tokens_into(t[:-1], dst_p[0], dst_s[0], starts, dests, table)


def test_tail_append_reset_flush(cuda_device):
    """One layer-stack of tail slots driven through append (with key shift), reset
    and flush; every buffer compared with the oracle's host restatement."""
    import nvfp4_attn_kernel_b200._lib as L
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import quantize_kv_kernel as qkv

    lib = L.load()
    heads, layers, slots = 2, 2, 4
    rng = np.random.default_rng(31)
    stream = torch.cuda.current_stream().cuda_stream
    tail_k = inputs.bf16(rng.standard_normal((layers, slots, 128, heads, 128)).astype(np.float32))
    tail_v = inputs.bf16(rng.standard_normal((layers, slots, 128, heads, 128)).astype(np.float32))
    tk, tv = bf16_tensor(tail_k, cuda_device), bf16_tensor(tail_v, cuda_device)
    # rows: decode row at seq 300 (slot 2), fresh 5-token prefill (slot 0), row without slot,
    # decode row whose token completes a page (seq 256, slot 3)
    qsl = np.array([0, 1, 6, 7, 8], dtype=np.int32)
    seq = np.array([300, 5, 40, 256], dtype=np.int32)
    slot = np.array([2, 0, -1, 3], dtype=np.int32)
    fp4, _ = O.split_lengths(seq)
    dev = lambda a: torch.from_numpy(a).to(cuda_device)
    d_qsl, d_seq, d_slot, d_fp4 = dev(qsl), dev(seq), dev(slot), dev(fp4)

    L.check(lib.nvfp4_tail_reset(tk.data_ptr(), tv.data_ptr(), tk.stride(0), tk.stride(1), layers,
                                 d_qsl.data_ptr(), d_seq.data_ptr(), d_slot.data_ptr(), 4, heads, stream))
    O.tail_reset(tail_k, tail_v, qsl, seq, slot)
    assert np.array_equal(to_np(tk), tail_k) and np.array_equal(to_np(tv), tail_v)
    assert not tail_k[:, 0].any() and tail_k[:, 2].any()

    key = inputs.bf16(rng.standard_normal((8, heads, 128)).astype(np.float32) + 1.5)
    val = inputs.bf16(rng.standard_normal((8, heads, 128)).astype(np.float32))
    shift = inputs.bf16(rng.standard_normal((heads, 128)).astype(np.float32))
    dk, dv, ds = bf16_tensor(key, cuda_device), bf16_tensor(val, cuda_device), bf16_tensor(shift, cuda_device)
    for layer in range(layers):
        use_shift = layer == 0
        L.check(lib.nvfp4_tail_append(dk.data_ptr(), dv.data_ptr(), dk.stride(0), dv.stride(0),
                                      ds.data_ptr() if use_shift else None,
                                      tk[layer].data_ptr(), tv[layer].data_ptr(), tk.stride(1),
                                      d_qsl.data_ptr(), d_seq.data_ptr(), d_fp4.data_ptr(),
                                      d_slot.data_ptr(), 8, 4, heads, stream))
        O.tail_append(tail_k[layer], tail_v[layer], key, val, qsl, seq, fp4, slot,
                      key_shift=shift if use_shift else None)
    assert np.array_equal(to_np(tk), tail_k) and np.array_equal(to_np(tv), tail_v)
    assert np.array_equal(tail_v[1, 3, 127], val[7])  # the page-completing token sits at offset 127

    # flush slot 3 (row 3 reached a page boundary) of every layer into block 1
    blocks = 3
    pitch = O.vllm_block_bytes(heads)
    caches = [torch.full((blocks, pitch), 0x5A, dtype=torch.uint8, device=cuda_device) for _ in range(layers)]
    o1 = 128 * heads * 64
    o2 = o1 + heads * 1024
    o3 = o2 + o1
    bases = torch.tensor([[c.data_ptr() + off for c in caches] for off in (0, o1, o2, o3)],
                         dtype=torch.int64, device=cuda_device)
    src_tok = torch.tensor([0, 128, 256, 384], dtype=torch.int32, device=cuda_device)
    dst = torch.tensor([-1, -1, -1, 1], dtype=torch.int32, device=cuda_device)
    L.check(lib.nvfp4_tail_flush(tk.data_ptr(), tv.data_ptr(), slots * 128, src_tok.data_ptr(),
                                 dst.data_ptr(), bases.data_ptr(), pitch, pitch, pitch, pitch, 4,
                                 layers, heads, stream))
    for layer in range(layers):
        host = caches[layer].cpu().numpy()
        kp, ks, vp, vs = O.tail_flush(tail_k[layer], tail_v[layer], 3)
        want = np.concatenate([kp.reshape(-1), ks.reshape(-1), vp.reshape(-1), vs.reshape(-1)])
        assert np.array_equal(host[1], want)
        assert (host[[0, 2]] == 0x5A).all()
    # the same bytes through the reference-shaped promotion calls (two launches)
    c2 = torch.zeros(blocks, pitch, dtype=torch.uint8, device=cuda_device)
    flat = c2.view(-1)
    kview = flat.as_strided((blocks, 128, heads, 64), (pitch, heads * 64, 64, 1), 0)
    vview = flat.as_strided((blocks, heads, 128, 64), (pitch, 128 * 64, 64, 1), o2)
    qkv.quantize_key_tokens_into(tk[0].reshape(-1, heads, 128), kview,
                                 qkv.scale_view(flat, blocks, heads, pitch, o1), src_tok, dst)
    qkv.quantize_value_tokens_into(tv[0].reshape(-1, heads, 128), vview,
                                   qkv.scale_view(flat, blocks, heads, pitch, o3), src_tok, dst)
    assert torch.equal(c2[1], caches[0][1])


@pytest.mark.parametrize("with_pages", [True, False])
def test_write_kv_single_launch_equals_the_three_launches(cuda_device, with_pages):
    """``nvfp4_write_kv`` (page quantisers + tail copy in one launch) against the separate
    K quantiser, V quantiser and tail append: identical blocks and identical tails.  The step mixes
    a 300-token prompt (two full pages + 44 tail tokens), a 128-token prompt (all tail), two
    decode rows and a row without a slot; without page work only the tail copy runs."""
    import nvfp4_attn_kernel_b200._lib as L
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel import quantize_kv_kernel as qkv

    lib = L.load()
    heads, slots, blocks = 2, 5, 6
    rng = np.random.default_rng(41)
    stream = torch.cuda.current_stream().cuda_stream
    if with_pages:
        qlen = np.array([1, 1, 1, 128, 300], dtype=np.int32)      # one-token rows first
        seq = np.array([200, 513, 77, 128, 300], dtype=np.int32)
        slot = np.array([4, 0, -1, 2, 1], dtype=np.int32)
    else:
        qlen = np.array([1, 1, 1], dtype=np.int32)
        seq = np.array([200, 513, 77], dtype=np.int32)
        slot = np.array([4, 0, -1], dtype=np.int32)
    qsl = np.concatenate([[0], np.cumsum(qlen)]).astype(np.int32)
    tokens = int(qsl[-1])
    fp4, _ = O.split_lengths(seq)
    dev = lambda a: torch.from_numpy(a).to(cuda_device)
    d_qsl, d_seq, d_slot, d_fp4 = dev(qsl), dev(seq), dev(slot), dev(fp4)
    key = bf16_tensor(rng.standard_normal((tokens, heads, 128)).astype(np.float32) + 1.0, cuda_device)
    val = bf16_tensor(rng.standard_normal((tokens, heads, 128)).astype(np.float32), cuda_device)
    shift = bf16_tensor(rng.standard_normal((heads, 128)).astype(np.float32), cuda_device)
    # page work of the 300-token prompt: its tokens start at qsl[4]; pages go to blocks 5 and 2
    if with_pages:
        src = torch.tensor([int(qsl[4]), int(qsl[4]) + 128, 0], dtype=torch.int32, device=cuda_device)
        dst = torch.tensor([5, 2, -1], dtype=torch.int32, device=cuda_device)
    else:
        src = torch.zeros(0, dtype=torch.int32, device=cuda_device)
        dst = torch.zeros(0, dtype=torch.int32, device=cuda_device)
    pitch = O.vllm_block_bytes(heads)
    o1 = 128 * heads * 64
    o2 = o1 + heads * 1024
    o3 = o2 + o1

    def views(cache):
        flat = cache.view(-1)
        return (flat.as_strided((blocks, 128, heads, 64), (pitch, heads * 64, 64, 1), 0),
                qkv.scale_view(flat, blocks, heads, pitch, o1),
                flat.as_strided((blocks, heads, 128, 64), (pitch, 128 * 64, 64, 1), o2),
                qkv.scale_view(flat, blocks, heads, pitch, o3))

    base_tail = torch.randn(2, slots, 128, heads, 128, device=cuda_device).to(torch.bfloat16)
    # three launches
    cache_a = torch.full((blocks, pitch), 0x3C, dtype=torch.uint8, device=cuda_device)
    tail_a = base_tail.clone()
    ka, ksa, va, vsa = views(cache_a)
    if with_pages:
        qkv.quantize_key_tokens_into(key, ka, ksa, src, dst, key_shift=shift)
        qkv.quantize_value_tokens_into(val, va, vsa, src, dst)
    L.check(lib.nvfp4_tail_append(key.data_ptr(), val.data_ptr(), key.stride(0), val.stride(0), shift.data_ptr(),
                                  tail_a[0].data_ptr(), tail_a[1].data_ptr(), tail_a.stride(1), d_qsl.data_ptr(),
                                  d_seq.data_ptr(), d_fp4.data_ptr(), d_slot.data_ptr(), tokens, len(seq), heads,
                                  stream))
    # one launch
    cache_b = torch.full((blocks, pitch), 0x3C, dtype=torch.uint8, device=cuda_device)
    tail_b = base_tail.clone()
    kb, ksb, vb, vsb = views(cache_b)
    work = int(dst.numel())
    L.check(lib.nvfp4_write_kv(
        key.data_ptr(), val.data_ptr(), key.stride(0), val.stride(0), shift.data_ptr(),
        kb.data_ptr() if work else None, pitch, ksb.data_ptr() if work else None, pitch,
        vb.data_ptr() if work else None, pitch, vsb.data_ptr() if work else None, pitch,
        src.data_ptr() if work else None, dst.data_ptr() if work else None, work,
        tail_b[0].data_ptr(), tail_b[1].data_ptr(), tail_b.stride(1), d_qsl.data_ptr(), d_seq.data_ptr(),
        d_fp4.data_ptr(), d_slot.data_ptr(), tokens, len(seq), heads, stream))
    torch.cuda.synchronize()
    assert torch.equal(cache_a, cache_b) and torch.equal(tail_a, tail_b)
    assert not torch.equal(tail_a, base_tail)
    if with_pages:
        assert not (cache_a[[5, 2]] == 0x3C).all() and (cache_a[[0, 1, 3, 4]] == 0x3C).all()


@pytest.mark.parametrize("tokens,heads,padded", [(1, 8, False), (7, 2, False), (333, 8, True), (40000, 8, False),
                                                 (4097, 1, True)])
def test_key_sum_accumulate_equals_the_fp64_sum(cuda_device, tokens, heads, padded):
    """The calibration's accumulation (reference: src/nvfp4_vllm/impl.py:137-144,
    ``key.double().sum(dim=0)``; its CPU test of the fp64 accumulator is
    tests/e2e/test_key_shift.py:134-153).  BF16 addends make every fp64 partial sum exact, so
    the launch must equal the fp64 sum bit for bit, whatever the order it added in; a second
    call adds on top of the first."""
    from nvfp4_attn_kernel_b200.nvfp4_vllm.write import accumulate_key_sum

    gen = torch.Generator(device=cuda_device)
    gen.manual_seed(tokens * 31 + heads)
    width = heads * 128
    # multiples of 1/64 below 16: every fp64 partial sum is exact, whatever the order
    store = torch.randn(tokens, width + (64 if padded else 0), device=cuda_device, generator=gen) * 3.0 + 1.5
    store = (torch.round(store.clamp(-15, 15) * 64) / 64).to(torch.bfloat16)
    key = store[:, :width].view(tokens, heads, 128) if not padded else \
        store.as_strided((tokens, heads, 128), (width + 64, 128, 1))
    acc = torch.zeros(heads, 128, dtype=torch.float64, device=cuda_device)
    accumulate_key_sum(key, acc)
    want = key.double().sum(dim=0)
    # the oracle side of the claim: numpy's own fp64 sum of the same values
    want_np = to_np(key.float()).astype(np.float64).sum(axis=0)
    assert np.array_equal(want.cpu().numpy(), want_np)
    assert torch.equal(acc, want)
    accumulate_key_sum(key[: max(1, tokens // 2)], acc)
    assert torch.equal(acc, want + key[: max(1, tokens // 2)].double().sum(dim=0))
    # unconstrained values (a few land next to zero, with bits far below the sum's last place)
    wild = (torch.randn(tokens, heads, 128, device=cuda_device, generator=gen) * 0.3).to(torch.bfloat16)
    acc.zero_()
    accumulate_key_sum(wild, acc)
    assert torch.allclose(acc, wild.double().sum(dim=0), rtol=0, atol=1e-10)
    with pytest.raises(ValueError):
        accumulate_key_sum(key, acc.float())
    with pytest.raises(ValueError):
        accumulate_key_sum(key.float(), acc)
