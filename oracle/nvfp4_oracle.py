"""CPU oracle for the paged NVFP4/BF16 hybrid decode-attention path.

TEST INFRASTRUCTURE ONLY.  This module is a numpy restatement of the reference
algorithm.  Nothing in the shipped package imports it; only the test-suite, the
smoke check and the CPU-baseline leg of the benchmark do, and only as the
checker or the thing timed as "the CPU path".

Parity pin: every function here is checked (tests/test_oracle_pins.py) against
golden vectors produced by importing the reference's own torch code
(``src/nvfp4_decode_kernel/reference.py`` and the attention oracle in
``tests/kernel/test_fp4_decode_correctness.py``) with the script
``tests/golden/make_golden.py``; the byte converters are additionally pinned
against NVIDIA's host conversion routines in ``cuda_fp4.h``/``cuda_fp8.h``
(``oracle/cvt_check.cpp``) and against torch's ``float8_e4m3fn`` cast.

All arrays are numpy.  BF16 tensors are carried as float32 arrays whose values
are exactly representable in bfloat16 (use :func:`bf16_round`).

Reference citations are relative to the reference project root.
"""

from __future__ import annotations

import numpy as np

PAGE = 128
HEAD_DIM = 128
GROUP = 16

E2M1_MAGNITUDES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


# --------------------------------------------------------------------------
# number formats  (reference: reference.py:8-27, quantize_q_kernel.py:20-95)
# --------------------------------------------------------------------------

def bf16_round(x) -> np.ndarray:
    """Round float32 values to the nearest bfloat16 (ties to even), as float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    bias = np.uint64(0x7FFF) + ((bits >> np.uint64(16)) & np.uint64(1))
    out = (((bits + bias) >> np.uint64(16)) << np.uint64(16)).astype(np.uint32)
    out = np.where(np.isnan(x), x.view(np.uint32), out).astype(np.uint32)
    return out.view(np.float32).reshape(x.shape)


def bf16_bits(x) -> np.ndarray:
    """uint16 bit patterns of bf16-exact float32 values."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    return (x.view(np.uint32) >> np.uint32(16)).astype(np.uint16).reshape(x.shape)


def bf16_from_bits(u16) -> np.ndarray:
    u = np.ascontiguousarray(u16, dtype=np.uint16).astype(np.uint32) << np.uint32(16)
    return u.view(np.float32).reshape(np.shape(u16))


def e4m3_encode(x) -> np.ndarray:
    """float32 -> E4M3 (fn) byte, round-to-nearest-even, saturate-to-finite.

    Semantics of ``cvt.rn.satfinite.e4m3x2.f32`` (quantize_q_kernel.py:38-43):
    magnitudes above 448 saturate to 448 (0x7E), NaN -> 0x7F.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    sign = (x.view(np.uint32) >> np.uint32(24)) & np.uint32(0x80)
    a = np.abs(x)
    bits = a.view(np.uint32).astype(np.uint64)
    # normal range of e4m3: exponent >= -6
    rb = np.uint64(0x7FFFF) + ((bits >> np.uint64(20)) & np.uint64(1))
    norm = ((bits + rb) >> np.uint64(20)).astype(np.int64) - ((127 - 7) << 3)
    sub = np.rint(a.astype(np.float64) * 512.0).astype(np.int64)  # RN-even, units of 2^-9
    code = np.where(a < np.float32(2.0 ** -6), sub, norm)
    code = np.clip(code, 0, 0x7E)
    code = np.where(np.isnan(x), 0x7F, code)
    return (code.astype(np.uint32) | sign).astype(np.uint8).reshape(x.shape)


def e4m3_decode(b) -> np.ndarray:
    """E4M3 (fn) byte -> float32."""
    b = np.ascontiguousarray(b, dtype=np.uint8).astype(np.int32)
    sign = np.where(b & 0x80, -1.0, 1.0).astype(np.float32)
    e = (b >> 3) & 0xF
    m = b & 7
    normal = np.ldexp((8 + m).astype(np.float32), e - 7 - 3)
    subn = np.ldexp(m.astype(np.float32), -9)
    out = np.where(e == 0, subn, normal).astype(np.float32)
    out = np.where((b & 0x7F) == 0x7F, np.float32(np.nan), out)
    return (sign * out).astype(np.float32)


def e2m1_encode(x) -> np.ndarray:
    """float32 -> E2M1 nibble (sign bit 3), RN-even, saturate to +-6.

    Semantics of ``cvt.rn.satfinite.e2m1x2.f32`` (quantize_q_kernel.py:84-88).
    A tie goes to the code with an even index: 0.25->0, 0.75->1.0, 1.25->1.0,
    1.75->2.0, 2.5->2.0, 3.5->4.0, 5.0->4.0.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    a = np.abs(x)
    code = (
        (a > 0.25).astype(np.uint8)
        + (a >= 0.75)
        + (a > 1.25)
        + (a >= 1.75)
        + (a > 2.5)
        + (a >= 3.5)
        + (a > 5.0)
    ).astype(np.uint8)
    sign = (np.signbit(x).astype(np.uint8) << 3).astype(np.uint8)
    sign = np.where(np.isnan(x), 0, sign).astype(np.uint8)
    code = np.where(np.isnan(x), 7, code).astype(np.uint8)  # NaN saturates to max magnitude
    return (code | sign).astype(np.uint8)


def e2m1_decode(n) -> np.ndarray:
    n = np.ascontiguousarray(n, dtype=np.uint8)
    mag = E2M1_MAGNITUDES[n & 7]
    return np.where(n & 8, -mag, mag).astype(np.float32)


def round_e2m1_ties_down(x) -> np.ndarray:
    """The reference value oracle's rounding (reference.py:8-27).

    ``bucketize(|x|, midpoints, right=False)`` sends an exact midpoint to the
    LOWER magnitude; non-finite inputs map to 0.
    """
    x = np.asarray(x, dtype=np.float32)
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    a = np.abs(x)
    idx = np.searchsorted(mids, a, side="left")
    idx = np.where(np.isfinite(a), idx, 0)
    return (np.sign(x) * E2M1_MAGNITUDES[idx]).astype(np.float32)


def nvfp4_round_trip(x, group: int = GROUP) -> np.ndarray:
    """Restatement of ``nvfp4_round_trip`` (reference.py:30-46), fp32 in/out."""
    x = np.asarray(x, dtype=np.float32)
    if group <= 0:
        raise ValueError(f"group must be positive, got {group}")
    if x.shape[-1] % group != 0:
        raise ValueError(
            f"last dimension {x.shape[-1]} must be divisible by group {group}"
        )
    g = x.reshape(*x.shape[:-1], -1, group)
    scale = np.abs(g).max(axis=-1, keepdims=True) / np.float32(6.0)
    scale = e4m3_decode(e4m3_encode(scale.astype(np.float32)))
    zero = scale == 0
    safe = np.where(zero, np.float32(1.0), scale)
    q = round_e2m1_ties_down((g / safe).astype(np.float32)) * scale
    q = np.where(zero, g, q)
    return q.reshape(x.shape).astype(np.float32)


# --------------------------------------------------------------------------
# byte oracle: the quantiser kernels' arithmetic
# (quantize_q_kernel.py:133-227, quantize_kv_kernel.py:70-176)
# --------------------------------------------------------------------------

_INV6 = np.float32(1.0 / 6.0)


def quantize_groups(x):
    """Quantise the last axis in groups of 16 with the kernels' arithmetic.

    ``s = e4m3_rn_satfinite(amax * fp32(1/6))``; ``inv = 1.0f / (float(s) + 1e-30f)``
    (IEEE division); nibble = ``e2m1_rn_satfinite(x * inv)``.

    Returns (nibbles uint8 [..., n], scale bytes uint8 [..., n/16]).
    """
    x = np.asarray(x, dtype=np.float32)
    g = x.reshape(*x.shape[:-1], -1, GROUP)
    amax = np.abs(g).max(axis=-1)
    sbytes = e4m3_encode((amax * _INV6).astype(np.float32))
    s = e4m3_decode(sbytes)
    inv = (np.float32(1.0) / (s + np.float32(1.0e-30))).astype(np.float32)
    y = (g * inv[..., None]).astype(np.float32)
    nib = e2m1_encode(y).reshape(x.shape)
    return nib, sbytes


def dequantize_groups(nib, sbytes) -> np.ndarray:
    v = e2m1_decode(nib).reshape(*nib.shape[:-1], -1, GROUP)
    return (v * e4m3_decode(sbytes)[..., None]).reshape(nib.shape).astype(np.float32)


def pack_nibbles(nib) -> np.ndarray:
    """Two nibbles per byte along the last axis, even element in the LOW nibble
    (quantize_q_kernel.py:84-88)."""
    nib = np.asarray(nib, dtype=np.uint8)
    return (nib[..., 0::2] | (nib[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed) -> np.ndarray:
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = packed >> 4
    return out


def sf_atom_offset(row, group):
    """Byte offset of (row in [0,128), 16-element group in [0,8)) inside one
    1024-byte per-head scale block (two 512-byte atoms).

    quantize_kv_kernel.py:119 / 420-441: shape (32,4,rest_m,4,rest_k), strides
    (16,4,.,1,512): row -> (row%32)*16 + (row//32)*4, group -> (g//4)*512 + g%4.
    """
    row = np.asarray(row)
    group = np.asarray(group)
    return (group // 4) * 512 + (row % 32) * 16 + (row // 32) * 4 + (group % 4)


def quantize_query(q_bf16, heads_kv: int):
    """Q quantiser bytes (quantize_query, _quantize.py:14-117; K1).

    q_bf16: [rows, Hq, 128] bf16-exact float32.
    Returns packed [rows, 1, Hq, 64] uint8 and the scale storage
    [rows, 1, Hq, 2, 32, 4, 4] uint8 (zero except the written slots).
    """
    q = np.asarray(q_bf16, dtype=np.float32)
    rows, hq, d = q.shape
    assert d == HEAD_DIM and hq % heads_kv == 0
    g_per = hq // heads_kv
    nib, sb = quantize_groups(q)
    packed = pack_nibbles(nib).reshape(rows, 1, hq, d // 2)
    storage = np.zeros((rows, hq * 1024), dtype=np.uint8)
    for h in range(hq):
        slot = h % g_per
        base = (h // g_per) * 1024
        offs = base + sf_atom_offset(slot, np.arange(8))
        storage[:, offs] = sb[:, h, :]
    return packed, storage.reshape(rows, 1, hq, 2, 32, 4, 4)


def quantize_key_pages(k_pages_bf16, key_shift_bf16=None):
    """K page quantiser bytes (quantize_key_pages, quantize_kv_kernel.py:750-784; K2)
    with the optional per-channel key shift applied first as one BF16 subtract
    (impl.py:145-152).

    k_pages: [pages, 128, Hkv, 128]; key_shift: [Hkv, 128] or None.
    Returns packed [pages, 128, Hkv, 64] and scales [pages, Hkv*1024] uint8.
    """
    k = np.asarray(k_pages_bf16, dtype=np.float32)
    if key_shift_bf16 is not None:
        k = bf16_round(k - np.asarray(key_shift_bf16, dtype=np.float32)[None, None])
    pages, page, hkv, d = k.shape
    assert page == PAGE and d == HEAD_DIM
    nib, sb = quantize_groups(k)  # sb [pages, tok, head, 8]
    packed = pack_nibbles(nib)
    scales = np.zeros((pages, hkv * 1024), dtype=np.uint8)
    tok = np.arange(PAGE)[:, None]
    grp = np.arange(8)[None, :]
    off = sf_atom_offset(tok, grp)  # [128, 8]
    for h in range(hkv):
        scales[:, (h * 1024 + off).reshape(-1)] = sb[:, :, h, :].reshape(pages, -1)
    return packed, scales


def quantize_value_pages(v_pages_bf16):
    """V page quantiser bytes (quantize_value_pages, quantize_kv_kernel.py:787-822; K3).

    Groups run along the TOKEN axis: for each (head, channel) the 128 tokens of
    the page form 8 groups of 16.  packed [pages, Hkv, 128(d), 64]: byte j of
    row d holds tokens 2j (low nibble) and 2j+1 (high).
    """
    v = np.asarray(v_pages_bf16, dtype=np.float32)
    pages, page, hkv, d = v.shape
    assert page == PAGE and d == HEAD_DIM
    vt = np.ascontiguousarray(v.transpose(0, 2, 3, 1))  # [pages, head, d, tok]
    nib, sb = quantize_groups(vt)  # sb [pages, head, d, 8]
    packed = pack_nibbles(nib)
    scales = np.zeros((pages, hkv * 1024), dtype=np.uint8)
    ch = np.arange(HEAD_DIM)[:, None]
    grp = np.arange(8)[None, :]
    off = sf_atom_offset(ch, grp)
    for h in range(hkv):
        scales[:, (h * 1024 + off).reshape(-1)] = sb[:, h].reshape(pages, -1)
    return packed, scales


def dequantize_query(packed, storage, heads_kv: int) -> np.ndarray:
    rows, _, hq, _ = packed.shape
    g_per = hq // heads_kv
    flat = storage.reshape(rows, hq * 1024)
    nib = unpack_nibbles(packed.reshape(rows, hq, 64))
    sb = np.zeros((rows, hq, 8), dtype=np.uint8)
    for h in range(hq):
        offs = (h // g_per) * 1024 + sf_atom_offset(h % g_per, np.arange(8))
        sb[:, h, :] = flat[:, offs]
    return dequantize_groups(nib, sb)


def dequantize_key_pages(packed, scales) -> np.ndarray:
    pages, _, hkv, _ = packed.shape
    nib = unpack_nibbles(packed)
    off = sf_atom_offset(np.arange(PAGE)[:, None], np.arange(8)[None, :])
    sb = np.zeros((pages, PAGE, hkv, 8), dtype=np.uint8)
    for h in range(hkv):
        sb[:, :, h, :] = scales[:, (h * 1024 + off).reshape(-1)].reshape(pages, PAGE, 8)
    return dequantize_groups(nib, sb)  # [pages, tok, head, d]


def dequantize_value_pages(packed, scales) -> np.ndarray:
    pages, hkv, _, _ = packed.shape
    nib = unpack_nibbles(packed)  # [pages, head, d, tok]
    off = sf_atom_offset(np.arange(HEAD_DIM)[:, None], np.arange(8)[None, :])
    sb = np.zeros((pages, hkv, HEAD_DIM, 8), dtype=np.uint8)
    for h in range(hkv):
        sb[:, h] = scales[:, (h * 1024 + off).reshape(-1)].reshape(pages, HEAD_DIM, 8)
    vt = dequantize_groups(nib, sb)
    return np.ascontiguousarray(vt.transpose(0, 3, 1, 2))  # [pages, tok, head, d]


def vllm_block_bytes(heads_kv: int) -> int:
    """Bytes of one vLLM block: K packed, K scales, V packed, V scales
    (backend.py:30-41, layout.py:63-103)."""
    return 2 * (PAGE * heads_kv * 64 + heads_kv * 1024)


def assemble_vllm_blocks(k_packed, k_scales, v_packed, v_scales) -> np.ndarray:
    pages = k_packed.shape[0]
    return np.concatenate(
        [
            k_packed.reshape(pages, -1),
            k_scales.reshape(pages, -1),
            v_packed.reshape(pages, -1),
            v_scales.reshape(pages, -1),
        ],
        axis=1,
    )


# --------------------------------------------------------------------------
# write path: split rule, tail append / reset / flush
# (control.py:279-282, write.py:79-179, promote.py:33-62)
# --------------------------------------------------------------------------

def split_lengths(seq_len):
    """seqused_fp4 = ((seq-1)//128)*128, seqused_residual = seq - seqused_fp4."""
    seq_len = np.asarray(seq_len, dtype=np.int64)
    fp4 = np.where(seq_len > 0, ((seq_len - 1) // PAGE) * PAGE, 0)
    return fp4.astype(np.int32), (seq_len - fp4).astype(np.int32)


def tail_append(tail_key, tail_value, key, value, query_start_loc, seq_lens,
                seqused_fp4, row_to_slot, key_shift=None):
    """Tail write (write.py:79-130) for one layer, in place.

    tail_*: [slots, 128, Hkv, D]; key/value: [tokens, Hkv, D] bf16-exact.
    ``offset = seq_len + token - row_end - seqused_fp4``; written iff the row's
    slot >= 0 and offset >= 0.  The shift is a BF16 subtract (impl.py:152).
    """
    tokens = key.shape[0]
    ends = np.asarray(query_start_loc)[1:]
    for t in range(tokens):
        row = int(np.sum(ends <= t))
        if row >= len(seq_lens):
            continue
        slot = int(row_to_slot[row])
        off = int(seq_lens[row]) + t - int(ends[row]) - int(seqused_fp4[row])
        if slot >= 0 and off >= 0:
            k = key[t]
            if key_shift is not None:
                k = bf16_round(k - key_shift)
            tail_key[slot, off] = k
            tail_value[slot, off] = value[t]


def tail_reset(tail_key, tail_value, query_start_loc, seq_lens, row_to_slot):
    """Tail reset (write.py:133-179): tail_*: [L, slots, 128, Hkv, D]."""
    qsl = np.asarray(query_start_loc)
    for row in range(len(seq_lens)):
        slot = int(row_to_slot[row])
        if slot >= 0 and int(seq_lens[row]) <= int(qsl[row + 1] - qsl[row]):
            tail_key[:, slot] = 0
            tail_value[:, slot] = 0


def tail_flush(tail_key_layer, tail_value_layer, slot: int):
    """Promotion of one filled tail page (promote.py:33-62): returns the four
    byte regions for the destination block."""
    kp, ks = quantize_key_pages(tail_key_layer[slot][None])
    vp, vs = quantize_value_pages(tail_value_layer[slot][None])
    return kp[0], ks[0], vp[0], vs[0]


# --------------------------------------------------------------------------
# attention oracle
# (tests/kernel/test_fp4_decode_correctness.py:145-247)
# --------------------------------------------------------------------------

def online_softmax_pv(scores, v, residual_mask, return_lse: bool = False):
    """Restatement of ``_online_softmax_pv`` (test_fp4_decode_correctness.py:194-247).

    scores: [H, L] fp32 for one batch row (masked positions = -inf), L a
    multiple of 128; v: [L, H, D]; residual_mask: [L] bool.
    Pages are walked from the last to the first; P of an FP4 page goes through
    ``nvfp4_round_trip`` (groups of 16 positions), P of residual positions is
    cast to BF16; the row sum uses unquantised P.
    """
    heads, length = scores.shape
    d = v.shape[-1]
    out = np.zeros((heads, d), dtype=np.float32)
    run_max = np.full((heads,), -np.inf, dtype=np.float32)
    run_sum = np.zeros((heads,), dtype=np.float32)
    with np.errstate(invalid="ignore", over="ignore"):
        for start in range(length - PAGE, -1, -PAGE):
            block = scores[:, start:start + PAGE]
            block_max = np.maximum(run_max, block.max(axis=-1))
            rescale = np.exp(run_max - block_max)
            rescale = np.where(np.isfinite(rescale), rescale, 0.0).astype(np.float32)
            finite_max = np.where(block_max > -np.inf, block_max, 0.0).astype(np.float32)
            p = np.exp(block - finite_max[:, None]).astype(np.float32)
            run_sum = run_sum * rescale + p.sum(axis=-1, dtype=np.float32)
            out = out * rescale[:, None]
            res = residual_mask[start:start + PAGE]
            p_block = np.where(res[None, :], bf16_round(p), nvfp4_round_trip(p))
            vb = v[start:start + PAGE]  # [128, H, D]
            out = out + np.einsum("hk,khd->hd", p_block, vb).astype(np.float32)
            run_max = block_max
    with np.errstate(invalid="ignore", divide="ignore"):
        o = (out / run_sum[:, None]).astype(np.float32)
        if return_lse:
            lse = (run_max + np.log(run_sum)).astype(np.float32)
            return o, lse
    return o


def attention_from_dequantized(
    q_bf16,
    q_dq,
    k_dq_pages,
    v_dq_pages,
    page_table,
    seqused_fp4,
    tail_key=None,
    tail_value=None,
    tail_ids=None,
    seqused_residual=None,
    softmax_scale=None,
    page_range=None,
    owns_tail: bool = True,
    return_lse: bool = False,
):
    """Hybrid decode with the FP4 operands supplied already dequantised.

    Same arithmetic as ``_torch_fp4_decode`` (test_fp4_decode_correctness.py:145-191)
    after its round-trips: FP4 positions use ``q_dq . k_dq``, tail positions use
    ``q_bf16 . k_tail`` and BF16 P / V.  Feeding the kernel's own dequantised
    bytes removes the tie-rounding difference between the value oracle
    (ties to the lower magnitude) and the hardware converter (ties to even).

    q_bf16/q_dq: [rows, Hq, D]; k_dq_pages/v_dq_pages: [pages, 128, Hkv, D];
    tail_*: [slots, 128, Hkv, D]; ``page_range(n_pages) -> (first, last)``
    restricts the FP4 pages of every row to that logical range and
    ``owns_tail`` says whether this range also takes the BF16 tail (the split
    path gives it to split 0: _fa4/block_info.py:46-54, fp4_decode_kernel.py:159).
    """
    rows, hq, d = q_dq.shape
    hkv = k_dq_pages.shape[2]
    rep = hq // hkv
    if softmax_scale is None:
        softmax_scale = d ** -0.5
    scale = np.float32(softmax_scale)
    out = np.zeros((rows, hq, d), dtype=np.float32)
    lses = np.full((rows, hq), -np.inf, dtype=np.float32)
    for r in range(rows):
        n_pages = int(seqused_fp4[r]) // PAGE
        first, last = 0, n_pages
        if page_range is not None:
            first, last = page_range(n_pages)
        res_len = 0
        if seqused_residual is not None and tail_key is not None and owns_tail:
            res_len = int(seqused_residual[r])
        blocks_k, blocks_v, blocks_s, blocks_res = [], [], [], []
        for p in range(first, last):
            pid = int(page_table[r, p])
            kk = np.repeat(k_dq_pages[pid], rep, axis=1)  # [128, Hq, D]
            vv = np.repeat(v_dq_pages[pid], rep, axis=1)
            s = np.einsum("hd,khd->hk", q_dq[r], kk).astype(np.float32) * scale
            blocks_s.append(s)
            blocks_v.append(vv)
            blocks_res.append(np.zeros(PAGE, dtype=bool))
        if res_len > 0:
            slot = int(tail_ids[r])
            kk = np.repeat(tail_key[slot], rep, axis=1)
            vv = np.repeat(tail_value[slot], rep, axis=1)
            s = np.einsum("hd,khd->hk", q_bf16[r], kk).astype(np.float32) * scale
            s[:, res_len:] = -np.inf
            blocks_s.append(s)
            blocks_v.append(vv)
            m = np.zeros(PAGE, dtype=bool)
            m[:res_len] = True
            blocks_res.append(m)
        if not blocks_s:
            continue
        scores = np.concatenate(blocks_s, axis=1)
        v = np.concatenate(blocks_v, axis=0)
        res = np.concatenate(blocks_res)
        o, lse = online_softmax_pv(scores, v, res, return_lse=True)
        out[r] = o
        lses[r] = lse
    if return_lse:
        return out, lses
    return out


def reference_decode(
    q_bf16,
    k_pages_bf16,
    v_pages_bf16,
    page_table,
    seqused_k,
    residual_page_ids,
    seqused_residual,
    softmax_scale,
):
    """Restatement of ``_torch_fp4_decode`` (test_fp4_decode_correctness.py:145-191):
    the oracle quantises Q/K/V itself with ``nvfp4_round_trip`` (ties to the
    lower magnitude) and restores the BF16 residual pages.

    q: [rows, Hq, D]; k/v pages: [pages, 128, Hkv, D] (one cache that holds both
    the full pages and, at ``residual_page_ids``, the BF16 residual page);
    page_table [rows, pages_per_row] lists every logical page INCLUDING the
    residual page as the row's last one.
    """
    q_dq = bf16_round(nvfp4_round_trip(q_bf16))
    k_dq = bf16_round(nvfp4_round_trip(k_pages_bf16))
    vt = np.ascontiguousarray(np.asarray(v_pages_bf16).transpose(0, 2, 3, 1))
    v_dq = bf16_round(nvfp4_round_trip(vt)).transpose(0, 3, 1, 2)
    seqused_k = np.asarray(seqused_k)
    seqused_residual = np.asarray(seqused_residual)
    fp4 = seqused_k - seqused_residual
    return attention_from_dequantized(
        q_bf16,
        q_dq,
        k_dq,
        v_dq,
        page_table,
        fp4,
        tail_key=k_pages_bf16,
        tail_value=v_pages_bf16,
        tail_ids=residual_page_ids,
        seqused_residual=seqused_residual,
        softmax_scale=softmax_scale,
    )


# --------------------------------------------------------------------------
# split-KV partials and the LSE merge
# (_fa4/block_info.py:46-54, split_k_combine.py:516-554)
# --------------------------------------------------------------------------

def split_page_range(n_pages: int, split: int, num_splits: int):
    per = -(-n_pages // num_splits) if n_pages > 0 else 0
    first = min(split * per, n_pages)
    last = min((split + 1) * per, n_pages)
    return first, last


def balanced_split_counts(seqused_fp4, target_pages: int):
    """Page pieces per row of the balanced split (an extension of this build, no counterpart in
    the reference, whose ``num_splits`` is one number per batch): ``ceil(pages / target_pages)``.
    Piece ``s`` of a row with count ``c`` owns ``split_page_range(pages, s, c)`` and never the
    tail: a row that holds a BF16 tail gets one more piece for the tail alone
    (:func:`balanced_pieces`).  A row with neither pages nor a tail keeps one empty piece."""
    pages = np.asarray(seqused_fp4, dtype=np.int64) // PAGE
    return (-(-pages // int(target_pages))).astype(np.int64)


def balanced_pieces(seqused_fp4, seqused_tail, target_pages: int):
    """Per row the pieces of the balanced split as ``[(first_page, last_page, owns_tail), ...]``:
    the tail piece (no pages) when the row holds a tail, then the page pieces."""
    counts = balanced_split_counts(seqused_fp4, target_pages)
    out = []
    for r, count in enumerate(counts):
        pages = int(seqused_fp4[r]) // PAGE
        tail = seqused_tail is not None and int(seqused_tail[r]) > 0
        row = [(0, 0, True)] if tail else []
        row += [split_page_range(pages, s, int(count)) + (False,) for s in range(int(count))]
        out.append(row or [(0, 0, False)])
    return out


def balanced_capacity(rows: int, max_pages: int, target_pages: int) -> int:
    """Upper bound on the number of pieces: every row at ``max_pages`` pages, with a tail."""
    return 2 * rows + rows * max_pages // target_pages


# --------------------------------------------------------------------------
# schedule of the persistent decode launch (no counterpart in the reference, whose persistent
# scheduler hands out whole tiles: _fa4/tile_scheduler.py:202-211).  Restated here so that the
# parity tests can run the attention oracle piece by piece and merge, which is what the
# reference's split path defines for a row cut into page ranges (_decode.py:982-1171).
# --------------------------------------------------------------------------

PERSISTENT_MIN_SHARE = 4


def persistent_tail_units(tail_len: int) -> int:
    """Cost of a BF16 tail in units of one NVFP4 page."""
    return 4 + (tail_len >> 3) if tail_len > 0 else 0


def persistent_pieces(seqused_fp4, seqused_tail, tail_ids, tail_pages: int, heads_kv: int,
                      max_pages: int, ctas: int):
    """Pieces of every (row, KV head) tile: ``{(row, kvh): [(first_page, last_page, owns_tail), ...]}``
    in the order they are merged.  A row costs ``max(1, pages + tail units)`` units, the rows lie
    end to end, and the CTAs form ``ctas // heads_kv`` groups of ``heads_kv``: group j of
    ``ce = min(groups, ceil(T / 4))`` owns units ``[j T // ce, (j + 1) T // ce)`` and its CTA h
    walks KV head h of them, so every KV head of a row is cut at the same places.  Unit 0 of a row
    stands for its tail, the units after the tail units for pages 0, 1, ...  A group whose share
    of a row holds neither the tail nor a page still contributes an (empty) piece."""
    rows = len(seqused_fp4)
    info = []
    for r in range(rows):
        fp4 = int(seqused_fp4[r])
        n = fp4 >> 7
        if fp4 < 0 or n > max_pages:
            n = 0 if fp4 < 0 else max_pages
        tl = 0
        if seqused_tail is not None and int(seqused_tail[r]) > 0:
            ln = min(int(seqused_tail[r]), PAGE)
            tid = int(tail_ids[r])
            if 0 <= tid < tail_pages:
                tl = ln
        info.append((n, tl, max(1, n + persistent_tail_units(tl))))
    total = sum(c for _, _, c in info)
    ce = min(ctas // heads_kv, -(-total // PERSISTENT_MIN_SHARE))
    pieces = {}
    u = 0
    for r, (n, tl, cost) in enumerate(info):
        tw = persistent_tail_units(tl)
        c_first = ((u + 1) * ce - 1) // total
        c_last = ((u + cost) * ce - 1) // total
        tile = []
        for c in range(c_first, c_last + 1):
            u0, u1 = c * total // ce, (c + 1) * total // ce
            lo, hi = max(u0, u) - u, min(u1, u + cost) - u
            first = min(max(lo, tw) - tw, n)
            last = min(max(hi, tw) - tw, n)
            tile.append((first, last, tl > 0 and lo == 0))
        for h in range(heads_kv):
            pieces[(r, h)] = tile
        u += cost
    return pieces


def attention_in_pieces(pieces, q_bf16, q_dq, k_dq_pages, v_dq_pages, page_table, seqused_fp4,
                        tail_key=None, tail_value=None, tail_ids=None, seqused_residual=None,
                        softmax_scale=None, tiles=None):
    """The attention oracle run piece by piece over ``pieces`` (see ``persistent_pieces``) and
    merged by LSE weight per tile.  ``tiles``: restrict to these (row, kvh) keys; other output
    rows stay zero."""
    rows, hq, d = q_dq.shape
    hkv = k_dq_pages.shape[2]
    g = hq // hkv
    out = np.zeros((rows, hq, d), dtype=np.float32)
    for (r, h), tile in pieces.items():
        if tiles is not None and (r, h) not in tiles:
            continue
        hs = slice(h * g, (h + 1) * g)
        parts, lses = [], []
        for first, last, owns_tail in tile:
            o, lse = attention_from_dequantized(
                q_bf16[r:r + 1, hs], q_dq[r:r + 1, hs], k_dq_pages[:, :, h:h + 1], v_dq_pages[:, :, h:h + 1],
                page_table[r:r + 1], seqused_fp4[r:r + 1],
                tail_key=None if tail_key is None else tail_key[:, :, h:h + 1],
                tail_value=None if tail_value is None else tail_value[:, :, h:h + 1],
                tail_ids=None if tail_ids is None else tail_ids[r:r + 1],
                seqused_residual=None if seqused_residual is None else seqused_residual[r:r + 1],
                softmax_scale=softmax_scale, page_range=(lambda n, a=first, b=last: (a, b)),
                owns_tail=owns_tail, return_lse=True)
            parts.append(o)
            lses.append(lse)
        out[r, hs] = lse_merge(np.stack(parts), np.stack(lses))[0]
    return out


def lse_merge(o_parts, lse_parts, return_lse: bool = False):
    """o_parts [S, rows, Hq, D] fp32 normalised, lse_parts [S, rows, Hq].

    ``lse = log sum_s exp(lse_s)``; ``O = sum_s exp(lse_s - lse) O_s``; a split
    whose LSE is -inf weighs 0; all -inf -> zeros.
    """
    o_parts = np.asarray(o_parts, dtype=np.float32)
    lse_parts = np.asarray(lse_parts, dtype=np.float32)
    m = lse_parts.max(axis=0)
    m_safe = np.where(np.isfinite(m), m, 0.0).astype(np.float32)
    with np.errstate(invalid="ignore"):
        w = np.exp(lse_parts - m_safe[None]).astype(np.float32)
    w = np.where(np.isfinite(lse_parts), w, 0.0).astype(np.float32)
    tot = w.sum(axis=0)
    with np.errstate(invalid="ignore", divide="ignore"):
        wn = np.where(tot > 0, w / tot, 0.0).astype(np.float32)
    o_safe = np.where(wn[..., None] > 0, o_parts, 0.0)
    out = (wn[..., None] * o_safe).sum(axis=0).astype(np.float32)
    if return_lse:
        with np.errstate(divide="ignore"):
            lse = np.where(tot > 0, m_safe + np.log(tot), -np.inf).astype(np.float32)
        return out, lse
    return out


# --------------------------------------------------------------------------
# slot control plane, written out the long way
# (tests/e2e/test_control.py:107-221 restates src/nvfp4_vllm/control.py:114-334)
# --------------------------------------------------------------------------

class SlotTable:
    """Serial restatement of the tail-slot control plane.

    A row is a request iff its length is positive and its first block is not the null block
    (0).  A row keeps the slot keyed on its first block; a new row takes the unclaimed slot
    seen longest ago (ties: lowest index).  Error flags accumulate in ``errors``.
    """

    FREE, NULL_BLOCK, INACTIVE = -1, 0, -1
    E_CONT_PREFILL, E_SLOT_LOST, E_STALE, E_NO_FREE, E_DUP, E_PROMO = 1, 2, 4, 8, 16, 32

    def __init__(self, num_slots: int):
        self.n = num_slots
        self.keys = [self.FREE] * num_slots
        self.last_seq = [-1] * num_slots
        self.last_seen = [-1] * num_slots
        self.step = 0
        self.errors = 0

    def prepare(self, block_table, seq_lens, query_lens):
        self.step += 1
        rows = len(seq_lens)
        key = [int(block_table[r][0]) for r in range(rows)]
        live = [seq_lens[r] > 0 and key[r] != self.NULL_BLOCK for r in range(rows)]
        slot_of = [self.INACTIVE] * rows
        taken = set()
        seen = set()
        for r in range(rows):
            if live[r]:
                if key[r] in seen:
                    self.errors |= self.E_DUP
                seen.add(key[r])
        for r in range(rows):
            if not live[r]:
                continue
            computed = seq_lens[r] - query_lens[r]
            if query_lens[r] > 1 and computed > 0:
                self.errors |= self.E_CONT_PREFILL
            for s in range(self.n):
                if self.keys[s] == key[r]:
                    slot_of[r] = s
                    taken.add(s)
                    if computed > 0 and self.last_seq[s] != computed:
                        self.errors |= self.E_STALE
                    break
        for r in range(rows):
            if not live[r] or slot_of[r] != self.INACTIVE:
                continue
            if seq_lens[r] - query_lens[r] > 0:
                self.errors |= self.E_SLOT_LOST
            free = [s for s in range(self.n) if s not in taken]
            if not free:
                self.errors |= self.E_NO_FREE
                continue
            victim = min(free, key=lambda s: (self.last_seen[s], s))
            slot_of[r] = victim
            taken.add(victim)
        written = set()
        for r, s in enumerate(slot_of):
            if s == self.INACTIVE or s in written:
                continue
            written.add(s)
            self.keys[s], self.last_seq[s], self.last_seen[s] = key[r], seq_lens[r], self.step
        fp4 = [((seq_lens[r] - 1) // PAGE) * PAGE if live[r] else 0 for r in range(rows)]
        residual = [seq_lens[r] - fp4[r] if live[r] else 0 for r in range(rows)]
        token_to_slot = [slot_of[r] if live[r] else 0 for r in range(rows) for _ in range(query_lens[r])]
        sources, pages = [0] * self.n, [-1] * self.n
        for r in range(rows):
            if not live[r]:
                continue
            sources[r] = slot_of[r] * PAGE
            if seq_lens[r] % PAGE:
                continue
            column = seq_lens[r] // PAGE - 1
            if column >= len(block_table[r]):
                self.errors |= self.E_PROMO
                continue
            pages[r] = int(block_table[r][column])
        return dict(row_to_slot=slot_of, token_to_slot=token_to_slot, seqused_fp4=fp4,
                    seqused_residual=residual, promotion_source_tokens=sources,
                    promotion_pages=pages, error_code=self.errors)


def work_table(query_start_loc, seqused_fp4, row_to_slot, block_table, columns):
    """Page work table of a step (write.py:30-76)."""
    src, dst = [], []
    for r in range(len(seqused_fp4)):
        start, end = query_start_loc[r], query_start_loc[r + 1]
        writes = (end - start > 1) and row_to_slot[r] >= 0
        for c in range(columns):
            src.append(start + c * PAGE)
            dst.append(int(block_table[r][c]) if writes and c < seqused_fp4[r] // PAGE else -1)
    return src, dst
