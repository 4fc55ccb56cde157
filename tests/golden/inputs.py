"""Seeded synthetic inputs shared by the golden-vector generator and the tests.

Everything comes from ``numpy.random.default_rng`` (PCG64), whose stream is the
same on every machine, so a golden file only needs to store OUTPUTS.
BF16 tensors are float32 arrays holding bf16-exact values.
"""

from __future__ import annotations

import numpy as np

PAGE = 128
D = 128


def bf16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    bias = np.uint64(0x7FFF) + ((bits >> np.uint64(16)) & np.uint64(1))
    out = (((bits + bias) >> np.uint64(16)) << np.uint64(16)).astype(np.uint32)
    return out.view(np.float32).reshape(x.shape)


def value_kat(seed: int = 7):
    """Inputs for the NVFP4 round-trip known-answer test: random magnitudes over
    several decades, exact E2M1 ties, zeros, a zero group, tiny groups."""
    rng = np.random.default_rng(seed)
    a = bf16(rng.standard_normal((64, 128)).astype(np.float32) * 3.0)
    b = bf16(rng.standard_normal((32, 128)).astype(np.float32) * 0.01)
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0], dtype=np.float32)
    c = np.zeros((16, 128), dtype=np.float32)
    for i in range(16):
        for g in range(8):
            grp = rng.choice(ties, size=16) * rng.choice([-1.0, 1.0], size=16)
            grp[0] = 6.0  # amax 6 -> scale exactly 1 -> every element a tie
            c[i, g * 16:(g + 1) * 16] = grp * (2.0 ** (g - 4))
    d = np.zeros((4, 128), dtype=np.float32)
    d[1, :16] = 1e-4
    d[2, 5] = 448.0 * 6.0
    d[3] = bf16(rng.standard_normal(128).astype(np.float32) * 1e-3)
    return np.concatenate([a, b, bf16(c), bf16(d)], axis=0)


def attention_case(seed, rows, heads_q, heads_kv, seq_lens, scale=1.0, k_offset=0.0,
                   shuffle=True):
    """One paged decode problem in the layout the reference oracle consumes:
    a BF16 page cache that holds every logical page (the last page of each row
    doubles as the BF16 residual page)."""
    rng = np.random.default_rng(seed)
    seq_lens = np.asarray(seq_lens, dtype=np.int64)
    pages_per_row = int(max(1, np.max((seq_lens + PAGE - 1) // PAGE)))
    num_pages = rows * pages_per_row
    q = bf16(rng.standard_normal((rows, heads_q, D)).astype(np.float32) * scale)
    k = rng.standard_normal((num_pages, PAGE, heads_kv, D)).astype(np.float32) * scale
    if k_offset:
        off = rng.standard_normal((heads_kv, D)).astype(np.float32) * k_offset
        k = k + off[None, None]
    k = bf16(k)
    v = bf16(rng.standard_normal((num_pages, PAGE, heads_kv, D)).astype(np.float32) * scale)
    ids = rng.permutation(num_pages) if shuffle else np.arange(num_pages)
    page_table = ids.reshape(rows, pages_per_row).astype(np.int32)
    fp4 = np.where(seq_lens > 0, ((seq_lens - 1) // PAGE) * PAGE, 0)
    residual = seq_lens - fp4
    cols = np.minimum(fp4 // PAGE, pages_per_row - 1)
    residual_ids = page_table[np.arange(rows), cols].astype(np.int32)
    return dict(
        q=q, k_pages=k, v_pages=v, page_table=page_table,
        seqused_k=seq_lens.astype(np.int32),
        seqused_fp4=fp4.astype(np.int32),
        seqused_residual=residual.astype(np.int32),
        residual_page_ids=residual_ids,
        softmax_scale=float(D ** -0.5),
    )


def config1(seed: int = 0):
    """The CPU-runnable headline case: one Llama-3.1-8B-shaped layer, batch 1,
    context 1000 (7 full pages + 104-token tail), Q/K/V ~ N(0,1), per-channel K
    offset ~ N(0, sigma=2) removed by the per-channel mean (BF16 subtract)."""
    rng = np.random.default_rng(seed)
    ctx, hq, hkv = 1000, 32, 8
    q = bf16(rng.standard_normal((1, hq, D)).astype(np.float32))
    off = rng.standard_normal((hkv, D)).astype(np.float32) * 2.0
    k_raw = bf16(rng.standard_normal((ctx, hkv, D)).astype(np.float32) + off[None])
    v = bf16(rng.standard_normal((ctx, hkv, D)).astype(np.float32))
    mu = bf16(k_raw.astype(np.float64).mean(axis=0).astype(np.float32))
    k = bf16(k_raw - mu[None])
    pages = 8
    kp = np.zeros((pages * PAGE, hkv, D), dtype=np.float32)
    vp = np.zeros((pages * PAGE, hkv, D), dtype=np.float32)
    table = rng.permutation(pages).astype(np.int32)
    kp = kp.reshape(pages, PAGE, hkv, D)
    vp = vp.reshape(pages, PAGE, hkv, D)
    for logical in range(pages):
        lo, hi = logical * PAGE, min((logical + 1) * PAGE, ctx)
        kp[table[logical], : hi - lo] = k[lo:hi]
        vp[table[logical], : hi - lo] = v[lo:hi]
    return dict(
        q=q, k_raw=k_raw, key_shift=mu, k_pages=kp, v_pages=vp,
        page_table=table.reshape(1, pages),
        seqused_k=np.array([ctx], dtype=np.int32),
        seqused_fp4=np.array([896], dtype=np.int32),
        seqused_residual=np.array([104], dtype=np.int32),
        residual_page_ids=table[7:8].copy(),
        softmax_scale=float(D ** -0.5),
    )


SMALL_CASES = {
    # name: (seed, rows, Hq, Hkv, seq_lens, scale, k_offset)
    "boundaries": (11, 7, 8, 2, (1, 127, 128, 129, 255, 256, 257), 1.0, 0.0),
    "gqa4_short": (12, 2, 8, 2, (300, 512), 1.0, 0.0),
    "scaled03": (13, 3, 8, 2, (200, 256, 640), 0.3, 0.0),
    "mha": (14, 1, 4, 4, (256,), 1.0, 0.0),
    "mqa": (15, 1, 16, 1, (384,), 1.0, 0.0),
}
