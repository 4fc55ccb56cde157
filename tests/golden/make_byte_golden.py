"""Generates ``tests/golden/quant_bytes.npz``: quantised bytes produced on a B200 by code this
repository did not write, for the seeded inputs of ``byte_golden_inputs`` below.

Two independent producers, both run through the reference project's own call sites:

* FlashInfer ``fp4_quantize`` (global scale 1, swizzled scale layout), called exactly as the
  reference's test aid ``_quantize_flashinfer.flashinfer_quantize_query`` calls it
  (``src/nvfp4_decode_kernel/_quantize_flashinfer.py:23-86``), on the row counts of
  ``tests/kernel/test_quantize_query.py:40-59`` (1, 7, 8; inputs ``randn * 3``);
* the reference's own CuTeDSL quantiser kernels (``quantize_query``, ``quantize_key_pages``,
  ``quantize_value_pages``, ``quantize_*_tokens_into``) on the windows of
  ``tests/kernel/test_quantize_kv.py:126-127`` (starts 0, 37, 1000, 128, 511 -> pages 4, 1, 0, 3, 2).

Needs a GPU of compute capability 10.x, ``flashinfer`` and ``nvidia-cutlass-dsl``, and the
reference's operator package under ``oracle/_ref/src`` (``make -C oracle ref``).  A producer
that cannot run leaves its exception text in the file instead of bytes.

    python tests/golden/make_byte_golden.py [output.npz]

The inputs come from numpy's PCG64 stream, so the file stores outputs only.  Full byte arrays
are stored for 2 KV heads; for 8 KV heads (the reference test's shape) SHA-256 digests.
"""

from __future__ import annotations

import hashlib
import os
import sys
import traceback

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, HERE)

import inputs  # noqa: E402

Q_ROWS = (1, 7, 8)
Q_HEADS = 32
STARTS = (0, 37, 1000, 128, 511)
DESTINATIONS = (4, 1, 0, 3, 2)
TOKENS = 1152            # covers the window that starts at token 1000
KV_HEADS_FULL = 2        # full bytes stored
KV_HEADS_DIGEST = 8      # digests stored


def query_input(rows: int) -> np.ndarray:
    rng = np.random.default_rng(0x5200 + rows)
    return inputs.bf16(rng.standard_normal((rows, Q_HEADS, 128)).astype(np.float32) * 3.0)


def token_input(heads: int) -> np.ndarray:
    rng = np.random.default_rng(0x4B56 + heads)
    return inputs.bf16(rng.standard_normal((TOKENS, heads, 128)).astype(np.float32) * 0.3)


def windows(tokens: np.ndarray) -> np.ndarray:
    return np.stack([tokens[s:s + 128] for s in STARTS])


def digest(a: np.ndarray) -> np.ndarray:
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), dtype=np.uint8).copy()


def _u8(t):
    import torch

    if t.dtype in (torch.float8_e4m3fn, torch.float4_e2m1fn_x2, torch.int8):
        t = t.view(torch.uint8)
    return t.contiguous().cpu().numpy()


def _bf16(x, device):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(device).to(torch.bfloat16)


def flashinfer_half(out: dict, device) -> None:
    from nvfp4_decode_kernel._quantize_flashinfer import flashinfer_quantize_query

    import flashinfer

    out["flashinfer_version"] = np.array(flashinfer.__version__)
    for rows in Q_ROWS:
        fp4, scales = flashinfer_quantize_query(_bf16(query_input(rows), device))
        out[f"fi_q{rows}_fp4"] = _u8(fp4[:, :1])                    # [rows, 1, heads, 64]
        out[f"fi_q{rows}_sf"] = _u8(scales)                          # (32, 4, 1, 4, 2, heads, rows)


def reference_half(out: dict, device) -> None:
    import torch
    from nvfp4_decode_kernel._quantize import quantize_query
    from nvfp4_decode_kernel.quantize_kv_kernel import (quantize_key_pages, quantize_key_tokens_into,
                                                       quantize_value_pages, quantize_value_tokens_into)

    import cutlass

    out["cutlass_dsl_version"] = np.array(getattr(cutlass, "__version__", "?"))
    for rows in Q_ROWS:
        fp4, scales = quantize_query(_bf16(query_input(rows), device))
        out[f"ref_q{rows}_fp4"] = _u8(fp4)
        out[f"ref_q{rows}_sf"] = _u8(scales)
    starts = torch.tensor(STARTS, dtype=torch.int32, device=device)
    dests = torch.tensor(DESTINATIONS, dtype=torch.int32, device=device)
    for heads in (KV_HEADS_FULL, KV_HEADS_DIGEST):
        tok_np = token_input(heads)
        tok = _bf16(tok_np, device)
        win = _bf16(windows(tok_np), device)
        store = (lambda key, a: out.__setitem__(key, a)) if heads == KV_HEADS_FULL else (
            lambda key, a: out.__setitem__(key + "_sha256", digest(a)))
        kp, ks = quantize_key_pages(win)
        vp, vs = quantize_value_pages(win)
        store(f"ref_k{heads}_packed", _u8(kp))                       # [5, 128, heads, 64]
        store(f"ref_k{heads}_sf", _u8(ks))                           # [5, 32, 4, 1, 4, 2, heads]
        store(f"ref_v{heads}_packed", _u8(vp))                       # [5, heads, 128, 64]
        store(f"ref_v{heads}_sf", _u8(vs))
        # the indexed quantisers into pages 100 KiB apart, as the reference's test lays them out
        pitch = 100 * 1024
        for which, fn, shape, strides in (
            ("k", quantize_key_tokens_into, (128, heads, 64), (heads * 64, 64, 1)),
            ("v", quantize_value_tokens_into, (heads, 128, 64), (128 * 64, 64, 1)),
        ):
            pbuf = torch.full((len(STARTS), pitch), 0xA5, dtype=torch.uint8, device=device)
            sbuf = torch.full((len(STARTS), pitch), 0xA5, dtype=torch.uint8, device=device)
            packed = pbuf.as_strided((len(STARTS),) + shape, (pitch,) + strides, 0)
            scales = sbuf.as_strided((len(STARTS), 32, 4, 1, 4, 2, heads), (pitch, 16, 4, 1024, 1, 512, 1024), 0)
            fn(tok, packed, scales, starts, dests)
            torch.cuda.synchronize()
            store(f"ref_{which}{heads}_into_packed", _u8(packed))    # page order = destination order
            store(f"ref_{which}{heads}_into_sf", _u8(scales))
            used_p, used_s = int(np.prod(shape)), heads * 1024
            out[f"ref_{which}{heads}_into_canaries_intact"] = np.array(
                bool((pbuf[:, used_p:] == 0xA5).all()) and bool((sbuf[:, used_s:] == 0xA5).all()))


def main() -> None:
    import torch

    target = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "quant_bytes.npz")
    ref_src = os.path.join(ROOT, "oracle", "_ref", "src")
    if not os.path.isdir(os.path.join(ref_src, "nvfp4_decode_kernel")):
        raise SystemExit("oracle/_ref/src is missing: run `make -C oracle ref` next to a reference checkout")
    sys.path.insert(0, ref_src)
    if not torch.cuda.is_available() or torch.cuda.get_device_capability()[0] != 10:
        raise SystemExit("needs a GPU of compute capability 10.x")
    device = torch.device("cuda", 0)
    out: dict = {"gpu": np.array(torch.cuda.get_device_name(0)), "torch": np.array(torch.__version__)}
    for name, half in (("flashinfer", flashinfer_half), ("reference", reference_half)):
        try:
            half(out, device)
            out[f"{name}_error"] = np.array("")
        except Exception:   # the text is the record of why that producer is absent
            out[f"{name}_error"] = np.array(traceback.format_exc()[-1500:])
            print(f"{name} half failed:\n{traceback.format_exc()}", file=sys.stderr)
    # the attempt to import the reference's decode kernel on this machine, for the record
    try:
        import nvfp4_decode_kernel._decode  # noqa: F401

        out["reference_decode_import"] = np.array("imports")
    except Exception as e:
        out["reference_decode_import"] = np.array(f"{type(e).__name__}: {e}"[:500])
    np.savez_compressed(target, **out)
    print(f"wrote {target}: {sorted(out)}")
    for key in ("flashinfer_error", "reference_error", "reference_decode_import"):
        print(key, "=", str(out[key])[-300:] or "(none)")


if __name__ == "__main__":
    main()
