"""Generate the golden vectors in this folder from the REFERENCE's own torch code.

Run in a container that has the reference checkout (read-only) mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports ``src/nvfp4_decode_kernel/reference.py`` and the attention oracle
that lives in ``tests/kernel/test_fp4_decode_correctness.py`` (its
``flash_attn.cute`` import is stubbed; nothing GPU-side is executed), feeds them
the seeded inputs of ``inputs.py`` and stores the OUTPUTS as small ``.npz``
files.  The test-suite then checks the numpy oracle against these files on any
machine, without the reference present.
"""

from __future__ import annotations

import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import inputs  # noqa: E402


def load_reference(root: str):
    sys.path.insert(0, os.path.join(root, "src"))
    fa = types.ModuleType("flash_attn")
    fac = types.ModuleType("flash_attn.cute")
    fac.flash_attn_func = None
    fa.cute = fac
    sys.modules["flash_attn"] = fa
    sys.modules["flash_attn.cute"] = fac
    from nvfp4_decode_kernel import reference as ref_values

    path = os.path.join(root, "tests", "kernel", "test_fp4_decode_correctness.py")
    spec = importlib.util.spec_from_file_location("ref_decode_tests", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ref_decode_tests"] = mod
    try:
        spec.loader.exec_module(mod)
    except Exception as error:  # pragma: no cover - depends on the container
        raise SystemExit(f"could not import the reference attention oracle: {error}")
    return ref_values, mod


def bf(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(torch.bfloat16)


def run_attention(mod, case):
    out = mod._torch_fp4_decode(
        bf(case["q"]).unsqueeze(1),
        bf(case["k_pages"]),
        bf(case["v_pages"]),
        torch.from_numpy(case["page_table"]),
        torch.from_numpy(case["seqused_k"]),
        torch.from_numpy(case["residual_page_ids"]),
        torch.from_numpy(case["seqused_residual"]),
        case["softmax_scale"],
    )
    return out[:, 0].float().numpy()


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <checkout of the reference project>")
    root = sys.argv[1]
    ref_values, mod = load_reference(root)
    torch.set_num_threads(os.cpu_count() or 1)

    x = inputs.value_kat()
    xt = torch.from_numpy(x)
    np.savez_compressed(
        os.path.join(HERE, "values_kat.npz"),
        round_trip=ref_values.nvfp4_round_trip(xt).numpy(),
        round_e2m1=ref_values.round_e2m1(xt).numpy(),
        # the V direction: groups along tokens of a [tok, d] tile
        round_trip_t=ref_values.nvfp4_round_trip(xt[:64].t().contiguous()).numpy(),
    )

    outs = {}
    for name, (seed, rows, hq, hkv, lens, scale, koff) in inputs.SMALL_CASES.items():
        case = inputs.attention_case(seed, rows, hq, hkv, lens, scale, koff)
        outs[name] = run_attention(mod, case)
    c1 = inputs.config1(0)
    outs["config1"] = run_attention(mod, c1)
    np.savez_compressed(os.path.join(HERE, "attention.npz"), **outs)

    # online-softmax building block on raw scores (exercises P quantisation)
    rng = np.random.default_rng(21)
    scores = rng.standard_normal((1, 4, 1, 384)).astype(np.float32) * 2.0
    scores[..., 300:] = -np.inf
    v = inputs.bf16(rng.standard_normal((1, 384, 4, 128)).astype(np.float32))
    res = np.zeros((1, 1, 1, 384), dtype=bool)
    res[..., 256:300] = True
    o = mod._online_softmax_pv(
        torch.from_numpy(scores), torch.from_numpy(v), torch.from_numpy(res)
    )
    np.savez_compressed(
        os.path.join(HERE, "online_softmax.npz"), out=o[0, 0].numpy()
    )
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
