"""The backend inside a live vLLM engine (vLLM 0.22, in-process engine core, dummy weights).

Each variant runs in a child process (``live_vllm_engine.py``).  Checked: the engine comes up
on the ``CUSTOM`` backend with the NVFP4 cache, serves six prompts of 5..300 tokens for 200
greedy tokens each (every request crosses a page boundary, so tails are flushed), the slot
control plane reports no error, and the token streams are IDENTICAL between the fused launch
structure (query quantised in the decode kernel, tail copy in the decode launch) and the
reference's separate launches, and between eager mode and CUDA graphs.  Against vLLM's own
FlashAttention backend with a BF16 cache the first token of every request (prefill attention, no
cache involved) must agree.
"""

import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


_RESULTS: dict = {}


def run_engine(*flags):
    if flags in _RESULTS:      # an engine start takes most of a minute: each variant runs once
        return _RESULTS[flags]
    try:
        import vllm  # noqa: F401
    except ImportError:
        pytest.skip("vLLM is not installed")
    proc = subprocess.run([sys.executable, os.path.join(HERE, "live_vllm_engine.py"), *flags],
                          capture_output=True, text=True, timeout=600)
    lines = [line for line in proc.stdout.splitlines() if line.startswith("RESULT ")]
    assert proc.returncode == 0 and lines, (proc.stdout[-2000:], proc.stderr[-4000:])
    _RESULTS[flags] = json.loads(lines[-1][len("RESULT "):])
    return _RESULTS[flags]


def test_live_engine_serves_and_fused_equals_separate_launches(cuda_device):
    fused = run_engine()
    assert [len(t) for t in fused["tokens"]] == [200] * 6
    assert all(word == 0 for words in fused["control_plane_errors"] for word in words)
    assert fused["control_plane_errors"] and fused["control_plane_errors"][0]
    separate = run_engine("--separate")
    assert separate["tokens"] == fused["tokens"]
    assert all(word == 0 for words in separate["control_plane_errors"] for word in words)


def test_live_engine_first_tokens_agree_with_the_stock_backend(cuda_device):
    ours = run_engine()
    stock = run_engine("--stock")
    assert [t[0] for t in ours["tokens"]] == [t[0] for t in stock["tokens"]]


def test_live_engine_cuda_graphs_equal_eager_mode(cuda_device):
    """With CUDA graphs vLLM captures padded decode batches first (the slot table must start
    empty afterwards, padding rows must own no slot) and replays them while serving: the tokens
    must be those of eager mode and the control plane must report nothing."""
    eager = run_engine()
    graphs = run_engine("--graphs")
    assert graphs["tokens"] == eager["tokens"]
    assert all(word == 0 for words in graphs["control_plane_errors"] for word in words)


def test_live_engine_key_shift_measurement_and_switch(cuda_device):
    """The key shift is measured through the worker extension while the engine runs (fp64 sum of
    K over a 700-token prefill, per layer), the engine serves with it, and with the shift switched
    off again it produces exactly the tokens of an engine that never had one."""
    plain = run_engine()
    shifted = run_engine("--shift")
    report = shifted["report"]
    assert report["tokens"] == 700 and report["shape"] == [2, 2, 128] and report["mean_abs"] > 0
    assert shifted["active"] == [True] and shifted["switched_off"] is True
    assert [len(t) for t in shifted["tokens_shifted"]] == [200] * 6
    assert [t[0] for t in shifted["tokens_shifted"]] == [t[0] for t in plain["tokens"]]
    assert shifted["tokens"] == plain["tokens"]
    assert all(word == 0 for words in shifted["control_plane_errors"] for word in words)
