"""The reference project's own quantiser test files, run unmodified against this library.

``make -C oracle ref`` copies ``tests/kernel/test_quantize_kv.py`` and ``test_quantize_query.py``
of a reference checkout into the git-ignored ``oracle/_ref/``.  Each file runs in a child process
in which :func:`nvfp4_attn_kernel_b200.install_aliases` has made ``import nvfp4_decode_kernel``
resolve to this package, so every assertion of those files is made about this library's bytes.
``test_quantize_query.py`` compares with FlashInfer through the reference's own test aid
``_quantize_flashinfer.py``, which is loaded from ``oracle/_ref`` (it is not part of the product).
"""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")

DRIVER = r"""
import importlib.util, sys
sys.path.insert(0, {root!r})
import nvfp4_attn_kernel_b200 as pkg
pkg.install_aliases()
import nvfp4_decode_kernel
assert nvfp4_decode_kernel.__file__.startswith({root!r}) and "_ref" not in nvfp4_decode_kernel.__file__
aid = {aid!r}
if aid:
    spec = importlib.util.spec_from_file_location("nvfp4_decode_kernel._quantize_flashinfer", aid)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
import pytest
sys.exit(pytest.main(["-q", "-x", "-p", "no:cacheprovider", "-rs", {test!r}]))
"""


def _run(test_file: str, aid: str = "") -> str:
    path = os.path.join(REF, "tests", "kernel", test_file)
    if not os.path.exists(path):
        pytest.skip("oracle/_ref is not populated (make -C oracle ref, next to a reference checkout)")
    code = DRIVER.format(root=ROOT, aid=aid, test=path)
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600,
                          cwd=os.path.join(REF, "tests"))
    tail = (proc.stdout + proc.stderr)[-3000:]
    assert proc.returncode == 0, tail
    assert " passed" in proc.stdout and "skipped" not in proc.stdout.splitlines()[-1], tail
    return proc.stdout


def test_reference_quantize_kv_tests_pass_on_this_library(cuda_device):
    _run("test_quantize_kv.py")


def test_reference_quantize_query_tests_pass_on_this_library(cuda_device):
    pytest.importorskip("flashinfer")
    aid = os.path.join(REF, "src", "nvfp4_decode_kernel", "_quantize_flashinfer.py")
    _run("test_quantize_query.py", aid)
