"""The install description: the package list, the stand-in packages that carry the reference
project's top-level names, and vLLM's plugin entry point (the reference publishes
``nvfp4_vllm = "nvfp4_vllm:register"`` under ``vllm.general_plugins``, pyproject.toml:20-21)."""

import os
import subprocess
import sys
import tomllib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _project():
    with open(os.path.join(ROOT, "pyproject.toml"), "rb") as f:
        return tomllib.load(f)


def test_entry_point_and_package_layout():
    cfg = _project()
    assert cfg["project"]["entry-points"]["vllm.general_plugins"] == {"nvfp4_vllm": "nvfp4_vllm:register"}
    tool = cfg["tool"]["setuptools"]
    for name in tool["packages"]:
        folder = tool.get("package-dir", {}).get(name, name.replace(".", "/"))
        assert os.path.isfile(os.path.join(ROOT, folder, "__init__.py")), name
    assert {"nvfp4_decode_kernel", "nvfp4_vllm"} <= set(tool["packages"])
    # every sub-package with Python sources is listed (a forgotten one would be left out of a wheel)
    home = os.path.join(ROOT, "nvfp4_attn_kernel_b200")
    for entry in sorted(os.listdir(home)):
        if os.path.isfile(os.path.join(home, entry, "__init__.py")):
            assert f"nvfp4_attn_kernel_b200.{entry}" in tool["packages"], entry


def test_installed_names_resolve_to_the_one_package():
    """What an installed tree looks like to the interpreter: the package and the two stand-ins
    side by side on the path, nothing else.  The entry point's target resolves, and the
    reference's import lines reach the real modules (one module object each)."""
    cfg = _project()["tool"]["setuptools"]["package-dir"]
    target = _project()["project"]["entry-points"]["vllm.general_plugins"]["nvfp4_vllm"]
    module, _, attr = target.partition(":")
    code = f"""
import importlib, sys
plugin = getattr(importlib.import_module({module!r}), {attr!r})
assert callable(plugin)
import nvfp4_attn_kernel_b200.nvfp4_vllm as real_vllm
import nvfp4_vllm, nvfp4_vllm.runtime, nvfp4_vllm.metadata
assert nvfp4_vllm is real_vllm and plugin is real_vllm.register
assert nvfp4_vllm.runtime is sys.modules["nvfp4_attn_kernel_b200.nvfp4_vllm.runtime"]
from nvfp4_decode_kernel import fp4_decode, quantize_kv_kernel
import nvfp4_attn_kernel_b200.nvfp4_decode_kernel as real_op
assert fp4_decode is real_op.fp4_decode
assert quantize_kv_kernel is sys.modules["nvfp4_attn_kernel_b200.nvfp4_decode_kernel.quantize_kv_kernel"]
from nvfp4_decode_kernel._quantize import quantize_query
print("ok")
"""
    standins = {os.path.dirname(os.path.join(ROOT, folder)) for folder in cfg.values()}
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT, *sorted(standins)]))
    done = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, cwd="/",
                          timeout=300)
    assert done.returncode == 0 and done.stdout.strip().endswith("ok"), done.stderr[-2000:]
