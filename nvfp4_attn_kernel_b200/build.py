"""In-tree build of ``libnvfp4_b200.so`` with nvcc for sm_100a.

The shared library is written next to this file so that it travels with the
source tree.  ``python -m nvfp4_attn_kernel_b200.build`` rebuilds it.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_NAME = "libnvfp4_b200.so"
LIB_PATH = os.path.join(HERE, LIB_NAME)

SOURCES = ["capi.cu", "quantize.cu", "decode_generic.cu", "decode_sm100.cu", "decode_persistent.cu", "merge.cu",
           "decode_static_ws.cu", "control.cu", "key_sum.cu"]
# measurement aid of bench.py, a library of its own so that the product's ABI carries no test code
BENCH_AID_SOURCE = "bench_read_floor.cu"
BENCH_AID_PATH = os.path.join(HERE, "libnvfp4_bench_read_floor.so")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _stale() -> bool:
    if not os.path.exists(LIB_PATH) or not os.path.exists(BENCH_AID_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "nvfp4_b200.h"))
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source into the shared library; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", LIB_PATH + ".tmp"] + [os.path.join(CSRC, s) for s in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode:
        raise RuntimeError(f"nvcc failed with exit code {proc.returncode}")
    aid = subprocess.run([_nvcc(), *NVCC_FLAGS, "-o", BENCH_AID_PATH + ".tmp", os.path.join(CSRC, BENCH_AID_SOURCE)],
                         capture_output=True, text=True)
    if aid.returncode:
        sys.stderr.write(aid.stdout + aid.stderr)
        raise RuntimeError(f"nvcc failed with exit code {aid.returncode} on {BENCH_AID_SOURCE}")
    os.replace(BENCH_AID_PATH + ".tmp", BENCH_AID_PATH)
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
