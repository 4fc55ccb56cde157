"""B200-native (sm_100a) paged NVFP4/BF16 hybrid decode attention.

The device code lives in ``csrc/`` and is reached through the C ABI declared in
``include/nvfp4_b200.h`` (``libnvfp4_b200.so``, loaded with ctypes by
:mod:`nvfp4_attn_kernel_b200._lib`).  Two sub-packages mirror the operator and
vLLM-backend surface of the reference project so that existing callers keep
their imports:

* ``nvfp4_attn_kernel_b200.nvfp4_decode_kernel`` - ``fp4_decode`` and the quantisers
* ``nvfp4_attn_kernel_b200.nvfp4_vllm``          - the vLLM v1 ``CUSTOM`` attention backend

:func:`install_aliases` registers them under the reference's top-level module
names (``nvfp4_decode_kernel``, ``nvfp4_vllm``).
"""

from __future__ import annotations

import importlib
import sys

__version__ = "0.1.0"


def install_aliases() -> None:
    """Make ``import nvfp4_decode_kernel`` / ``import nvfp4_vllm`` resolve here."""
    for name in ("nvfp4_decode_kernel", "nvfp4_vllm"):
        if name not in sys.modules:
            sys.modules[name] = importlib.import_module(f"{__name__}.{name}")
