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
import importlib.abc
import importlib.util
import sys

__version__ = "0.1.0"

_ALIASES = ("nvfp4_decode_kernel", "nvfp4_vllm")


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """Resolves ``nvfp4_vllm.x`` to the one module object of ``<this package>.nvfp4_vllm.x`` so
    that a submodule is never executed twice under two names."""

    def find_spec(self, fullname, path=None, target=None):
        if fullname.partition(".")[0] not in _ALIASES:
            return None
        return importlib.util.spec_from_loader(fullname, self)

    def create_module(self, spec):
        module = importlib.import_module(f"{__name__}.{spec.name}")
        self._real_spec = module.__spec__   # the import machinery is about to overwrite it
        return module

    def exec_module(self, module):
        # already executed under its real name; keep the spec its relative imports rely on
        module.__spec__ = self._real_spec


def install_aliases() -> None:
    """Make ``import nvfp4_decode_kernel`` / ``import nvfp4_vllm`` (and their submodules)
    resolve here."""
    if not any(isinstance(finder, _AliasFinder) for finder in sys.meta_path):
        sys.meta_path.insert(0, _AliasFinder())
    for name in _ALIASES:
        # set, not imported: when this runs from the installed stand-in package of the same
        # name, that stand-in is in sys.modules already and must be replaced by the real one
        sys.modules[name] = importlib.import_module(f"{__name__}.{name}")
