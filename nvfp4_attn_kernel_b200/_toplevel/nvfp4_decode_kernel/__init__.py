"""Installed as the top-level package ``nvfp4_decode_kernel`` (the name the reference project's callers,
its tests and vLLM's plugin entry point import).  Importing it hands the name over to
``nvfp4_attn_kernel_b200.nvfp4_decode_kernel``: after this module has run, ``sys.modules["nvfp4_decode_kernel"]`` is that
package itself and every ``nvfp4_decode_kernel.<submodule>`` resolves to the one module object of the real
submodule, so nothing is executed twice under two names."""

import nvfp4_attn_kernel_b200 as _home

_home.install_aliases()
