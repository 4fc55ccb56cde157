"""Installed as the top-level package ``nvfp4_vllm`` (the name the reference project's callers,
its tests and vLLM's plugin entry point import).  Importing it hands the name over to
``nvfp4_attn_kernel_b200.nvfp4_vllm``: after this module has run, ``sys.modules["nvfp4_vllm"]`` is that
package itself and every ``nvfp4_vllm.<submodule>`` resolves to the one module object of the real
submodule, so nothing is executed twice under two names."""

import nvfp4_attn_kernel_b200 as _home

_home.install_aliases()
