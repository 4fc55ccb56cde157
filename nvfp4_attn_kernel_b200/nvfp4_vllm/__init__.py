"""vLLM v1 out-of-tree attention backend over the NVFP4 KV cache (drop-in for ``nvfp4_vllm``).

``register`` is the ``vllm.general_plugins`` entry point; the engine helpers are imported on
first use so that importing this package does not import vLLM.
"""

from __future__ import annotations


def register() -> None:
    """Point vLLM's ``CUSTOM`` attention backend at :class:`backend.NVFP4Backend`."""
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend

    register_backend(
        AttentionBackendEnum.CUSTOM,
        f"{__name__}.backend.NVFP4Backend",
    )


def __getattr__(name: str):
    if name == "build_llm":
        from .engine import build_llm

        return build_llm
    if name in ("calibrate_key_shift", "set_key_shift_enabled"):
        from . import calibrate

        return getattr(calibrate, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = ["register", "build_llm", "calibrate_key_shift", "set_key_shift_enabled"]
