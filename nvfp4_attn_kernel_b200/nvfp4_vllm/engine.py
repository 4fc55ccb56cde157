"""``build_llm``: a vLLM ``LLM`` on the NVFP4 cache with the key shift in force.

Counterpart of the reference project's ``src/nvfp4_vllm/engine.py:31-113``: binds the five engine
arguments the cache cannot work without (contradicting one raises), defaults ``max_num_seqs`` to
the slot count and ``max_num_batched_tokens`` to the window, installs the worker extension, and
resolves ``key_shift`` ("auto" = measure at start-up, a path = load a sidecar, None = no shift).
"""

from __future__ import annotations

import os
from typing import Any

PAGE_SIZE = 128
MAX_SLOTS = 32
KEY_SHIFT_ENV = "NVFP4_KEY_SHIFT"

REQUIRED_ENGINE_KWARGS: dict[str, Any] = {
    "kv_cache_dtype": "nvfp4",
    "attention_config": {"backend": "CUSTOM"},
    "block_size": PAGE_SIZE,
    "enable_prefix_caching": False,
    "enable_chunked_prefill": False,
}


def build_llm(model: str, *, key_shift: Any = "auto", **kwargs: Any):
    from vllm import LLM

    from . import register
    from .calibrate import WORKER_EXTENSION_CLS, calibrate_key_shift

    # The plugin entry point does this in every vLLM process of an installed package; doing it
    # here as well covers an in-process engine core of a source checkout.
    register()

    clash = {name: kwargs[name] for name, need in REQUIRED_ENGINE_KWARGS.items()
             if name in kwargs and kwargs[name] != need}
    if clash:
        wanted = {name: REQUIRED_ENGINE_KWARGS[name] for name in clash}
        raise ValueError(
            f"this backend requires {wanted}, and was given {clash}; an engine holding only "
            "some of these settings still starts, and serves from a different cache"
        )
    engine = {**REQUIRED_ENGINE_KWARGS, **kwargs, "model": model}
    engine.setdefault("max_num_seqs", MAX_SLOTS)   # one BF16 tail slot per running request
    if engine.get("max_model_len") is not None:
        # a prompt cannot be split, so it has to fit one batch
        engine.setdefault("max_num_batched_tokens",
                          max(engine["max_model_len"], engine["max_num_seqs"]))
    # the worker reads the variable while the layers are built
    if key_shift is None or key_shift == "auto":
        os.environ.pop(KEY_SHIFT_ENV, None)
    else:
        os.environ[KEY_SHIFT_ENV] = str(key_shift)
    supplied = engine.get("worker_extension_cls")
    if supplied is None:
        engine["worker_extension_cls"] = WORKER_EXTENSION_CLS   # also carries the on/off switch
    elif key_shift == "auto" and supplied != WORKER_EXTENSION_CLS:
        raise ValueError(
            f"measuring the shift needs worker_extension_cls={WORKER_EXTENSION_CLS!r}, and vLLM "
            "accepts one; either pass a sidecar path instead or mix that class into your own"
        )
    llm = LLM(**engine)
    if key_shift == "auto" and calibrate_key_shift(llm) is None:
        raise RuntimeError(
            "the engine came up without the NVFP4 cache, so there was no K mean to measure"
        )
    return llm
