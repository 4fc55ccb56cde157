"""Fail-closed checks of the engine and layer configuration for the NVFP4 KV cache.

Same checks, same exception type and the same advice as the reference project's
``src/nvfp4_vllm/guards.py`` (``check_supported`` :30-116, ``check_layer_supported`` :119-153).
They run from ``NVFP4Impl.__init__`` (once per layer per engine), not from the backend selector,
whose verdicts vLLM memoises on a key that carries none of these fields.
"""

from __future__ import annotations

from .control import MAX_SUPPORTED_SLOTS

NVFP4 = "nvfp4"
# one BF16 tail slot per running request
MAX_SLOTS = MAX_SUPPORTED_SLOTS


class UnsupportedConfigError(ValueError):
    """An engine configuration the NVFP4 path cannot serve correctly."""


def check_supported(vllm_config) -> None:
    """Raise unless the engine is configured the way the NVFP4 cache needs.  No-op for any
    other ``kv_cache_dtype`` (the backend is then a FlashAttention pass-through)."""
    cache = vllm_config.cache_config
    if cache is None or cache.cache_dtype != NVFP4:
        return
    sched = vllm_config.scheduler_config
    parallel = vllm_config.parallel_config

    if sched is not None and sched.max_num_seqs > MAX_SLOTS:
        raise UnsupportedConfigError(
            f"max_num_seqs={sched.max_num_seqs} exceeds the {MAX_SLOTS} BF16 tail slots the "
            f"NVFP4 path preallocates. Pass max_num_seqs<={MAX_SLOTS}, or use a BF16 KV cache."
        )
    if cache.enable_prefix_caching:
        raise UnsupportedConfigError(
            "prefix caching is not supported by the NVFP4 KV cache: a cache hit resumes a "
            "sequence mid-page, and prefill over an FP4 prefix is not implemented. "
            "Pass enable_prefix_caching=False."
        )
    # From here on: a step either runs a whole prompt from nothing or extends a sequence by
    # exactly one token.
    if sched is not None and sched.enable_chunked_prefill:
        raise UnsupportedConfigError(
            "chunked prefill is not supported by the NVFP4 KV cache: the second chunk of a "
            "split prompt resumes mid-page, which needs prefill over an FP4 prefix. Pass "
            "enable_chunked_prefill=False; vLLM then requires max_num_batched_tokens >= "
            "max_model_len so that no prompt has to be split."
        )
    if sched is not None and sched.long_prefill_token_threshold:
        raise UnsupportedConfigError(
            f"long_prefill_token_threshold={sched.long_prefill_token_threshold} splits long "
            "prompts even with chunked prefill disabled. Leave it at 0."
        )
    if vllm_config.speculative_config is not None:
        raise UnsupportedConfigError(
            "speculative decoding is not supported by the NVFP4 KV cache: it verifies several "
            "draft tokens per step, and the decode kernel attends one query token per sequence."
        )
    if cache.kv_cache_dtype_skip_layers:
        raise UnsupportedConfigError(
            f"kv_cache_dtype_skip_layers={cache.kv_cache_dtype_skip_layers} leaves some layers "
            "on a different cache dtype, which splits the model into KV cache groups with their "
            "own metadata builders (the slot table would advance more than once per step). "
            "Leave it empty."
        )
    if cache.kv_offloading_size is not None:
        raise UnsupportedConfigError(
            "KV offloading is not supported by the NVFP4 KV cache: it copies pages by address "
            "and size, which does not describe the packed FP4 layout. Leave kv_offloading_size "
            "unset."
        )
    if parallel is not None and parallel.use_ubatching:
        raise UnsupportedConfigError(
            "microbatching is not supported by the NVFP4 KV cache: each ubatch builds its own "
            "attention metadata, so the slot table would advance twice per step. Leave "
            "enable_dbo unset and ubatch_size at 0."
        )
    if parallel is not None and parallel.pipeline_parallel_size > 1:
        raise UnsupportedConfigError(
            f"pipeline_parallel_size={parallel.pipeline_parallel_size} is not supported by the "
            "NVFP4 KV cache: page promotion is driven from the last attention layer, which a "
            "pipeline stage does not own. Pass pipeline_parallel_size=1."
        )


def check_layer_supported(impl) -> None:
    """Raise unless this attention layer is plain scaled dot-product decoder attention."""
    from vllm.v1.attention.backend import AttentionType

    if impl.attn_type != AttentionType.DECODER:
        raise UnsupportedConfigError(
            f"attention type {impl.attn_type} is not supported by the NVFP4 KV cache, which is "
            "a decoder cache."
        )
    if impl.kv_sharing_target_layer_name is not None:
        raise UnsupportedConfigError(
            "cross-layer KV sharing is not supported by the NVFP4 KV cache: the BF16 tail is "
            "indexed by layer, so a layer that reads another layer's cache would read its own "
            "empty tail."
        )
    modifiers = {
        "sliding window": impl.sliding_window != (-1, -1),
        "logit soft capping": bool(impl.logits_soft_cap),
        "ALiBi": impl.alibi_slopes is not None,
        "attention sinks": impl.sinks is not None,
    }
    present = [name for name, on in modifiers.items() if on]
    if present:
        raise UnsupportedConfigError(
            f"{', '.join(present)} is not supported by the NVFP4 decode kernel, which computes "
            "unmodified scaled dot-product attention over the whole cache."
        )
