"""Runs a live vLLM engine (in-process engine core, dummy weights, a two-layer Llama-shaped model
with 8 query / 2 KV heads of 128 channels) on the NVFP4 ``CUSTOM`` backend and prints the greedy
tokens of six prompts as one JSON line.  Started as a child process by ``test_vllm_live_gpu.py``;
the flags choose the variant:

    --graphs          CUDA graphs instead of eager mode
    --separate        the reference's launch structure: separate query quantiser and tail copy
    --stock           vLLM's own FlashAttention backend with a BF16 cache (for comparison)
    --shift           measure the key shift through the worker extension, serve with it, switch
                      it off and serve again
"""

import json
import os
import sys
import tempfile

os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")   # the plugin is registered in this process
os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    import numpy as np

    import nvfp4_attn_kernel_b200 as pkg

    pkg.install_aliases()
    import nvfp4_vllm
    from nvfp4_decode_kernel import _kernel
    from nvfp4_vllm import impl

    flags = set(sys.argv[1:])
    model_dir = tempfile.mkdtemp(prefix="tiny_llama_")
    config = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "hidden_size": 1024, "intermediate_size": 2048, "num_hidden_layers": 2,
        "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128,
        "vocab_size": 2048, "max_position_embeddings": 4096, "rms_norm_eps": 1e-5,
        "rope_theta": 10000.0, "hidden_act": "silu", "tie_word_embeddings": False,
        "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2,
    }
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(config, f)
    common = dict(load_format="dummy", skip_tokenizer_init=True, max_model_len=2048,
                  enforce_eager="--graphs" not in flags, gpu_memory_utilization=0.2, max_num_seqs=8,
                  seed=0, dtype="bfloat16")
    if "--stock" in flags:
        from vllm import LLM

        llm = LLM(model=model_dir, enable_prefix_caching=False, **common)
    else:
        nvfp4_vllm.register()
        if "--separate" in flags:
            _kernel.FUSE_QUERY_QUANT = False
            impl.FUSE_TAIL_APPEND = False
        llm = nvfp4_vllm.build_llm(model_dir, key_shift=None, **common)

    from vllm import SamplingParams, TokensPrompt

    rng = np.random.default_rng(0)
    # lengths around the page size: the 128- and 257-token prompts seal pages at once, every
    # request crosses a page boundary (a tail flush) while it decodes 200 tokens
    prompts = [TokensPrompt(prompt_token_ids=rng.integers(3, 2000, n).tolist()) for n in (5, 130, 300, 128, 40, 257)]
    params = SamplingParams(temperature=0.0, max_tokens=200, ignore_eos=True, detokenize=False)
    result = {}
    if "--shift" in flags:
        # what calibrate_key_shift does, with token prompts (this engine has no tokenizer): let
        # every layer accumulate the K sum over one long prefill, freeze the mean, serve with it
        from nvfp4_vllm import calibrate

        assert any(llm.collective_rpc("nvfp4_begin_key_shift_measurement"))
        llm.generate([TokensPrompt(prompt_token_ids=rng.integers(3, 2000, 700).tolist())],
                     SamplingParams(temperature=0.0, max_tokens=1, detokenize=False), use_tqdm=False)
        result["report"] = llm.collective_rpc("nvfp4_finish_key_shift_measurement", args=(None,))[0]
        result["active"] = llm.collective_rpc("nvfp4_key_shift_is_active")
        shifted = llm.generate(prompts, params, use_tqdm=False)
        result["tokens_shifted"] = [list(o.outputs[0].token_ids) for o in shifted]
        result["switched_off"] = calibrate.set_key_shift_enabled(llm, False)
    outs = llm.generate(prompts, params, use_tqdm=False)
    result["tokens"] = [list(o.outputs[0].token_ids) for o in outs]

    if "--stock" not in flags:
        def error_words(worker):
            from nvfp4_vllm.builder import NVFP4MetadataBuilder

            found = []
            for groups in getattr(worker.model_runner, "attn_groups", []):
                for group in groups:
                    for builder in getattr(group, "metadata_builders", []):
                        if isinstance(builder, NVFP4MetadataBuilder) and builder.plane is not None:
                            found.append(int(builder.plane.error_code.item()))
            return found

        result["control_plane_errors"] = llm.collective_rpc(error_words)
    print("RESULT " + json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
