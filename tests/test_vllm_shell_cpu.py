"""Host logic of the vLLM backend shell, on CPU: configuration guards, engine argument binding,
the decode-prefix split, the runtime's key-shift state machine and layer-order check, the page
carving and the control plane's argument checks.  No kernel is launched here.

The behaviours follow the reference project's ``tests/test_nvfp4_vllm.py`` and
``tests/test_llm_example.py`` (fail-closed guards, ``build_llm`` binding, layer order,
key-shift measurement); the carving is checked against the oracle's block assembly.
"""

from __future__ import annotations

import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import nvfp4_attn_kernel_b200 as pkg
import nvfp4_oracle as orc
from helpers import scale_bytes

pkg.install_aliases()

from nvfp4_vllm import control, guards, layout, runtime  # noqa: E402


def engine_config(**over):
    cache = SimpleNamespace(cache_dtype="nvfp4", enable_prefix_caching=False,
                            kv_cache_dtype_skip_layers=[], kv_offloading_size=None)
    sched = SimpleNamespace(max_num_seqs=32, enable_chunked_prefill=False,
                            long_prefill_token_threshold=0, max_num_batched_tokens=4096)
    parallel = SimpleNamespace(use_ubatching=False, pipeline_parallel_size=1)
    config = SimpleNamespace(cache_config=cache, scheduler_config=sched, parallel_config=parallel,
                             speculative_config=None)
    for dotted, value in over.items():
        section, _, field = dotted.partition("__")
        if field:
            setattr(getattr(config, section), field, value)
        else:
            setattr(config, section, value)
    return config


def test_guards_accept_the_supported_engine():
    guards.check_supported(engine_config())


@pytest.mark.parametrize("override, needle", [
    ({"scheduler_config__max_num_seqs": 33}, "max_num_seqs=33"),
    ({"cache_config__enable_prefix_caching": True}, "prefix caching"),
    ({"scheduler_config__enable_chunked_prefill": True}, "chunked prefill"),
    ({"scheduler_config__long_prefill_token_threshold": 512}, "long_prefill_token_threshold"),
    ({"speculative_config": object()}, "speculative"),
    ({"cache_config__kv_cache_dtype_skip_layers": ["3"]}, "kv_cache_dtype_skip_layers"),
    ({"cache_config__kv_offloading_size": 4.0}, "offloading"),
    ({"parallel_config__use_ubatching": True}, "microbatching"),
    ({"parallel_config__pipeline_parallel_size": 2}, "pipeline_parallel_size=2"),
])
def test_guards_refuse(override, needle):
    with pytest.raises(guards.UnsupportedConfigError, match=needle):
        guards.check_supported(engine_config(**override))


def test_guards_ignore_other_cache_dtypes():
    config = engine_config(cache_config__cache_dtype="auto",
                           cache_config__enable_prefix_caching=True,
                           scheduler_config__max_num_seqs=256)
    guards.check_supported(config)


def layer(**over):
    from vllm.v1.attention.backend import AttentionType

    fields = dict(attn_type=AttentionType.DECODER, kv_sharing_target_layer_name=None,
                  sliding_window=(-1, -1), logits_soft_cap=0, alibi_slopes=None, sinks=None)
    fields.update(over)
    return SimpleNamespace(**fields)


def test_layer_guards():
    from vllm.v1.attention.backend import AttentionType

    guards.check_layer_supported(layer())
    for over, needle in [
        ({"attn_type": AttentionType.ENCODER_ONLY}, "decoder cache"),
        ({"kv_sharing_target_layer_name": "model.layers.0.attn"}, "KV sharing"),
        ({"sliding_window": (4095, 0)}, "sliding window"),
        ({"logits_soft_cap": 30.0}, "soft capping"),
        ({"alibi_slopes": torch.ones(4)}, "ALiBi"),
        ({"sinks": torch.ones(4)}, "sinks"),
    ]:
        with pytest.raises(guards.UnsupportedConfigError, match=needle):
            guards.check_layer_supported(layer(**over))


# ---------------------------------------------------------------- build_llm


class RecordingLLM:
    """Stands in for ``vllm.LLM``: keeps the engine arguments, answers the calibration calls."""

    last = None

    def __init__(self, **kwargs):
        self.kwargs = kwargs
        self.rpc = []
        RecordingLLM.last = self


@pytest.fixture
def fake_llm(monkeypatch):
    import vllm

    from nvfp4_vllm import calibrate

    monkeypatch.setattr(vllm, "LLM", RecordingLLM, raising=False)
    calls = []

    def measured(llm, **kwargs):
        calls.append(llm)
        return {"tokens": 1}

    monkeypatch.setattr(calibrate, "calibrate_key_shift", measured)
    monkeypatch.delenv("NVFP4_KEY_SHIFT", raising=False)
    return calls


def test_build_llm_binds_the_required_arguments(fake_llm):
    from nvfp4_vllm import engine

    llm = engine.build_llm("some/model", max_model_len=8192, gpu_memory_utilization=0.5)
    for name, need in engine.REQUIRED_ENGINE_KWARGS.items():
        assert llm.kwargs[name] == need
    assert llm.kwargs["model"] == "some/model"
    assert llm.kwargs["max_num_seqs"] == 32
    assert llm.kwargs["max_num_batched_tokens"] == 8192
    assert llm.kwargs["gpu_memory_utilization"] == 0.5
    assert llm.kwargs["worker_extension_cls"].endswith("calibrate.NVFP4WorkerExtension")
    assert fake_llm == [llm]                      # "auto" measured once
    assert "NVFP4_KEY_SHIFT" not in os.environ


def test_build_llm_refuses_a_contradiction(fake_llm):
    from nvfp4_vllm import engine

    with pytest.raises(ValueError, match="block_size"):
        engine.build_llm("m", block_size=16)
    with pytest.raises(ValueError, match="enable_prefix_caching"):
        engine.build_llm("m", enable_prefix_caching=True)
    # restating a required value is fine
    engine.build_llm("m", block_size=128, kv_cache_dtype="nvfp4")


def test_build_llm_key_shift_modes(fake_llm, tmp_path):
    from nvfp4_vllm import engine

    engine.build_llm("m", key_shift=None)
    assert fake_llm == [] and "NVFP4_KEY_SHIFT" not in os.environ
    sidecar = tmp_path / "shift.safetensors"
    engine.build_llm("m", key_shift=sidecar)
    assert fake_llm == [] and os.environ["NVFP4_KEY_SHIFT"] == str(sidecar)
    engine.build_llm("m", key_shift=None)          # a stale path must not leak into the next engine
    assert "NVFP4_KEY_SHIFT" not in os.environ
    with pytest.raises(ValueError, match="worker_extension_cls"):
        engine.build_llm("m", worker_extension_cls="mine.Extension")
    llm = engine.build_llm("m", key_shift=None, worker_extension_cls="mine.Extension")
    assert llm.kwargs["worker_extension_cls"] == "mine.Extension"


def test_build_llm_reports_an_engine_without_the_cache(fake_llm, monkeypatch):
    from nvfp4_vllm import calibrate, engine

    monkeypatch.setattr(calibrate, "calibrate_key_shift", lambda llm, **kw: None)
    with pytest.raises(RuntimeError, match="without the NVFP4 cache"):
        engine.build_llm("m")


def test_small_max_model_len_still_covers_one_token_per_row(fake_llm):
    from nvfp4_vllm import engine

    llm = engine.build_llm("m", max_model_len=16, key_shift=None)
    assert llm.kwargs["max_num_batched_tokens"] == 32


# ---------------------------------------------------------------- calibration client


class RpcLLM:
    def __init__(self, replies):
        self.replies = replies
        self.calls = []
        self.resets = 0

    def collective_rpc(self, method, args=()):
        self.calls.append((method, args))
        return self.replies[method]

    def reset_prefix_cache(self):
        self.resets += 1

    def get_tokenizer(self):
        return SimpleNamespace(encode=lambda text, add_special_tokens=False: list(range(len(text.split()))))


def test_set_key_shift_enabled_round_trip():
    from nvfp4_vllm import calibrate

    llm = RpcLLM({"nvfp4_set_key_shift_enabled": [28, 28]})
    assert calibrate.set_key_shift_enabled(llm, False) is True
    assert llm.calls == [("nvfp4_set_key_shift_enabled", (False,))] and llm.resets == 1
    assert calibrate.set_key_shift_enabled(RpcLLM({"nvfp4_set_key_shift_enabled": [0]}), True) is False


def test_long_prompt_tiles_to_the_budget():
    from nvfp4_vllm import calibrate

    llm = RpcLLM({})
    ids = calibrate._long_prompt(llm, ["a b c", "d e"], 23)
    assert len(ids) == 23 and ids[:5] == [0, 1, 2, 3, 4] and ids[5] == 0
    with pytest.raises(ValueError, match="no calibration text"):
        calibrate._long_prompt(llm, ["", "  "], 8)


def test_seeds_are_short_ordinary_text():
    from nvfp4_vllm import calibrate

    assert len(calibrate.SEEDS) >= 4 and len(set(calibrate.SEEDS)) == len(calibrate.SEEDS)
    assert all(20 < len(s) < 200 for s in calibrate.SEEDS)


# ---------------------------------------------------------------- decode prefix


def batch(query_lens, max_query_len=None):
    starts = torch.tensor([0, *np.cumsum(query_lens)], dtype=torch.int32)
    return SimpleNamespace(query_start_loc_cpu=starts, num_reqs=len(query_lens),
                           num_actual_tokens=int(starts[-1]),
                           max_query_len=max_query_len or max(query_lens), is_prefilling=None)


def test_decode_split():
    from nvfp4_vllm.builder import decode_split

    assert decode_split(batch([1, 1, 1])) == (3, 3)
    assert decode_split(batch([1, 1, 40, 300])) == (2, 2)
    assert decode_split(batch([40, 300])) == (0, 0)
    assert decode_split(batch([1, 1, 0, 0], max_query_len=1)) == (4, 2)   # graph padding rows
    with pytest.raises(ValueError, match="front of the batch"):
        decode_split(batch([1, 40, 1, 7]))


# ---------------------------------------------------------------- runtime


def small_runtime(layers=3, heads_kv=2):
    return runtime.LayerRuntime(num_layers=layers, num_slots=4, num_heads=2 * heads_kv,
                                num_kv_heads=heads_kv, head_dim=128, device="cpu")


def test_runtime_key_shift_state_machine(monkeypatch):
    monkeypatch.delenv(runtime.KEY_SHIFT_ENV, raising=False)
    rt = small_runtime()
    assert rt.key_shift is None and rt.active_key_shift is None
    with pytest.raises(ValueError, match="nothing to enable"):
        rt.set_key_shift_enabled(True)
    with pytest.raises(ValueError, match="no tokens were measured"):
        rt.finish_key_shift_measurement()
    rt.begin_key_shift_measurement()
    with pytest.raises(ValueError, match="no tokens were measured"):
        rt.finish_key_shift_measurement()
    rt.begin_key_shift_measurement()
    keys = torch.randn(5, 2, 128, dtype=torch.float64)
    for layer_index in range(3):
        rt.key_shift_sum[layer_index] += keys.sum(0) * (layer_index + 1)
    rt.key_shift_tokens = 5
    shift = rt.finish_key_shift_measurement()
    assert shift.dtype is torch.bfloat16 and tuple(shift.shape) == (3, 2, 128)
    assert torch.equal(shift[1], (2 * keys.mean(0)).to(torch.bfloat16))
    assert rt.active_key_shift is shift and rt.key_shift_sum is None
    rt.set_key_shift_enabled(False)
    assert rt.active_key_shift is None and rt.key_shift is shift
    rt.set_key_shift_enabled(True)
    assert rt.active_key_shift is shift


def test_runtime_loads_a_sidecar(monkeypatch, tmp_path):
    from safetensors.torch import save_file

    path = tmp_path / "shift.safetensors"
    save_file({"key_shift": torch.full((3, 2, 128), 0.25)}, str(path))
    monkeypatch.setenv(runtime.KEY_SHIFT_ENV, str(path))
    rt = small_runtime()
    assert rt.key_shift.dtype is torch.bfloat16 and float(rt.key_shift[2, 1, 7]) == 0.25
    with pytest.raises(ValueError, match="this model needs"):
        small_runtime(layers=4)
    save_file({"other": torch.zeros(1)}, str(path))
    with pytest.raises(ValueError, match="no 'key_shift'"):
        small_runtime()


def test_runtime_layer_order(monkeypatch):
    monkeypatch.delenv(runtime.KEY_SHIFT_ENV, raising=False)
    rt = small_runtime()
    for _ in range(2):
        for layer_index in range(3):
            rt.expect_layer(layer_index)
    rt.expect_layer(0)
    with pytest.raises(ValueError, match="layer 2 ran where layer 1 was expected"):
        rt.expect_layer(2)
    rt.expect_layer(0)   # after the error the next step starts clean


def test_runtime_destination_bases(monkeypatch):
    monkeypatch.delenv(runtime.KEY_SHIFT_ENV, raising=False)
    rt = small_runtime(layers=2, heads_kv=2)
    pitch = layout.page_bytes(2)
    caches = [torch.zeros(5, pitch, dtype=torch.uint8) for _ in range(2)]
    rt.views(0, caches[0])
    with pytest.raises(ValueError, match=r"layers \[1\]"):
        rt.destination_bases
    rt.views(1, caches[1])
    bases = rt.destination_bases
    assert tuple(bases.shape) == (4, 2)
    packed, scales = 128 * 2 * 64, 2 * 1024
    for layer_index, cache in enumerate(caches):
        start = cache.data_ptr()
        assert bases[:, layer_index].tolist() == [start, start + packed, start + packed + scales,
                                                  start + 2 * packed + scales]
    assert rt.views(0, caches[0]) is rt.layer_regions(0)
    assert rt.tail_bytes == 2 * 2 * 4 * 128 * 2 * 128 * 2


# ---------------------------------------------------------------- layout


def test_carve_matches_the_oracle_block_assembly():
    rng = np.random.default_rng(5)
    pages, heads = 3, 2
    key = orc.bf16_round(rng.standard_normal((pages, 128, heads, 128)).astype(np.float32))
    value = orc.bf16_round(rng.standard_normal((pages, 128, heads, 128)).astype(np.float32))
    k_packed, k_sf = orc.quantize_key_pages(key)
    v_packed, v_sf = orc.quantize_value_pages(value)
    blocks = orc.assemble_vllm_blocks(k_packed, k_sf, v_packed, v_sf)
    assert blocks.shape == (pages, layout.page_bytes(heads))
    cache = torch.from_numpy(blocks.copy())
    got = layout.carve(cache, heads, 128)
    assert np.array_equal(got[0].numpy(), k_packed)
    assert np.array_equal(got[2].numpy(), v_packed)
    assert np.array_equal(scale_bytes(got[1]), k_sf.reshape(pages, -1))
    assert np.array_equal(scale_bytes(got[3]), v_sf.reshape(pages, -1))
    # element (page, row%32, row/32, 0, group%4, group/4, head) of the view is the scale of
    # (row, 16-wide group) of that head: spot-check against the atom offset rule
    row, group, head = 77, 5, 1
    assert int(got[1].view(torch.uint8)[2, row % 32, row // 32, 0, group % 4, group // 4, head]) == \
        int(k_sf.reshape(pages, heads, 1024)[2, head, orc.sf_atom_offset(row, group)])
    with pytest.raises(ValueError, match="cannot hold"):
        layout.carve(torch.zeros(3, 1000, dtype=torch.uint8), heads, 128)
    with pytest.raises(ValueError, match="byte cache"):
        layout.carve(torch.zeros(3, 8, dtype=torch.float16), heads, 128)


def test_backend_declares_the_page():
    from nvfp4_vllm import backend

    assert backend.NVFP4Backend.get_name() == "CUSTOM"
    assert backend.nvfp4_page_size_bytes(128, 8, 128) == 147456 == layout.page_bytes(8)
    assert backend.NVFP4Backend.get_kv_cache_shape(7, 128, 8, 128, "nvfp4") == (7, 147456)
    assert backend.NVFP4Backend.supports_block_size(128)
    assert not backend.NVFP4Backend.supports_block_size(16)
    assert backend.NVFP4Backend.get_supported_kernel_block_sizes() == [128]
    assert backend.NVFP4Backend.supports_compute_capability(SimpleNamespace(major=10, minor=0))
    assert not backend.NVFP4Backend.supports_compute_capability(SimpleNamespace(major=9, minor=0))
    assert not backend.NVFP4Backend.supports_kv_connector()
    assert "nvfp4" in backend.NVFP4Backend.supported_kv_cache_dtypes


def test_register_points_custom_at_the_backend():
    import nvfp4_vllm
    from vllm.v1.attention.backends.registry import AttentionBackendEnum

    nvfp4_vllm.register()
    assert AttentionBackendEnum.CUSTOM.get_path().endswith("nvfp4_vllm.backend.NVFP4Backend")


# ---------------------------------------------------------------- control plane arguments


def test_control_plane_argument_checks():
    with pytest.raises(ValueError, match="positive"):
        control.ControlPlane(max_num_seqs=0, max_num_batched_tokens=8, device="cpu")
    with pytest.raises(ValueError, match="at most 128"):
        control.ControlPlane(max_num_seqs=129, max_num_batched_tokens=256, device="cpu")
    with pytest.raises(ValueError, match="one token per row"):
        control.ControlPlane(max_num_seqs=8, max_num_batched_tokens=4, device="cpu")
    plane = control.ControlPlane(max_num_seqs=4, max_num_batched_tokens=64, device="cpu")
    table = torch.zeros(4, 3, dtype=torch.int32)
    lens = torch.zeros(4, dtype=torch.int32)
    starts = torch.zeros(5, dtype=torch.int32)
    with pytest.raises(ValueError, match="exceeds the 4 tail slots"):
        plane.prepare(block_table=table, seq_lens=lens, query_start_loc=starts, num_reqs=5,
                      num_actual_tokens=5)
    with pytest.raises(ValueError, match="exceeds the 64"):
        plane.prepare(block_table=table, seq_lens=lens, query_start_loc=starts, num_reqs=4,
                      num_actual_tokens=65)
    with pytest.raises(ValueError, match="INT32"):
        plane.prepare(block_table=table.long(), seq_lens=lens, query_start_loc=starts, num_reqs=4,
                      num_actual_tokens=4)
    with pytest.raises(ValueError, match="2-D"):
        plane.prepare(block_table=table[0], seq_lens=lens, query_start_loc=starts, num_reqs=4,
                      num_actual_tokens=4)
    plane.error_code.fill_(control.ERR_NO_FREE_SLOT | control.ERR_DUPLICATE_KEY)
    with pytest.raises(control.ControlPlaneError, match="none free.*share a physical block"):
        plane.raise_for_errors()
    plane.reset()
    plane.raise_for_errors()
    assert int(plane.slot_keys.max()) == control.FREE_KEY


def test_balance_pages_heuristic():
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel._decode import balance_pages_heuristic

    # 1152 pages x 8 KV heads over 296 resident CTAs: an even share of 31 pages, pieces of 47
    assert balance_pages_heuristic(1152, 8, sms=148) == 47
    assert balance_pages_heuristic(10, 8, sms=148) == 16          # never below the floor
    assert balance_pages_heuristic(0, 8, sms=148) == 16
    assert balance_pages_heuristic(1152, 8, sms=148, floor=64) == 64
    # more work, longer pieces; more SMs, shorter ones
    assert balance_pages_heuristic(4000, 8, sms=148) > balance_pages_heuristic(2000, 8, sms=148)
    assert balance_pages_heuristic(4000, 8, sms=296) < balance_pages_heuristic(4000, 8, sms=148)


def test_piece_pages_policy(monkeypatch):
    from nvfp4_attn_kernel_b200.nvfp4_vllm.runtime import BALANCE_PAGES_ENV, piece_pages

    monkeypatch.delenv(BALANCE_PAGES_ENV, raising=False)
    # a batch that fills the GPU with whole rows is left alone
    assert piece_pages(32, 8, 32, 148) == 0
    # one long row: 8 CTAs would walk 256 pages each; pieces of 16 pages make 128 CTAs
    assert piece_pages(1, 8, 256, 148) == 16
    assert piece_pages(4, 8, 256, 148) == 42
    # short tables are never cut
    assert piece_pages(1, 8, 16, 148) == 0
    # explicit settings
    assert piece_pages(32, 8, 32, 148, "0") == 0
    assert piece_pages(32, 8, 32, 148, "8") == 8
    assert piece_pages(32, 8, 8, 148, "8") == 0
    monkeypatch.setenv(BALANCE_PAGES_ENV, "0")
    assert piece_pages(1, 8, 256, 148) == 0
    monkeypatch.setenv(BALANCE_PAGES_ENV, "24")
    assert piece_pages(1, 8, 256, 148) == 24
    with pytest.raises(ValueError):
        piece_pages(1, 8, 256, 148, "-3")


def test_runtime_reserves_the_balanced_split_scratch(monkeypatch):
    from nvfp4_attn_kernel_b200.nvfp4_decode_kernel._decode import balanced_workspace_bytes

    monkeypatch.delenv(runtime.KEY_SHIFT_ENV, raising=False)
    monkeypatch.delenv(runtime.BALANCE_PAGES_ENV, raising=False)
    rt = runtime.LayerRuntime(num_layers=1, num_slots=8, num_heads=8, num_kv_heads=2, head_dim=128,
                              device="cpu", max_pages=256)
    held = rt._balance_workspace
    assert held is not None
    # EVERY step shape that the policy would cut fits the reserved scratch (the need is not
    # monotone in the table width), and the scratch handed out is always the reserved one
    for rows in range(1, 9):
        for columns in range(1, 257):
            piece = runtime.piece_pages(rows, 2, columns, rt.sm_count)
            if piece:
                need = rt.balance_need(rows, 8, columns, piece)
                assert need == balanced_workspace_bytes(rows, 8, columns, piece)   # the library's own figure
                assert need <= held.numel()
                assert rt.balance_workspace(rows, 8, columns, piece) is held
    # a step that does not fit gets None (it runs with whole rows); the buffer is never replaced
    assert rt.balance_workspace(8, 8, 256, 1) is None
    assert rt._balance_workspace is held
    # the shape the advisor found short of its reservation: 32 slots, one KV head, 1024 pages
    tp = runtime.LayerRuntime(num_layers=1, num_slots=32, num_heads=4, num_kv_heads=1, head_dim=128,
                              device="cpu", max_pages=1024)
    piece = runtime.piece_pages(32, 1, 111, tp.sm_count)
    assert piece and tp.balance_need(32, 4, 111, piece) <= tp._balance_workspace.numel()
    # switched off, or a short model: nothing is reserved
    monkeypatch.setenv(runtime.BALANCE_PAGES_ENV, "0")
    assert runtime.LayerRuntime(num_layers=1, num_slots=8, num_heads=8, num_kv_heads=2, head_dim=128,
                                device="cpu", max_pages=256)._balance_workspace is None
    monkeypatch.delenv(runtime.BALANCE_PAGES_ENV)
    assert runtime.LayerRuntime(num_layers=1, num_slots=8, num_heads=8, num_kv_heads=2, head_dim=128,
                                device="cpu", max_pages=8)._balance_workspace is None
    # an explicit tiny piece whose worst case is huge: nothing reserved, steps leave their rows whole
    monkeypatch.setenv(runtime.BALANCE_PAGES_ENV, "1")
    big = runtime.LayerRuntime(num_layers=1, num_slots=64, num_heads=64, num_kv_heads=8, head_dim=128,
                               device="cpu", max_pages=4096)
    assert big._balance_workspace is None


def test_work_list_is_reused_only_for_the_step_that_built_it():
    rt = runtime.LayerRuntime(num_layers=2, num_slots=4, num_heads=8, num_kv_heads=2, head_dim=128,
                              device="cpu", max_pages=64)
    key = (1234, 4, 40, 16, 99)
    rt.work_list_reusable(None)                           # layer 0 clears the record
    assert rt.work_list_reusable(key) is False            # nobody built this list yet
    assert rt.work_list_reusable(key) is True             # the next layer of the step finds it
    assert rt.work_list_reusable((1234, 3, 40, 16, 99)) is False   # another shape: rebuilt
