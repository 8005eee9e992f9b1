"""Import-level and host-logic checks of the ``nvfp4_vllm`` plugin against the installed vLLM
(no GPU): entry point, backend declarations, engine guards, cache carving, host split policy."""

import types

import pytest
import torch

vllm = pytest.importorskip("vllm")


def test_register_claims_the_custom_backend():
    import nvfp4_vllm
    from vllm.v1.attention.backends.registry import AttentionBackendEnum

    nvfp4_vllm.register()
    assert AttentionBackendEnum.CUSTOM.get_path() == "nvfp4_vllm.backend.NVFP4Backend"
    assert AttentionBackendEnum.CUSTOM.get_class().__name__ == "NVFP4Backend"


def test_backend_declarations():
    from nvfp4_vllm.backend import NVFP4Backend, nvfp4_page_size_bytes

    assert NVFP4Backend.get_name() == "CUSTOM"
    assert NVFP4Backend.get_supported_kernel_block_sizes() == [128]
    assert NVFP4Backend.supports_block_size(128) and not NVFP4Backend.supports_block_size(256)
    assert not NVFP4Backend.supports_kv_connector()
    assert NVFP4Backend.supports_compute_capability(types.SimpleNamespace(major=10, minor=0))
    assert not NVFP4Backend.supports_compute_capability(types.SimpleNamespace(major=9, minor=0))
    assert nvfp4_page_size_bytes(128, 8, 128) == 2 * 128 * 8 * 72
    assert NVFP4Backend.get_kv_cache_shape(7, 128, 8, 128, "nvfp4") == (7, 147456)
    assert "nvfp4" in NVFP4Backend.supported_kv_cache_dtypes
    reason = NVFP4Backend.supports_combination(64, torch.bfloat16, "nvfp4", 128, False, False, False, False, None)
    assert reason is not None and "128" in reason
    assert NVFP4Backend.get_impl_cls().__name__ == "NVFP4Impl"
    assert NVFP4Backend.get_builder_cls().__name__ == "NVFP4MetadataBuilder"


def test_carve_matches_the_declared_page_size():
    from nvfp4_vllm import layout

    heads = 2
    cache = torch.arange(3 * layout.page_bytes(heads, 128), dtype=torch.int64).remainder(251).to(torch.uint8)
    cache = cache.reshape(3, -1)
    kc, ks, vc, vs = layout.carve(cache, heads, 128)
    assert kc.shape == (3, 128, heads, 64) and vc.shape == (3, heads, 128, 64)
    assert ks.shape == (3, 32, 4, 1, 4, 2, heads) and ks.dtype is torch.float8_e4m3fn
    pitch = cache.shape[1]
    assert kc.stride(0) == ks.stride(0) == vc.stride(0) == vs.stride(0) == pitch
    # byte offsets of the four regions inside a block
    offsets = [t.storage_offset() for t in (kc, ks, vc, vs)]
    assert offsets == [0, 8192 * heads, 9216 * heads, 17408 * heads]
    assert int(vc[1, 1, 5, 7]) == int(cache[1, 9216 * heads + 8192 + 5 * 64 + 7])
    with pytest.raises(ValueError):
        layout.carve(cache[:, :-16].contiguous(), heads, 128)


def _config(**overrides):
    cache = types.SimpleNamespace(cache_dtype="nvfp4", enable_prefix_caching=False, kv_cache_dtype_skip_layers=None,
                                  kv_offloading_size=None)
    scheduler = types.SimpleNamespace(max_num_seqs=32, enable_chunked_prefill=False, long_prefill_token_threshold=0)
    parallel = types.SimpleNamespace(use_ubatching=False, pipeline_parallel_size=1)
    config = types.SimpleNamespace(cache_config=cache, scheduler_config=scheduler, parallel_config=parallel,
                                   speculative_config=None, additional_config={})
    for path, value in overrides.items():
        target, _, name = path.rpartition(".")
        setattr(getattr(config, target) if target else config, name, value)
    return config


def test_guards_refuse_what_the_cache_cannot_serve():
    from nvfp4_vllm import guards

    guards.check_supported(_config())
    for override in ({"cache_config.enable_prefix_caching": True}, {"scheduler_config.enable_chunked_prefill": True},
                     {"scheduler_config.max_num_seqs": 129}, {"speculative_config": object()},
                     {"parallel_config.pipeline_parallel_size": 2}, {"cache_config.kv_offloading_size": 1.0},
                     {"scheduler_config.long_prefill_token_threshold": 512}):
        with pytest.raises(guards.UnsupportedConfigError):
            guards.check_supported(_config(**override))
    other = _config(**{"cache_config.cache_dtype": "auto", "cache_config.enable_prefix_caching": True})
    guards.check_supported(other)  # any other cache dtype is a FlashAttention pass-through


def test_guards_resolve_additional_config():
    from nvfp4_vllm import guards

    assert guards.resolve_scale_mode(_config()) == ("amax6", "amax6", "amax6")
    config = _config(additional_config={"nvfp4_scale_mode": {"key": "four_six", "value": "amax6", "query": "amax6"},
                                        "nvfp4_query_terms": 2, "nvfp4_rotation": "hadamard"})
    assert guards.resolve_scale_mode(config).key == "four_six"
    assert guards.resolve_query_terms(config) == 2 and guards.resolve_rotation(config) == "hadamard"
    for bad in ({"nvfp4_scale_mode": "amax7"}, {"nvfp4_scale_mode": {"key": "amax6"}},
                {"nvfp4_scale_mode": {"key": "mxfp4_ocp", "value": "amax6", "query": "amax6"}}):
        with pytest.raises(guards.UnsupportedConfigError):
            guards.resolve_scale_mode(_config(additional_config=bad))
    with pytest.raises(guards.UnsupportedConfigError):
        guards.resolve_query_terms(_config(additional_config={"nvfp4_query_terms": 3}))
    with pytest.raises(guards.UnsupportedConfigError):
        guards.resolve_rotation(_config(additional_config={"nvfp4_rotation": "dct"}))


def test_engine_kwargs():
    from nvfp4_vllm import engine

    kwargs = engine.engine_kwargs("some/model", max_model_len=65536)
    assert kwargs["kv_cache_dtype"] == "nvfp4" and kwargs["block_size"] == 128
    assert kwargs["attention_config"] == {"backend": "CUSTOM"}
    assert kwargs["max_num_seqs"] == 32 and kwargs["max_num_batched_tokens"] == 65536
    with pytest.raises(ValueError):
        engine.engine_kwargs("m", enable_prefix_caching=True)
    # smoothing defaults to calibration at start-up, which needs the plugin's worker extension
    from nvfp4_vllm.calibrate import WORKER_EXTENSION_CLS

    assert kwargs["additional_config"]["nvfp4_key_smoothing"] == "auto"
    assert kwargs["worker_extension_cls"] == WORKER_EXTENSION_CLS
    with pytest.raises(ValueError):
        engine.engine_kwargs("m", worker_extension_cls="other.Extension")
    sidecar = engine.engine_kwargs("m", additional_config={"nvfp4_key_smoothing": "/tmp/shift.safetensors"},
                                   worker_extension_cls="other.Extension")
    assert sidecar["worker_extension_cls"] == "other.Extension"


def test_split_policies_match_reference_values(golden):
    from nvfp4_decode_kernel import split_partial_count
    from nvfp4_decode_kernel._decode import split_k_heuristic
    from nvfp4_vllm.builder import decode_num_splits

    for rows, heads, sms, want in golden["policy_decode_num_splits"]:
        assert decode_num_splits(int(rows), int(heads), int(sms)) == int(want)
    for rows, heads, pages, sms, want in golden["policy_split_k_heuristic"]:
        assert split_k_heuristic(int(rows), int(heads), int(pages), sms=int(sms)) == int(want)
    for rows, heads, splits, residual, sms, want in golden["policy_split_partial_count"]:
        assert split_partial_count(int(rows), int(heads), int(splits), residual=bool(residual), sms=int(sms)) == int(want)


def test_key_shift_sidecar_loading(tmp_path, monkeypatch):
    from safetensors.torch import save_file

    from nvfp4_vllm import runtime

    shift = torch.randn(3, 8, 128)
    path = tmp_path / "shift.safetensors"
    save_file({"key_shift": shift}, str(path))
    monkeypatch.setenv(runtime.KEY_SHIFT_ENV, str(path))
    local = runtime.load_key_shift(3, 4, 128, "cpu", torch.float32, tensor_parallel_size=2, tensor_parallel_rank=1)
    assert torch.equal(local, shift[:, 4:])
    rotation = runtime.sylvester_hadamard(128, "cpu", torch.float32)
    rotated = runtime.load_key_shift(3, 8, 128, "cpu", torch.float32, rotation=rotation)
    want = (shift.double() @ rotation.double().T).float()
    assert torch.equal(rotated, want)
    with pytest.raises(ValueError):
        runtime.load_key_shift(3, 5, 128, "cpu", torch.float32)
    monkeypatch.delenv(runtime.KEY_SHIFT_ENV)
    assert runtime.load_key_shift(3, 8, 128, "cpu", torch.float32) is None
