"""Build a vLLM engine on the NVFP4 KV-cache backend (src/nvfp4_vllm/engine.py:14-95 of
OpenBitSys/BitDecoding-FP4)."""

from __future__ import annotations

import os
from typing import Any

from .guards import DEFAULT_SLOTS

PAGE_SIZE = 128
KEY_SHIFT_ENV = "NVFP4_KEY_SHIFT"
REQUIRED_ENGINE_KWARGS: dict[str, Any] = {
    "kv_cache_dtype": "nvfp4",
    "attention_config": {"backend": "CUSTOM"},
    "block_size": PAGE_SIZE,
    "enable_prefix_caching": False,
    "enable_chunked_prefill": False,
}


def engine_kwargs(model: str, *, additional_config: dict[str, Any] | None = None, **kwargs: Any) -> dict[str, Any]:
    """The keyword arguments ``build_llm`` hands to ``vllm.LLM``. ``additional_config`` carries the
    backend options (``nvfp4_scale_mode``, ``nvfp4_query_terms``, ``nvfp4_rotation``,
    ``nvfp4_key_scale_geometry``) and ``nvfp4_key_smoothing``: ``"auto"`` (the default: measure the
    key mean before serving), a sidecar path, or None for no smoothing. A keyword that contradicts
    a required engine setting is refused: an engine holding only some of them still starts, and
    serves from a different cache."""
    additional = dict(additional_config or {})
    smoothing = additional.setdefault("nvfp4_key_smoothing", "auto")
    if smoothing is not None:
        smoothing = os.fsdecode(smoothing)
    additional["nvfp4_key_smoothing"] = smoothing
    contradicted = {name: kwargs[name] for name, required in REQUIRED_ENGINE_KWARGS.items()
                    if name in kwargs and kwargs[name] != required}
    if contradicted:
        wanted = {name: REQUIRED_ENGINE_KWARGS[name] for name in contradicted}
        raise ValueError(
            f"this backend requires {wanted}, and was given {contradicted}; "
            "an engine holding only some of these settings still starts, and "
            "serves from a different cache"
        )
    engine = {**REQUIRED_ENGINE_KWARGS, **kwargs, "model": model, "additional_config": additional}
    engine.setdefault("max_num_seqs", DEFAULT_SLOTS)
    if engine.get("max_model_len") is not None:
        engine.setdefault("max_num_batched_tokens", max(engine["max_model_len"], engine["max_num_seqs"]))
    # the worker extension carries the calibration RPCs and the smoothing toggle
    from .calibrate import WORKER_EXTENSION_CLS

    supplied = engine.get("worker_extension_cls")
    if supplied is None:
        engine["worker_extension_cls"] = WORKER_EXTENSION_CLS
    elif smoothing == "auto" and supplied != WORKER_EXTENSION_CLS:
        raise ValueError(
            f"calibrating key smoothing needs worker_extension_cls={WORKER_EXTENSION_CLS!r}, and vLLM "
            "accepts one; either pass a sidecar path instead or mix that class into your own"
        )
    return engine


def build_llm(model: str, *, additional_config: dict[str, Any] | None = None, **kwargs: Any):
    """Register the backend, force the engine settings it needs and construct ``vllm.LLM``."""
    engine = engine_kwargs(model, additional_config=additional_config, **kwargs)
    from . import register as register_custom_backend

    register_custom_backend()
    os.environ.setdefault("VLLM_WORKER_MULTIPROC_METHOD", "spawn")
    smoothing = engine["additional_config"]["nvfp4_key_smoothing"]
    if smoothing is None or smoothing == "auto":
        os.environ.pop(KEY_SHIFT_ENV, None)  # workers read the sidecar path while the engine is built
    else:
        os.environ[KEY_SHIFT_ENV] = smoothing
    from vllm import LLM

    llm = LLM(**engine)
    if smoothing == "auto":
        from .calibrate import calibrate_key_shift

        if calibrate_key_shift(llm) is None:
            raise RuntimeError("the engine came up without the NVFP4 cache, so there was no K mean to measure")
    return llm
