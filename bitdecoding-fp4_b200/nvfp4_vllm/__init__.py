"""Out-of-tree NVFP4 KV-cache attention backend for vLLM V1, served by libbdfp4.

Drop-in for the ``nvfp4_vllm`` package of OpenBitSys/BitDecoding-FP4
(src/nvfp4_vllm/__init__.py:4-47): same entry point (``vllm.general_plugins`` →
``nvfp4_vllm:register``), same backend, builder, impl and metadata class names.
"""


def register() -> None:
    """Entry point of the ``vllm.general_plugins`` group: claim the CUSTOM backend slot."""
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend

    register_backend(AttentionBackendEnum.CUSTOM, "nvfp4_vllm.backend.NVFP4Backend")


def build_llm(model, **kwargs):
    """See :func:`nvfp4_vllm.engine.build_llm` (imported lazily: ``register`` must stay light)."""
    from .engine import build_llm as _build

    return _build(model, **kwargs)


def calibrate_key_smoothing(llm, **kwargs):
    """Calibrate static key smoothing, optionally fitting the probability threshold
    (:func:`nvfp4_vllm.calibrate.calibrate_key_shift`)."""
    from .calibrate import calibrate_key_shift as _calibrate

    return _calibrate(llm, **kwargs)


def set_key_smoothing_enabled(llm, enabled: bool):
    """Enable or disable an engine's calibrated static key smoothing between requests."""
    from .calibrate import set_key_shift_enabled as _set

    return _set(llm, enabled)


__all__ = ["register", "build_llm", "calibrate_key_smoothing", "set_key_smoothing_enabled"]
