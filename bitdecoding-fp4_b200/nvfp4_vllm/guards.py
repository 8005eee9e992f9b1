"""Engine configurations the NVFP4 KV-cache path refuses to run under.

Same names and refusals as src/nvfp4_vllm/guards.py of OpenBitSys/BitDecoding-FP4. The checks
run from ``NVFP4Impl.__init__`` (once per layer per engine) because vLLM memoizes backend
validation on a key that carries none of these fields.
"""

from __future__ import annotations

from typing import NamedTuple

from nvfp4_decode_kernel.scale_mode import DEFAULT_SCALE_MODE, scale_format, scale_rule

from .control import MAX_SUPPORTED_SLOTS

NVFP4 = "nvfp4"
SCALE_MODE_KEY = "nvfp4_scale_mode"
KEY_SCALE_GEOMETRY_KEY = "nvfp4_key_scale_geometry"
KEY_SCALE_GEOMETRIES = ("local", "gaussian_global")
QUERY_TERMS_KEY = "nvfp4_query_terms"
ROTATION_KEY = "nvfp4_rotation"
ROTATIONS = ("none", "hadamard", "block_hadamard_64")
DEFAULT_SLOTS = 32
MAX_SLOTS = MAX_SUPPORTED_SLOTS


class UnsupportedConfigError(ValueError):
    """An engine configuration the NVFP4 path cannot serve correctly."""


class ScaleModes(NamedTuple):
    """One block-scale mode per quantized tensor."""

    key: str
    value: str
    query: str


def _additional(vllm_config) -> dict | None:
    additional = getattr(vllm_config, "additional_config", None) or {}
    return additional if isinstance(additional, dict) else None


def resolve_scale_mode(vllm_config) -> ScaleModes:
    """The block-scale modes of K, V and Q from ``additional_config["nvfp4_scale_mode"]``: a bare
    name for all three, or a mapping with exactly ``key``/``value``/``query``. Unknown names and a
    mix of NVFP4 and MXFP4 are refused here, before a model is loaded."""
    additional = _additional(vllm_config)
    if additional is None:
        return ScaleModes(*(DEFAULT_SCALE_MODE,) * 3)
    requested = additional.get(SCALE_MODE_KEY, DEFAULT_SCALE_MODE)
    if isinstance(requested, dict):
        if set(requested) != set(ScaleModes._fields):
            raise UnsupportedConfigError(
                f"additional_config[{SCALE_MODE_KEY!r}] as a mapping needs "
                f"exactly {sorted(ScaleModes._fields)}, got {sorted(requested)}"
            )
        modes = ScaleModes(**requested)
    else:
        modes = ScaleModes(*(requested,) * 3)
    for tensor, mode in zip(ScaleModes._fields, modes):
        try:
            scale_rule(mode)
        except (ValueError, TypeError) as error:
            raise UnsupportedConfigError(f"additional_config[{SCALE_MODE_KEY!r}] for {tensor}: {error}") from None
    formats = {scale_format(mode) for mode in modes}
    if len(formats) != 1:
        raise UnsupportedConfigError(
            f"additional_config[{SCALE_MODE_KEY!r}] mixes {sorted(formats)}; "
            "key, value and query must share one scale format"
        )
    return modes


def check_mxfp4_options(scale_modes: ScaleModes, *, key_scale_geometry: str) -> None:
    """Refuse the NVFP4-only cache options under an MXFP4 scale mode."""
    if scale_format(scale_modes.key) != "mxfp4":
        return
    if key_scale_geometry != "local":
        raise UnsupportedConfigError(f"MXFP4 scale modes do not support {[KEY_SCALE_GEOMETRY_KEY]} yet")


def _choice(vllm_config, key: str, default, allowed, describe: str):
    additional = _additional(vllm_config)
    if additional is None:
        return default
    requested = additional.get(key, default)
    if type(requested) is not type(default) or requested not in allowed:
        raise UnsupportedConfigError(f"additional_config[{key!r}] must be {describe}, got {requested!r}")
    return requested


def resolve_key_scale_geometry(vllm_config) -> str:
    return _choice(vllm_config, KEY_SCALE_GEOMETRY_KEY, "local", KEY_SCALE_GEOMETRIES,
                   f"one of {list(KEY_SCALE_GEOMETRIES)}")


def resolve_query_terms(vllm_config) -> int:
    return _choice(vllm_config, QUERY_TERMS_KEY, 1, (1, 2), "1 or 2")


def resolve_rotation(vllm_config) -> str:
    return _choice(vllm_config, ROTATION_KEY, "none", ROTATIONS, "'none', 'hadamard', or 'block_hadamard_64'")


def check_supported(vllm_config) -> None:
    """Raise unless the engine is configured for the NVFP4 KV-cache path; a no-op for any other
    ``kv_cache_dtype`` (the backend is then a FlashAttention pass-through)."""
    cache = vllm_config.cache_config
    if cache is None or cache.cache_dtype != NVFP4:
        return
    scheduler = vllm_config.scheduler_config
    parallel = vllm_config.parallel_config
    refusals = (
        (scheduler is not None and scheduler.max_num_seqs > MAX_SLOTS,
         lambda: f"max_num_seqs={scheduler.max_num_seqs} exceeds the {MAX_SLOTS} BF16 tail slots the NVFP4 "
                 f"path preallocates. Pass max_num_seqs<={MAX_SLOTS}, or use a BF16 KV cache."),
        (bool(cache.enable_prefix_caching),
         lambda: "prefix caching is not supported by the NVFP4 KV cache: a cache hit resumes a sequence "
                 "mid-page, and prefill over an FP4 prefix is not implemented. Pass enable_prefix_caching=False."),
        (scheduler is not None and bool(scheduler.enable_chunked_prefill),
         lambda: "chunked prefill is not supported by the NVFP4 KV cache: the second chunk of a split prompt "
                 "resumes mid-page, which needs prefill over an FP4 prefix. Pass enable_chunked_prefill=False; "
                 "vLLM then requires max_num_batched_tokens >= max_model_len so that no prompt has to be split."),
        (scheduler is not None and bool(getattr(scheduler, "long_prefill_token_threshold", 0)),
         lambda: f"long_prefill_token_threshold={scheduler.long_prefill_token_threshold} splits long prompts "
                 "even with chunked prefill disabled. Leave it at 0."),
        (vllm_config.speculative_config is not None,
         lambda: "speculative decoding is not supported by the NVFP4 KV cache: it verifies several draft tokens "
                 "per step, and the decode kernel attends one query token per sequence."),
        (bool(getattr(cache, "kv_cache_dtype_skip_layers", None)),
         lambda: f"kv_cache_dtype_skip_layers={cache.kv_cache_dtype_skip_layers} leaves some layers on a "
                 "different cache dtype, which splits the model into KV cache groups with their own metadata "
                 "builders, so the slot table would advance more than once per step. Leave it empty."),
        (getattr(cache, "kv_offloading_size", None) is not None,
         lambda: "KV offloading is not supported by the NVFP4 KV cache: it copies pages by address and size, "
                 "which does not describe the packed FP4 layout. Leave kv_offloading_size unset."),
        (parallel is not None and bool(getattr(parallel, "use_ubatching", False)),
         lambda: "microbatching is not supported by the NVFP4 KV cache: each ubatch builds its own attention "
                 "metadata, so the slot table would advance twice per step. Leave enable_dbo unset and "
                 "ubatch_size at 0."),
        (parallel is not None and parallel.pipeline_parallel_size > 1,
         lambda: f"pipeline_parallel_size={parallel.pipeline_parallel_size} is not supported by the NVFP4 KV "
                 "cache: page promotion is driven from the last attention layer, which a pipeline stage does "
                 "not own. Pass pipeline_parallel_size=1."),
    )
    for refused, message in refusals:
        if refused:
            raise UnsupportedConfigError(message())


def check_layer_supported(impl) -> None:
    """Raise unless this attention layer is one the decode kernel can serve: a decoder layer with
    head size 128 and none of the score modifiers the kernel does not implement (a silently wrong
    mask is the failure worth a check)."""
    from vllm.v1.attention.backend import AttentionType

    problems = (
        (impl.attn_type != AttentionType.DECODER, f"attention type {impl.attn_type}"),
        (getattr(impl, "head_size", 128) != 128, f"head_size {getattr(impl, 'head_size', None)}"),
        (getattr(impl, "alibi_slopes", None) is not None, "ALiBi slopes"),
        (getattr(impl, "sliding_window", (-1, -1)) not in ((-1, -1), None), "a sliding window"),
        (bool(getattr(impl, "logits_soft_cap", 0)), "a logits soft cap"),
        (getattr(impl, "sinks", None) is not None, "learnable attention sinks"),
        (getattr(impl, "kv_sharing_target_layer_name", None) is not None, "cross-layer KV sharing"),
    )
    for refused, what in problems:
        if refused:
            raise UnsupportedConfigError(f"{what} is not supported by the NVFP4 attention path")
