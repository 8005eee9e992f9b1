"""Calibrate static key smoothing, and optionally the probability threshold, before serving
(src/nvfp4_vllm/calibrate.py of OpenBitSys/BitDecoding-FP4).

Text the model itself generates is tiled across the context window, so that post-RoPE keys are
sampled at representative positions; subtracting their per-(layer, head, channel) mean lowers the
quantization error of K and leaves softmax unchanged. The measurement runs inside each worker
(named ``collective_rpc`` methods), which also writes the sidecar, so no tensor travels through
the engine client. It must finish before serving: every cached key has to see the same mean.
"""

from __future__ import annotations

from collections import Counter
from typing import Any

import torch

# vLLM mixes this class into its worker; an engine that is to calibrate is built with
# worker_extension_cls="nvfp4_vllm.calibrate.NVFP4WorkerExtension" (build_llm does).
WORKER_EXTENSION_CLS = "nvfp4_vllm.calibrate.NVFP4WorkerExtension"

# Short, varied instructions; the model's own continuations of them are what gets tiled.
SEEDS = (
    "Explain to a new engineer how a B-tree keeps its height small as rows are inserted.",
    "Give a plain account of why the Roman republic gave way to rule by emperors.",
    "Tell a short story about a night-shift baker who finds a letter in a sack of flour.",
    "Show, step by step, why the sum of the first n odd numbers is n squared.",
    "Describe how a vaccine trains the immune system, for a curious teenager.",
    "Contrast row-oriented and column-oriented storage for analytical queries.",
    "Explain the cost of skipping code review to someone who manages a budget, not a codebase.",
    "Outline how you would find the cause of a memory leak that appears only after days of uptime.",
)
TOKENS_PER_SEED = 256
CONTEXT_TOKENS = 32_768  # positions the calibration prompt spans, clamped to the engine's window


def _runtimes(model: torch.nn.Module) -> list[Any]:
    """The distinct ``LayerRuntime`` objects the model's NVFP4 attention layers share."""
    from .impl import NVFP4Impl

    found: list[Any] = []
    for module in model.modules():
        impl = getattr(module, "impl", None)
        runtime = getattr(impl, "runtime", None)
        if isinstance(impl, NVFP4Impl) and runtime is not None and all(runtime is not other for other in found):
            found.append(runtime)
    return found


class NVFP4WorkerExtension:
    """Named RPC methods for calibration and cache inspection; workers keep the tensors and return
    summaries."""

    def nvfp4_layer_cache_contract(self) -> dict[str, dict[str, int]]:
        """What every loaded attention layer reports as its cache dtype and backend."""
        dtypes, backends = Counter(), Counter()
        for module in self.get_model().modules():
            dtype = getattr(module, "kv_cache_dtype", None)
            backend = getattr(module, "attn_backend", None)
            if dtype is None or backend is None:
                continue
            dtypes[str(dtype)] += 1
            backends[str(backend.get_name())] += 1
        return {"layer_cache_dtype_counts": dict(dtypes), "layer_attention_backend_counts": dict(backends)}

    def nvfp4_key_shift_is_active(self) -> bool:
        return all(runtime.active_key_shift is not None for runtime in _runtimes(self.get_model()))

    def nvfp4_set_key_shift_enabled(self, enabled: bool) -> int:
        runtimes = _runtimes(self.get_model())
        for runtime in runtimes:
            runtime.set_key_shift_enabled(enabled)
        return len(runtimes)

    def nvfp4_begin_key_shift_measurement(self) -> int:
        runtimes = _runtimes(self.get_model())
        for runtime in runtimes:
            runtime.begin_key_shift_measurement()
        return len(runtimes)

    def nvfp4_begin_probability_calibration(self, tokens: int, multiplier: float, samples: int) -> None:
        from .probability_calibration import ProbabilityCalibration

        if hasattr(self, "_probability_calibration"):
            raise RuntimeError("probability calibration is already active")
        collector = ProbabilityCalibration(tokens, multiplier, samples)
        collector.install(self.get_model())
        self._probability_calibration = collector

    def nvfp4_end_probability_calibration(self, complete: bool = True) -> list[dict] | None:
        collector = self._probability_calibration
        try:
            return collector.finish() if complete else None
        finally:
            collector.close()
            del self._probability_calibration

    def nvfp4_finish_key_shift_measurement(self, save_to: str | None = None) -> dict[str, Any] | None:
        runtimes = _runtimes(self.get_model())
        if not runtimes:
            return None
        tokens = runtimes[0].key_shift_tokens
        shift = runtimes[0].finish_key_shift_measurement()
        for other in runtimes[1:]:
            other.finish_key_shift_measurement()
        if save_to is not None:
            shift, writes = self._gather_for_export(shift, tokens)
            if writes:
                from safetensors.torch import save_file

                save_file({"key_shift": shift.cpu()}, save_to,
                          metadata={"schema": "1", "source": "calibrate_key_shift"})
        return {"tokens": int(tokens), "shape": list(shift.shape), "mean_abs": float(shift.abs().mean()),
                "saved_to": save_to}

    def _gather_for_export(self, shift: torch.Tensor, tokens: int) -> tuple[torch.Tensor, bool]:
        """The full-model mean (KV heads of all tensor-parallel ranks, in rank order) and whether
        this worker writes the sidecar: rank 0 of the group, or the only worker."""
        if not torch.distributed.is_initialized():
            return shift, True
        from vllm.distributed import get_tp_group

        group = get_tp_group()
        if group.world_size == 1:
            return shift, True
        total_heads = self.vllm_config.model_config.get_total_num_kv_heads()
        if total_heads != shift.shape[1] * group.world_size:
            raise ValueError("key-shift export requires unreplicated, evenly partitioned KV heads")
        counts = group.all_gather(torch.tensor([tokens], dtype=torch.int64, device=shift.device), dim=0)
        if not bool((counts == tokens).all()):
            raise ValueError("TP workers disagree on key-shift measurement token counts")
        # original-basis means, KV heads contiguous in rank order: what the loader slices again
        return group.all_gather(shift, dim=1), group.rank_in_group == 0


def set_key_shift_enabled(llm, enabled: bool) -> bool:
    """Turn the loaded or measured shift on or off between requests (the vector survives being
    off, so one engine can answer both ways). Safe only while no request is cached: keys already
    stored keep the setting they were written under. Returns whether any worker had a runtime."""
    switched = llm.collective_rpc("nvfp4_set_key_shift_enabled", args=(enabled,))
    llm.reset_prefix_cache()
    return any(switched)


def _long_prompt(llm, texts: list[str], context_tokens: int) -> list[int]:
    """About ``context_tokens`` token ids: ``texts`` joined and tiled. Repetition is fine for a
    mean; the point of the length is to visit high positions."""
    if not any(text.strip() for text in texts):
        raise ValueError(
            "the model returned no calibration text to tile, so the mean would be measured over separators"
        )
    unit = llm.get_tokenizer().encode("\n\n".join(texts) + "\n\n", add_special_tokens=False)
    repeats = -(-context_tokens // len(unit))
    return (unit * repeats)[:context_tokens]


def calibrate_key_shift(llm, *, seeds: tuple[str, ...] = SEEDS, tokens_per_seed: int = TOKENS_PER_SEED,
                        context_tokens: int = CONTEXT_TOKENS, save_to: str | None = None,
                        probability_multiplier: float | None = None,
                        probability_samples: int = 8) -> dict[str, Any] | None:
    """Measure the key mean over one long prefill and start subtracting it.

    Returns the measurement summary (token count, shape, mean magnitude, sidecar path), or None
    when the engine runs no NVFP4 cache. ``save_to`` writes a sidecar reusable through
    ``additional_config["nvfp4_key_smoothing"]``: it needs one tensor-parallel group with evenly
    partitioned, unreplicated KV heads and no pipeline or data parallelism; rank 0 writes the
    gathered full-model tensor. With ``probability_multiplier`` the same prefill also yields the
    probability threshold (``probability_scaling`` in the result); that needs an eager engine so
    that the attention hooks run."""
    from vllm import SamplingParams, TokensPrompt

    if probability_multiplier is not None and not llm.llm_engine.vllm_config.model_config.enforce_eager:
        raise ValueError("probability calibration requires an eager engine")
    try:
        found = llm.collective_rpc("nvfp4_begin_key_shift_measurement")
    except AttributeError as error:
        raise RuntimeError(
            f'the engine was built without worker_extension_cls="{WORKER_EXTENSION_CLS}", '
            "so the K mean cannot be read out of the worker"
        ) from error
    if not any(found):
        return None
    if save_to is not None:
        config = llm.llm_engine.vllm_config
        parallel = config.parallel_config
        ranks = parallel.tensor_parallel_size
        heads = config.model_config.get_total_num_kv_heads()
        if (not all(found) or len(found) != ranks or parallel.pipeline_parallel_size != 1
                or parallel.data_parallel_size != 1 or heads < ranks or heads % ranks):
            raise ValueError(
                "key-shift export requires one TP group with unreplicated, "
                "evenly partitioned KV heads and no pipeline/data parallelism"
            )
    sampled = llm.generate(list(seeds),
                           SamplingParams(temperature=0.0, top_p=1.0, max_tokens=tokens_per_seed, seed=42),
                           use_tqdm=False)
    budget = min(context_tokens, llm.llm_engine.model_config.max_model_len - 1)
    if probability_multiplier is not None:
        llm.collective_rpc("nvfp4_begin_probability_calibration",
                           args=(budget, probability_multiplier, probability_samples))
    try:
        texts = [output.prompt + output.outputs[0].text for output in sampled]
        llm.generate(TokensPrompt(prompt_token_ids=_long_prompt(llm, texts, budget)),
                     SamplingParams(temperature=0.0, max_tokens=1), use_tqdm=False)
    except BaseException:
        if probability_multiplier is not None:
            llm.collective_rpc("nvfp4_end_probability_calibration", args=(False,))
        raise
    report = None
    if probability_multiplier is not None:
        from .probability_calibration import fit_probability_threshold

        samples = llm.collective_rpc("nvfp4_end_probability_calibration")
        positions = [row["position"] for row in samples[0]]
        if len(samples) != len(found) or any([row["position"] for row in worker] != positions for worker in samples):
            raise ValueError("TP workers disagree on probability calibration samples")
        report = fit_probability_threshold(samples, probability_multiplier)
    measurements = llm.collective_rpc("nvfp4_finish_key_shift_measurement", args=(save_to,))
    measured = measurements[0]
    if save_to is not None and len(found) > 1:
        if len(measurements) != len(found) or any(
            item is None or item["shape"] != measured["shape"] or item["tokens"] != measured["tokens"]
            or item["saved_to"] != save_to for item in measurements
        ):
            raise ValueError("TP workers disagree on the exported key-shift measurement")
    if report is not None:
        measured = {**measured, "probability_scaling": report}
    # keys cached during the measurement were stored unshifted; no later request may read one
    llm.reset_prefix_cache()
    return measured
