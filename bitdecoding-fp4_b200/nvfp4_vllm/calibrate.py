"""Measuring what the cache's quantizer is calibrated with: the key-smoothing mean and, optionally,
the probability threshold tau. Both come out of ONE long prefill that runs before serving.

Why a prefill of the model's own text: the key mean is taken after RoPE, so it depends on position,
and a prompt that spans the context window visits the positions serving will see. Eight short
instructions are completed by the model, the completions are tiled up to the window, and that prompt
is prefilled once while every attention layer adds its keys to an FP64 sum on the GPU
(``bdfp4_key_channel_sums``). Subtracting the resulting per-(layer, head, channel) mean from every
key leaves softmax unchanged (a constant per query) and lowers K's quantization error.

Who does what. The driver process (:func:`calibrate_key_shift`) only sequences the steps and checks
that the workers agree; the tensors never leave the workers. Each worker exposes the steps as named
methods (:class:`NVFP4WorkerExtension`, mixed into vLLM's worker through ``worker_extension_cls``),
and the worker that is rank 0 of its tensor-parallel group writes the sidecar.

Drop-in surface, kept from src/nvfp4_vllm/calibrate.py of OpenBitSys/BitDecoding-FP4:
``WORKER_EXTENSION_CLS``, the ``nvfp4_*`` method names and their return values,
``calibrate_key_shift`` / ``set_key_shift_enabled`` and the keys of the summary they return.
"""

from __future__ import annotations

from collections import Counter
from dataclasses import dataclass
from typing import Any, Iterator

import torch

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


# ---------------------------------------------------------------------------------------------
# worker side
# ---------------------------------------------------------------------------------------------

def _layer_runtimes(model: torch.nn.Module) -> Iterator[Any]:
    """Each ``LayerRuntime`` behind the model's NVFP4 attention layers, once (layers share them)."""
    from .impl import NVFP4Impl

    yielded: set[int] = set()
    for module in model.modules():
        impl = getattr(module, "impl", None)
        runtime = getattr(impl, "runtime", None) if isinstance(impl, NVFP4Impl) else None
        if runtime is not None and id(runtime) not in yielded:
            yielded.add(id(runtime))
            yield runtime


def _whole_model_shift(shift: torch.Tensor, tokens: int, total_kv_heads: int) -> tuple[torch.Tensor, bool]:
    """(the mean over all KV heads of the model, whether this worker is the one that writes it).

    A tensor-parallel worker holds a contiguous slice of the KV heads. The sidecar stores the model's
    heads in their original order, which is the ranks' slices side by side, and the loader cuts the
    same slices out again; so the export is an all-gather along the head axis, written by rank 0.
    Ranks must have measured the same tokens, or the slices would be means of different things."""
    if not torch.distributed.is_initialized():
        return shift, True
    from vllm.distributed import get_tp_group

    group = get_tp_group()
    if group.world_size == 1:
        return shift, True
    if shift.shape[1] * group.world_size != total_kv_heads:
        raise ValueError("key-shift export requires unreplicated, evenly partitioned KV heads")
    seen = group.all_gather(torch.tensor([tokens], dtype=torch.int64, device=shift.device), dim=0)
    if int(seen.min()) != tokens or int(seen.max()) != tokens:
        raise ValueError("TP workers disagree on key-shift measurement token counts")
    return group.all_gather(shift, dim=1), group.rank_in_group == 0


class NVFP4WorkerExtension:
    """The calibration steps as worker methods. A method acts on every runtime of the worker's model
    and returns something small: a count, a flag or a summary."""

    # -- inspection ---------------------------------------------------------------------------
    def nvfp4_layer_cache_contract(self) -> dict[str, dict[str, int]]:
        """Histogram of the cache dtype and attention backend the loaded layers report."""
        dtypes: Counter = Counter()
        backends: Counter = Counter()
        for module in self.get_model().modules():
            if hasattr(module, "kv_cache_dtype") and hasattr(module, "attn_backend"):
                dtype, backend = module.kv_cache_dtype, module.attn_backend
                if dtype is not None and backend is not None:
                    dtypes[str(dtype)] += 1
                    backends[str(backend.get_name())] += 1
        return {"layer_cache_dtype_counts": dict(dtypes), "layer_attention_backend_counts": dict(backends)}

    def nvfp4_key_shift_is_active(self) -> bool:
        return all(runtime.active_key_shift is not None for runtime in _layer_runtimes(self.get_model()))

    # -- key smoothing ------------------------------------------------------------------------
    def _for_each_runtime(self, action) -> int:
        count = 0
        for runtime in _layer_runtimes(self.get_model()):
            action(runtime)
            count += 1
        return count

    def nvfp4_set_key_shift_enabled(self, enabled: bool) -> int:
        return self._for_each_runtime(lambda runtime: runtime.set_key_shift_enabled(enabled))

    def nvfp4_begin_key_shift_measurement(self) -> int:
        return self._for_each_runtime(lambda runtime: runtime.begin_key_shift_measurement())

    def nvfp4_finish_key_shift_measurement(self, save_to: str | None = None) -> dict[str, Any] | None:
        """Close the measurement on every runtime, switch the mean on, optionally write the sidecar.
        Returns None on a worker whose model has no NVFP4 layer."""
        runtimes = list(_layer_runtimes(self.get_model()))
        if not runtimes:
            return None
        tokens = int(runtimes[0].key_shift_tokens)
        shifts = [runtime.finish_key_shift_measurement() for runtime in runtimes]
        shift = shifts[0]
        if save_to is not None:
            total_heads = self.vllm_config.model_config.get_total_num_kv_heads()
            shift, is_writer = _whole_model_shift(shift, tokens, total_heads)
            if is_writer:
                from safetensors.torch import save_file

                save_file({"key_shift": shift.cpu()}, save_to, metadata={"schema": "1", "source": "calibrate_key_shift"})
        return {"tokens": tokens, "shape": list(shift.shape), "mean_abs": float(shift.abs().mean()),
                "saved_to": save_to}

    # -- probability threshold ----------------------------------------------------------------
    def nvfp4_begin_probability_calibration(self, tokens: int, multiplier: float, samples: int) -> None:
        from .probability_calibration import ProbabilityCalibration

        if getattr(self, "_probability_calibration", None) is not None:
            raise RuntimeError("probability calibration is already active")
        collector = ProbabilityCalibration(tokens, multiplier, samples)
        collector.install(self.get_model())
        self._probability_calibration = collector

    def nvfp4_end_probability_calibration(self, complete: bool = True) -> list[dict] | None:
        """Unhook the collector; hand back its samples unless the prefill was abandoned."""
        collector, self._probability_calibration = self._probability_calibration, None
        try:
            return collector.finish() if complete else None
        finally:
            collector.close()


# ---------------------------------------------------------------------------------------------
# driver side
# ---------------------------------------------------------------------------------------------

def set_key_shift_enabled(llm, enabled: bool) -> bool:
    """Switch the loaded or measured mean on or off between requests; the vector itself is kept, so
    one engine can answer both ways. Only safe while nothing is cached (stored keys keep the setting
    they were written under), hence the prefix-cache reset. True if any worker had a runtime."""
    touched = llm.collective_rpc("nvfp4_set_key_shift_enabled", args=(enabled,))
    llm.reset_prefix_cache()
    return any(touched)


@dataclass
class _Engine:
    """The handful of engine facts the calibration reads, gathered in one place."""

    llm: Any

    @property
    def config(self):
        return self.llm.llm_engine.vllm_config

    def window(self) -> int:
        return self.llm.llm_engine.model_config.max_model_len - 1

    def eager(self) -> bool:
        return bool(self.config.model_config.enforce_eager)

    def check_exportable(self, runtimes_per_worker: list[int]) -> None:
        """A sidecar holds the whole model's KV heads in order; only a single tensor-parallel group
        whose ranks each own an equal, unreplicated share can reassemble that."""
        parallel = self.config.parallel_config
        ranks = parallel.tensor_parallel_size
        heads = self.config.model_config.get_total_num_kv_heads()
        single_group = parallel.pipeline_parallel_size == 1 and parallel.data_parallel_size == 1
        every_worker = len(runtimes_per_worker) == ranks and all(runtimes_per_worker)
        if not (single_group and every_worker and heads >= ranks and heads % ranks == 0):
            raise ValueError(
                "key-shift export requires one TP group with unreplicated, "
                "evenly partitioned KV heads and no pipeline/data parallelism")


def _tiled_prompt(tokenizer, texts: list[str], length: int) -> list[int]:
    """``length`` token ids made of ``texts`` joined by blank lines and repeated. Repetition does not
    hurt a mean; the length is what matters, because it decides which positions are visited."""
    if not any(text.strip() for text in texts):
        raise ValueError(
            "the model returned no calibration text to tile, so the mean would be measured over separators")
    unit = tokenizer.encode("\n\n".join(texts) + "\n\n", add_special_tokens=False)
    copies = (length + len(unit) - 1) // len(unit)
    return (unit * copies)[:length]


def _agreeing(items: list, what: str, key=lambda item: item):
    """All workers must report the same thing; returns it."""
    first = key(items[0])
    if any(key(item) != first for item in items[1:]):
        raise ValueError(f"TP workers disagree on {what}")
    return first


def calibrate_key_shift(llm, *, seeds: tuple[str, ...] = SEEDS, tokens_per_seed: int = TOKENS_PER_SEED,
                        context_tokens: int = CONTEXT_TOKENS, save_to: str | None = None,
                        probability_multiplier: float | None = None,
                        probability_samples: int = 8) -> dict[str, Any] | None:
    """Measure the key mean over one long prefill and start subtracting it.

    Returns rank 0's summary ``{"tokens", "shape", "mean_abs", "saved_to"}`` (plus
    ``"probability_scaling"``, the tau report, when ``probability_multiplier`` is given), or None when
    the engine runs no NVFP4 cache. ``save_to`` writes a sidecar that
    ``additional_config["nvfp4_key_smoothing"]`` loads again. Tau needs an eager engine: its collector
    is a forward hook, which a captured graph would not run."""
    from vllm import SamplingParams, TokensPrompt

    engine = _Engine(llm)
    wants_tau = probability_multiplier is not None
    if wants_tau and not engine.eager():
        raise ValueError("probability calibration requires an eager engine")
    try:
        runtimes = llm.collective_rpc("nvfp4_begin_key_shift_measurement")
    except AttributeError as error:
        raise RuntimeError(
            f'the engine was built without worker_extension_cls="{WORKER_EXTENSION_CLS}", '
            "so the K mean cannot be read out of the worker") from error
    if not any(runtimes):
        return None
    if save_to is not None:
        engine.check_exportable(runtimes)

    greedy = dict(temperature=0.0, top_p=1.0, seed=42)
    completions = llm.generate(list(seeds), SamplingParams(max_tokens=tokens_per_seed, **greedy), use_tqdm=False)
    texts = [item.prompt + item.outputs[0].text for item in completions]
    length = min(context_tokens, engine.window())
    prompt = _tiled_prompt(llm.get_tokenizer(), texts, length)

    if wants_tau:
        llm.collective_rpc("nvfp4_begin_probability_calibration",
                           args=(length, probability_multiplier, probability_samples))
    try:
        llm.generate(TokensPrompt(prompt_token_ids=prompt), SamplingParams(temperature=0.0, max_tokens=1),
                     use_tqdm=False)
    except BaseException:
        if wants_tau:  # leave no hook behind
            llm.collective_rpc("nvfp4_end_probability_calibration", args=(False,))
        raise

    tau_report = None
    if wants_tau:
        from .probability_calibration import fit_probability_threshold

        per_worker = llm.collective_rpc("nvfp4_end_probability_calibration")
        if len(per_worker) != len(runtimes):
            raise ValueError("TP workers disagree on probability calibration samples")
        _agreeing(per_worker, "probability calibration samples", key=lambda rows: [row["position"] for row in rows])
        tau_report = fit_probability_threshold(per_worker, probability_multiplier)

    summaries = llm.collective_rpc("nvfp4_finish_key_shift_measurement", args=(save_to,))
    summary = summaries[0]
    if save_to is not None and len(runtimes) > 1:
        if len(summaries) != len(runtimes) or any(item is None for item in summaries):
            raise ValueError("TP workers disagree on the exported key-shift measurement")
        _agreeing(summaries, "the exported key-shift measurement",
                  key=lambda item: (item["shape"], item["tokens"], item["saved_to"]))
    if tau_report is not None:
        summary = dict(summary, probability_scaling=tau_report)
    # keys cached while measuring were stored unshifted; nothing served later may read one of them
    llm.reset_prefix_cache()
    return summary
