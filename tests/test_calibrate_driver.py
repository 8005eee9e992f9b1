"""The calibration driver (nvfp4_vllm.calibrate) against stand-ins for the engine and its workers:
the order of the steps, what the workers are asked, what the driver refuses, and that no hook or
measurement is left behind when the prefill fails. No GPU and no model; vLLM is imported for its
parameter types only."""

import types

import pytest
import torch

pytest.importorskip("vllm")


class FakeRuntime:
    def __init__(self, layers=2, heads=2):
        self.measuring = False
        self.enabled = True
        self.key_shift_tokens = 0
        self.active_key_shift = None
        self.shift = torch.arange(layers * heads * 128, dtype=torch.float32).reshape(layers, heads, 128) / 100

    def begin_key_shift_measurement(self):
        self.measuring, self.key_shift_tokens = True, 0

    def finish_key_shift_measurement(self):
        assert self.measuring
        self.measuring, self.active_key_shift = False, self.shift
        return self.shift

    def set_key_shift_enabled(self, enabled):
        self.enabled = enabled


def make_worker(runtime, total_heads=2):
    from nvfp4_vllm.calibrate import NVFP4WorkerExtension
    from nvfp4_vllm.impl import NVFP4Impl

    model = torch.nn.Module()
    for index in range(3):  # three layers sharing one runtime
        layer = torch.nn.Module()
        layer.impl = NVFP4Impl.__new__(NVFP4Impl)
        layer.impl.runtime = runtime
        model.add_module(f"layer{index}", layer)

    class Worker(NVFP4WorkerExtension):
        def get_model(self):
            return model

    worker = Worker()
    worker.vllm_config = types.SimpleNamespace(
        model_config=types.SimpleNamespace(get_total_num_kv_heads=lambda: total_heads))
    return worker


class FakeLLM:
    def __init__(self, workers, runtimes, eager=True, window=4096, tp=1, fail_prefill=False, text="some words"):
        self.workers, self.runtimes, self.calls, self.prefills = workers, runtimes, [], []
        self.fail_prefill, self.text, self.resets = fail_prefill, text, 0
        model_config = types.SimpleNamespace(enforce_eager=eager, max_model_len=window,
                                             get_total_num_kv_heads=lambda: 2)
        parallel = types.SimpleNamespace(tensor_parallel_size=tp, pipeline_parallel_size=1, data_parallel_size=1)
        self.llm_engine = types.SimpleNamespace(
            vllm_config=types.SimpleNamespace(model_config=model_config, parallel_config=parallel),
            model_config=model_config)

    def collective_rpc(self, name, args=()):
        self.calls.append(name)
        return [getattr(worker, name)(*args) for worker in self.workers]

    def get_tokenizer(self):
        return types.SimpleNamespace(encode=lambda text, add_special_tokens=False: [ord(c) % 251 for c in text])

    def generate(self, prompts, params, use_tqdm=False):
        if isinstance(prompts, list):
            return [types.SimpleNamespace(prompt=p, outputs=[types.SimpleNamespace(text=self.text)]) for p in prompts]
        if self.fail_prefill:
            raise RuntimeError("prefill failed")
        ids = prompts["prompt_token_ids"]
        self.prefills.append(len(ids))
        for runtime in self.runtimes:
            assert runtime.measuring  # the long prefill runs while the workers are measuring
            runtime.key_shift_tokens += len(ids)
        return []

    def reset_prefix_cache(self):
        self.resets += 1


def test_measurement_sequence_and_summary(tmp_path):
    from nvfp4_vllm.calibrate import calibrate_key_shift, set_key_shift_enabled

    runtime = FakeRuntime()
    llm = FakeLLM([make_worker(runtime)], [runtime], window=1000)
    sidecar = tmp_path / "shift.safetensors"
    summary = calibrate_key_shift(llm, context_tokens=5000, save_to=str(sidecar))
    assert llm.calls == ["nvfp4_begin_key_shift_measurement", "nvfp4_finish_key_shift_measurement"]
    assert llm.prefills == [999]  # clamped to the engine's window
    assert summary["tokens"] == 999 and summary["shape"] == [2, 2, 128] and summary["saved_to"] == str(sidecar)
    assert summary["mean_abs"] == pytest.approx(float(runtime.shift.abs().mean()))
    assert runtime.active_key_shift is not None and llm.resets == 1
    from safetensors.torch import load_file

    assert torch.equal(load_file(str(sidecar))["key_shift"], runtime.shift)
    assert set_key_shift_enabled(llm, False) is True and runtime.enabled is False and llm.resets == 2
    assert llm.workers[0].nvfp4_key_shift_is_active() is True


def test_no_nvfp4_layers_means_nothing_to_do():
    from nvfp4_vllm.calibrate import NVFP4WorkerExtension, calibrate_key_shift

    class Bare(NVFP4WorkerExtension):
        def get_model(self):
            return torch.nn.Linear(2, 2)

    llm = FakeLLM([Bare()], [])
    assert calibrate_key_shift(llm) is None
    assert llm.calls == ["nvfp4_begin_key_shift_measurement"] and llm.prefills == []


def test_refusals():
    from nvfp4_vllm.calibrate import WORKER_EXTENSION_CLS, calibrate_key_shift

    runtime = FakeRuntime()
    worker = make_worker(runtime)
    with pytest.raises(ValueError, match="eager"):
        calibrate_key_shift(FakeLLM([worker], [runtime], eager=False), probability_multiplier=8.0)
    # an engine built without the worker extension has none of the methods
    plain = FakeLLM([object()], [])
    with pytest.raises(RuntimeError, match=WORKER_EXTENSION_CLS.rsplit(".", 1)[1]):
        calibrate_key_shift(plain)
    # export needs every rank of one TP group to hold an equal share of the KV heads
    with pytest.raises(ValueError, match="TP group"):
        calibrate_key_shift(FakeLLM([worker], [runtime], tp=2), save_to="/tmp/never-written.safetensors")
    with pytest.raises(ValueError, match="no calibration text"):
        calibrate_key_shift(FakeLLM([worker], [runtime], text="   "), seeds=("", ""))


def test_failed_prefill_leaves_no_hook_behind(monkeypatch):
    from nvfp4_vllm import calibrate

    runtime = FakeRuntime()
    worker = make_worker(runtime)
    events = []

    class Collector:
        def __init__(self, tokens, multiplier, samples):
            events.append(("made", tokens, multiplier, samples))

        def install(self, model):
            events.append("installed")

        def finish(self):
            events.append("finished")
            return [{"position": 128, "codes": {}}]

        def close(self):
            events.append("closed")

    import nvfp4_vllm.probability_calibration as pc

    monkeypatch.setattr(pc, "ProbabilityCalibration", Collector)
    llm = FakeLLM([worker], [runtime], fail_prefill=True, window=2000)
    with pytest.raises(RuntimeError, match="prefill failed"):
        calibrate.calibrate_key_shift(llm, probability_multiplier=8.0, probability_samples=3)
    assert events == [("made", 1999, 8.0, 3), "installed", "closed"]  # never finished, always closed
    assert llm.calls[-1] == "nvfp4_end_probability_calibration"
    with pytest.raises(RuntimeError, match="already active"):
        worker.nvfp4_begin_probability_calibration(512, 8.0, 2)
        worker.nvfp4_begin_probability_calibration(512, 8.0, 2)
