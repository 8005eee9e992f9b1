"""Benchmark of the NVFP4 decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one decode step of one attention layer over the whole batch: the step's query is
quantized to NVFP4 (two terms), each sequence's new K/V token is written into its BF16 tail
(fused into the same launch), then paged FP4 decode attention runs over the FP4 pages, the
BF16 tail and the BF16 sink. The default workload (`gqa`) is the Qwen3-4B-shaped configuration:
32 query / 8 KV heads, head_dim 128, batch 64, 65,536 tokens per sequence, randomly shuffled block
table, 4 sink + 128 recent BF16 tokens, K/V/Q BF16 from N(0,1) with four lognormal(0,1.5) outlier
channels per KV head of K. With N GPUs the KV heads are partitioned over the ranks (as tensor
parallelism does), then the rows when ranks remain, with no collective: the step time is the
maximum over ranks. Other workloads: `cfg1` (batch 4, contexts in [512, 2048]: small enough for the
CPU arm to run whole), `cfg3` (32 query / 4 KV heads, batch 32, 131,072 tokens), `mixed` (256
Zipf-length sequences plus one 1M-token sequence split along the KV axis over the ranks, the one
step with a collective), `mla` (latent-cache decode), `longseq` (the 1M-token sequence alone).

Prints one JSON line (rank 0). `value` is microseconds per step with inputs resident in HBM: the
median over rounds of K steps, rounds repeated until `--min-seconds` of device time are measured;
`e2e` is the same step driven from pinned host buffers, with the host->device copy of the step's
query and new K/V token and the device->host copy of its output inside the timed region.
`--impl reference` times the reference's own CPU model of the step (oracle/_ref, made from the
reference tree by oracle/make_ref.py; the oracle port when that is absent) on all host threads.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "bitdecoding-fp4_b200"))

import torch  # noqa: E402

HEADS_Q, HEADS_KV, BATCH, CONTEXT = 32, 8, 64, 65536
SINK_USED, SINK_ROWS = 4, 16
WORKLOAD_NAME = "qwen3-4b-shape decode layer: 32q/8kv heads, d128, batch 64, ctx 65536, page {page}"
LONG_TOKENS = 1 << 20


def measured_peak_gbs() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


_SAMPLER_SOURCE = r"""
import sys, time
index, period = int(sys.argv[1]), float(sys.argv[2])
try:
    import pynvml
    pynvml.nvmlInit()
    handle = pynvml.nvmlDeviceGetHandleByIndex(index)
    print("max", pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM), flush=True)
    while True:
        clock = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
        mask = pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
        print(f"{time.time():.6f} {clock} {mask}", flush=True)
        time.sleep(period)
except Exception as error:
    print("error", error, flush=True)
"""


class ClockSampler:
    """Samples SM clocks and clock-event reasons while a region runs, with read-only NVML queries
    from a helper process (so the launching thread's hold on the interpreter cannot starve it)."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, index: int, period_s: float = 0.001):
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        physical = index
        if visible:
            entries = [e.strip() for e in visible.split(",") if e.strip()]
            if index < len(entries) and entries[index].isdigit():
                physical = int(entries[index])
        self.command = [sys.executable, "-c", _SAMPLER_SOURCE, str(physical), str(period_s)]
        self.process = None
        self.windows: list[list[float]] = []  # [begin, end] of every timed region
        self.lines: list[str] = []

    def __enter__(self):
        try:
            self.process = subprocess.Popen(self.command, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            # the "max" line and the first two samples: the helper is up and its queries are warm
            for _ in range(3):
                self.lines.append(self.process.stdout.readline())
        except Exception:
            self.process = None
        return self

    def open_window(self):
        self.windows.append([time.time(), float("inf")])

    def close_window(self):
        self.windows[-1][1] = time.time()

    def __exit__(self, *exc):
        if self.process is not None:
            self.process.terminate()
            try:
                self.lines.extend(self.process.communicate(timeout=10)[0].splitlines())
            except Exception:
                self.process.kill()

    def samples(self) -> list[tuple[float, int]]:
        """(host time, SM MHz) of every reading; complete once the sampler has been left."""
        out = []
        for line in self.lines:
            fields = line.split()
            if len(fields) == 3:
                try:
                    out.append((float(fields[0]), int(fields[1])))
                except ValueError:
                    pass
        return out

    def summary(self) -> dict:
        clocks, reasons, max_mhz = [], set(), None
        for line in self.lines:
            fields = line.split()
            if len(fields) == 2 and fields[0] == "max":
                max_mhz = int(fields[1])
            elif len(fields) == 3 and any(lo <= float(fields[0]) <= hi for lo, hi in self.windows):
                clocks.append(int(fields[1]))
                reasons.update(name for bit, name in self.REASONS.items() if int(fields[2]) & bit)
        return {
            "sm_mhz": int(statistics.median(clocks)) if clocks else None,
            "sm_max_mhz": max_mhz,
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


# ---------------------------------------------------------------------------------------------
# Workloads of the grouped-query path
# ---------------------------------------------------------------------------------------------

def zipf_lengths(count: int, low: int, high: int, alpha: float, seed: int) -> list[int]:
    """`count` context lengths on [low, high] with density proportional to length^-alpha (the
    continuous Zipf / power law, by inverse transform), seeded."""
    gen = torch.Generator().manual_seed(seed)
    u = torch.rand(count, generator=gen, dtype=torch.float64)
    a = 1.0 - alpha
    lengths = (low ** a + u * (high ** a - low ** a)) ** (1.0 / a)
    return [int(x) for x in lengths.round().clamp(low, high).tolist()]


def workload_spec(args) -> dict:
    """Shape of the named workload: total heads, the rows' context lengths, and its description."""
    name = args.workload
    if name == "gqa":
        heads_q, heads_kv = args.heads_q or HEADS_Q, args.heads_kv or HEADS_KV
        rows, context = args.batch or BATCH, args.context
        label = WORKLOAD_NAME.format(page=args.page_tokens)
        if (context, rows, heads_kv, heads_q) != (CONTEXT, BATCH, HEADS_KV, HEADS_Q):
            label += f" [shape overridden: batch {rows}, {heads_q}q/{heads_kv}kv heads, context {context}]"
        return dict(name=name, heads_q=heads_q, heads_kv=heads_kv, lengths=[context] * rows, label=label)
    if name == "cfg1":
        gen = torch.Generator().manual_seed(0)
        lengths = torch.randint(512, 2049, (4,), generator=gen).tolist()
        return dict(name=name, heads_q=8, heads_kv=2, lengths=lengths,
                    label=f"small-batch decode layer: 8q/2kv heads, d128, batch 4, contexts uniform in [512, 2048] "
                          f"(seeded: {lengths}), page {args.page_tokens}")
    if name == "cfg3":
        rows, context = args.batch or 32, args.context if args.context != CONTEXT else 131072
        return dict(name=name, heads_q=32, heads_kv=4, lengths=[context] * rows,
                    label=f"qwen3-30b-a3b-shape decode layer: 32q/4kv heads (8 query heads per KV head), d128, "
                          f"batch {rows}, ctx {context}, page {args.page_tokens}")
    if name == "mixed":
        rows = args.batch or 256
        lengths = zipf_lengths(rows, 1024, 131072, 1.2, seed=5)
        return dict(name=name, heads_q=32, heads_kv=8, lengths=lengths,
                    label=f"mixed serving step: {rows} sequences of 32q/8kv heads, d128, contexts Zipf(1.2) on "
                          f"[1K, 128K] ({sum(lengths):,} tokens), page {args.page_tokens}, plus one "
                          f"{LONG_TOKENS:,}-token sequence split along the KV axis over the ranks")
    raise SystemExit(f"unknown workload {name!r}")


def ragged_row_splits(lengths: list[int], heads_kv: int, sms: int, limit: int = 16) -> list[int]:
    """Parts per row for a batch of very unequal lengths (`row_splits` of the decode call): a row is cut
    into parts of about a third of the share of one resident CTA, so the long rows no longer bound the
    launch and the short ones are not cut into set-up."""
    steps = [max(1, n // 128) for n in lengths]
    # a third of that share per part: the parts of a row start one launch wave apart (the grid is part-major),
    # so finer parts balance better. One GPU, 256 Zipf rows x 8 KV heads, batch kernel: one share per part
    # 1,110 us, a half 986 us, a third 968 us, a quarter 982 us; three parts for every row 990 us.
    target = max(1.0, sum(steps) * heads_kv / (4 * sms) / 3)
    return [max(1, min(limit, math.ceil(n / target))) for n in steps]


def partition(spec: dict, world: int, rank: int, kv_groups: int = 0) -> dict:
    """This rank's share: KV heads are dealt out first (contiguous groups, as tensor parallelism does),
    then, when there are more ranks than KV-head groups, the rows are sharded over the remaining factor.
    Ragged batches are dealt longest-first in a snake, so that the shards' token counts stay close.
    No rank needs anything from another."""
    total_kv = spec["heads_kv"]
    groups = kv_groups or min(world, total_kv)
    if world % groups or total_kv % groups:
        raise SystemExit(f"{total_kv} KV heads / {world} ranks do not partition into {groups} head groups")
    shards = world // groups
    rows = len(spec["lengths"])
    if rows < shards:
        raise SystemExit(f"{rows} rows cannot be sharded {shards} ways")
    order = sorted(range(rows), key=lambda r: -spec["lengths"][r])
    shard_of = {}
    for position, row in enumerate(order):
        lap, slot = divmod(position, shards)
        shard_of[row] = slot if lap % 2 == 0 else shards - 1 - slot
    mine = [r for r in range(rows) if shard_of[r] == rank // groups]
    ratio = spec["heads_q"] // total_kv
    heads_kv = total_kv // groups
    return dict(heads_kv=heads_kv, heads_q=heads_kv * ratio, lengths=[spec["lengths"][r] for r in mine],
                text=f"{heads_kv} of {total_kv} KV heads x {len(mine)} of {rows} rows per rank, no collective")


def common_config(spec: dict, part_text: str, page_tokens: int, scale_mode: str = "nvfp4") -> dict:
    """The `config` object both arms print, key for key."""
    mx = scale_mode.startswith("mxfp4")
    return {
        "workload": spec["label"],
        "partition": part_text,
        "sink_tokens": SINK_USED, "recent_tokens": 128,
        "query": f"two {'MXFP4' if mx else 'NVFP4'} terms, Hadamard",
        "key_scale_mode": scale_mode if mx else "four_six", "value_scale_mode": scale_mode if mx else "amax6",
        "p_scale_mode": "mxfp4 adjacent-exponent search" if mx else "amax2_or_amax6_c8", "page_tokens": page_tokens,
        "l2": "the cache walked per step exceeds the 126 MB L2 (or, for the small workloads, is re-read from "
              "HBM-resident pages after an L2-sized flush write between rounds)",
    }


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's own CPU model (oracle/_ref) or, without it, the oracle port
# ---------------------------------------------------------------------------------------------

def cpu_step(spec: dict, lengths: list[int], heads_kv: int, budget_s: float, page_tokens: int) -> dict:
    """Seconds of CPU time for one step of this rank's share. Rows no longer than 4,096 tokens are run
    whole, every one of them; longer rows are sampled: a slice of one KV head and at most 16,384 tokens is
    timed for about `budget_s` seconds and scaled by (heads x context ratio), which the result says."""
    from oracle import cpu_arm

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    ratio = spec["heads_q"] // spec["heads_kv"]
    cpu_arm.step_seconds(1024, ratio=ratio, page_tokens=page_tokens)  # warm the thread pool and allocator
    whole = max(lengths) <= 4096
    if whole:
        seconds, kind = 0.0, "port"
        for i, n in enumerate(lengths):
            s, kind = cpu_arm.step_seconds(n, heads_kv=heads_kv, ratio=ratio, seed=i, page_tokens=page_tokens)
            seconds += s
        return dict(seconds=seconds, kind=kind, cores=threads, extrapolated_x=1.0,
                    sample=f"every row whole: {len(lengths)} rows x {heads_kv} KV heads x {ratio} query heads each, "
                           f"{seconds:.3f} s on {threads} threads")
    sample_context = min(16384, max(lengths))
    spent, repeats, kind = 0.0, 0, "port"
    while spent < budget_s:
        s, kind = cpu_arm.step_seconds(sample_context, heads_kv=1, ratio=ratio, seed=repeats, page_tokens=page_tokens)
        spent += s
        repeats += 1
    per_token_head = spent / repeats / sample_context
    units = sum(lengths) * heads_kv
    factor = units / sample_context
    return dict(seconds=per_token_head * units, kind=kind, cores=threads, extrapolated_x=factor,
                sample=f"{repeats} steps of 1 row x 1 KV head ({ratio} query heads) x {sample_context} tokens, "
                       f"{spent / repeats:.3f} s each on {threads} threads ({spent:.1f} s in all); scaled by "
                       f"{factor:.0f} (tokens x KV heads of the rank's step over the sample's): an extrapolation, "
                       "not a run of the full step")


def cpu_baseline_entry(measured: dict) -> dict:
    return {"value": measured["seconds"] * 1e6, "unit": "us/step", "cores": measured["cores"],
            "kind": "reference" if measured["kind"] == "reference" else "port",
            "sample": measured["sample"], "extrapolated_x": measured["extrapolated_x"]}


def run_reference(args) -> None:
    """`--impl reference`: the reference's CPU implementation of the step on the host cores (rank 0 only)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    if args.scale_mode != "nvfp4":
        print(json.dumps({"impl": "reference", "unavailable": "the reference's CPU model timed here is the NVFP4 one; "
                          "run this arm without --scale-mode"}))
        return
    spec = workload_spec(args)
    part = partition(spec, args.gpus, 0, args.kv_groups)
    for _ in range(min(args.warmup, 2)):
        cpu_step(spec, part["lengths"][:1], 1, 0.5, args.page_tokens)
    runs = [cpu_step(spec, part["lengths"], part["heads_kv"], 3.0, args.page_tokens) for _ in range(args.steps)]
    seconds = statistics.mean(r["seconds"] for r in runs)
    last = dict(runs[-1], seconds=seconds)
    value = seconds * 1e6
    print(json.dumps({
        "impl": "reference", "metric": "decode_attn_us_per_step", "value": value, "unit": "us/step",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": value / 1e3,
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp4(e2m1)+ue4m3 / f32 accumulate", "data": "synthetic",
        "config": common_config(spec, part["text"], args.page_tokens),
        "cpu_baseline": cpu_baseline_entry(last),
        "reference_gpu_kernel": REFERENCE_GPU_NOTE,
        "e2e": {"value": value, "unit": "us/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


REFERENCE_GPU_NOTE = ("unavailable on this box: the reference's CuTeDSL kernels pin nvidia-cutlass-dsl 4.6.0 and the "
                      "image has 4.5.0; the arm timed here is the reference's CPU model")


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

class TimedRounds:
    """Rounds of K steps, each bracketed by CUDA events on the launching stream and a synchronise, until
    at least `min_seconds` of device time have been measured; the clock sampler's readings are binned
    per round, so a burst-clock round and a power-capped one can be told apart."""

    def __init__(self, steps: int, min_seconds: float, sampler: ClockSampler, barrier, agree=None):
        self.steps, self.min_seconds, self.sampler, self.barrier = steps, min_seconds, sampler, barrier
        # Every rank must run the same number of rounds (a step may hold a collective): the running total
        # each rank stops on is the maximum over ranks, agreed between rounds and outside the events.
        self.agree = agree or (lambda seconds: seconds)
        self.rounds: list[dict] = []

    def run(self, one_step, kernel_events_of=None) -> None:
        total = 0.0
        self.barrier()
        while True:
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            pairs = [] if kernel_events_of is None else [kernel_events_of() for _ in range(self.steps)]
            self.sampler.open_window()
            begin.record()
            for k in range(self.steps):
                one_step(pairs[k] if pairs else None)
            end.record()
            torch.cuda.synchronize()
            self.sampler.close_window()
            ms = begin.elapsed_time(end)
            kernel_ms = statistics.mean(a.elapsed_time(b) for a, b in pairs) if pairs else None
            self.rounds.append({"ms_per_step": ms / self.steps, "kernel_ms": kernel_ms,
                                "window": tuple(self.sampler.windows[-1])})
            total = self.agree(total + ms * 1e-3)
            if total >= self.min_seconds or len(self.rounds) >= 2000:
                break
        self.barrier()

    def median_ms(self) -> float:
        return statistics.median(r["ms_per_step"] for r in self.rounds)

    def median_kernel_ms(self) -> float:
        return statistics.median(r["kernel_ms"] for r in self.rounds)

    def clock_bins(self) -> list[dict]:
        """Rounds grouped by the median SM clock sampled while they ran (50 MHz bins)."""
        samples = self.sampler.samples()
        bins: dict[int, list[float]] = {}
        for r in self.rounds:
            lo, hi = r["window"]
            clocks = [c for t, c in samples if lo <= t <= hi]
            if clocks:
                bins.setdefault(int(statistics.median(clocks)) // 50 * 50, []).append(r["ms_per_step"])
        return [{"sm_mhz_from": mhz, "rounds": len(v), "us_per_step": statistics.median(v) * 1e3,
                 "us_x_mhz": statistics.median(v) * 1e3 * (mhz + 25)} for mhz, v in sorted(bins.items())]


def flush_l2(scratch: torch.Tensor) -> None:
    scratch.add_(1)


def sustained_copy_gbs(device, seconds: float = 0.8) -> dict:
    """What a plain device-to-device copy sustains on this GPU right now, for about `seconds`: the same
    STREAM-style measure as the burst figure the roofline divides by (read + written bytes over the
    time), but taken back to back so that it runs under whatever clocks a long step runs under."""
    elems = 1 << 29  # 1 GiB of BF16 in, 1 GiB out
    a = torch.empty(elems, dtype=torch.bfloat16, device=device)
    b = torch.empty_like(a)
    for _ in range(3):
        b.copy_(a)
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    copies = 0
    begin.record()
    start = time.time()
    while time.time() - start < seconds:
        for _ in range(10):
            b.copy_(a)
        copies += 10
        torch.cuda.synchronize()
    end.record()
    torch.cuda.synchronize()
    gbs = copies * 2 * elems * 2 / (begin.elapsed_time(end) * 1e-3) / 1e9
    del a, b
    return {"gb_s": gbs, "seconds": begin.elapsed_time(end) * 1e-3, "copies": copies}


def run_gqa(args) -> None:
    import torch.distributed as dist

    import bdfp4
    from bdfp4.workload import build_workload, split_lengths
    from nvfp4_decode_kernel import DecodeTailWrite, fp4_decode, split_partial_count
    from nvfp4_decode_kernel import _decode as decode_module
    from nvfp4_decode_kernel._quantize import quantize_query

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run, one rank per GPU")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    mixed = args.workload == "mixed"
    if world > 1 or mixed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    spec = workload_spec(args)
    kv_groups = args.kv_groups or (min(world, 4) if mixed and world >= 8 else 0)
    part = partition(spec, world, rank, kv_groups)
    heads_kv, heads_q, lengths = part["heads_kv"], part["heads_q"], part["lengths"]
    rows = len(lengths)
    page_tokens = args.page_tokens

    mx = args.scale_mode.startswith("mxfp4")
    if mx and page_tokens != 128:
        raise SystemExit("an MXFP4 cache has 128-token pages: pass --page-tokens 128")
    key_mode, value_mode, query_mode = (args.scale_mode,) * 3 if mx else ("four_six", "amax6", "amax6")
    scale_format = "mxfp4" if mx else "nvfp4"
    w = build_workload(rows=rows, heads_q=heads_q, heads_kv=heads_kv, seq_lens=lengths, sink_tokens=SINK_ROWS,
                       seed=1000 + rank, device=device, key_scale_mode=key_mode, value_scale_mode=value_mode,
                       rotate=True, page_tokens=page_tokens)
    w.seqused_sink.clamp_(max=SINK_USED)
    w.sink_tokens = SINK_USED
    algorithmic_bytes = w.algorithmic_bytes()
    if mx:  # one E8M0 byte per 32 values instead of one E4M3 byte per 16: 136 bytes per token and head side
        algorithmic_bytes -= sum(split_lengths(n, SINK_USED)[1] for n in lengths) * heads_kv * 8
    sms = decode_module._multiprocessor_count(local_rank)
    # split count from the batch width only (never from device lengths): enough partitions to keep the
    # whole launch resident at four CTAs per SM
    splits = args.splits or decode_module.resident_num_splits(rows, heads_kv, sms=sms)
    ragged = len(set(lengths)) > 1
    row_parts = None
    if ragged and not args.splits:
        # every row gets the parts its own length calls for; the launch has as many as the longest
        row_parts = ragged_row_splits(lengths, heads_kv, sms)
        splits = max(splits if max(row_parts) > 1 else 1, max(row_parts))
        row_parts = [min(n, splits) for n in row_parts]
    parts = split_partial_count(rows, heads_kv, splits, residual=True, sms=sms)
    row_splits = torch.tensor(row_parts, dtype=torch.int32, device=device) if row_parts and splits > 1 else None
    row_order = torch.argsort(w.seqused_fp4, descending=True).to(torch.int32) if ragged else None

    gen = torch.Generator(device=device).manual_seed(77 + rank)
    new_key = torch.randn(rows, heads_kv, 128, generator=gen, device=device).to(torch.bfloat16)
    new_value = torch.randn(rows, heads_kv, 128, generator=gen, device=device).to(torch.bfloat16)
    seq_lens = torch.tensor(lengths, dtype=torch.int32, device=device)
    scratch = dict(
        query_padded_scratch=torch.zeros(rows, 128, heads_q, 128, dtype=torch.bfloat16, device=device),
        query_fp4_scratch=torch.zeros(rows, 1, heads_q, 64, dtype=torch.uint8, device=device),
        query_scales_scratch=torch.zeros(rows, 1, heads_q, 1 if mx else 2, 32, 4, 4, dtype=torch.uint8, device=device),
        query_fp4_second_scratch=torch.zeros(rows, 1, heads_q, 64, dtype=torch.uint8, device=device),
        query_scales_second_scratch=torch.zeros(rows, 1, heads_q, 1 if mx else 2, 32, 4, 4, dtype=torch.uint8,
                                                device=device),
    )
    if splits > 1:
        scratch["split_partial_scratch"] = torch.empty(parts * rows * heads_q * 128, device=device)
        scratch["split_lse_scratch"] = torch.empty(parts * rows * heads_q, device=device)
        if args.fused_merge:
            scratch["split_merge_counters"] = torch.zeros(rows * heads_kv, dtype=torch.int32, device=device)
    out = torch.empty(rows, heads_q, 128, dtype=torch.bfloat16, device=device)

    # ---- the long sequence of the mixed step: this rank's KV shard of it ------------------------
    long_step, long_bytes = None, 0
    if mixed:
        from bdfp4.distributed import KvShardedDecoder

        shard = LONG_TOKENS // world // 128 * 128
        wl = build_workload(rows=1, heads_q=HEADS_Q, heads_kv=HEADS_KV, seq_lens=[shard + 128], sink_tokens=SINK_ROWS,
                            seed=7000 + rank, device=device, key_scale_mode="four_six", value_scale_mode="amax6",
                            rotate=True, page_tokens=page_tokens)
        wl.seqused_sink.clamp_(max=SINK_USED)
        wl.sink_tokens = SINK_USED
        owner_tail, owner_sink = rank == world - 1, rank == 0
        zeros = torch.zeros_like(wl.seqused_residual)
        long_out = torch.empty(1, HEADS_Q, 128, dtype=torch.bfloat16, device=device)
        long_decoder = KvShardedDecoder(
            *wl.regions, wl.page_table, wl.seqused_fp4, residual_key_pages_bf16=wl.tail_key[0],
            residual_value_pages_bf16=wl.tail_value[0], residual_page_ids=wl.slot_ids,
            seqused_residual=wl.seqused_residual if owner_tail else zeros,
            seqused_sink=wl.seqused_sink if owner_sink else zeros, heads_q=HEADS_Q, query_terms=2,
            query_rotation="hadamard", out=long_out, exchange=args.exchange)
        long_bytes = wl.algorithmic_bytes()

        def long_step():
            return long_decoder(wl.query)

    def step(query, key_token, value_token):
        tail = DecodeTailWrite(key_token, value_token, w.tail_key[0], w.tail_value[0], w.slot_ids, seq_lens,
                               w.seqused_fp4, True, None, SINK_ROWS)
        result = fp4_decode(
            query, *w.regions, w.page_table, w.seqused_fp4, residual_key_pages_bf16=w.tail_key[0],
            residual_value_pages_bf16=w.tail_value[0], residual_page_ids=w.slot_ids,
            seqused_residual=w.seqused_residual, seqused_sink=w.seqused_sink, out=out, trusted_metadata=True,
            num_splits=splits, query_terms=2, scale_mode=query_mode, query_rotation="hadamard", tail_write=tail,
            row_order=row_order, row_splits=row_splits, **scratch)
        if long_step is not None:
            long_step()
        return result

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(value: float) -> float:
        if world == 1:
            return value
        t = torch.tensor([value], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident arm ----------------------------------------------------------------
    # The step's launches are issued directly (query quantizer with the fused tail write, the decode
    # kernel, the split merge) so that CUDA events on the launching stream bracket the decode kernel
    # inside the same timed region the step time comes from.
    tail = DecodeTailWrite(new_key, new_value, w.tail_key[0], w.tail_value[0], w.slot_ids, seq_lens,
                           w.seqused_fp4, True, None, SINK_ROWS)

    def quantize_step():
        return quantize_query(
            w.query, query_padded_out=scratch["query_padded_scratch"], heads_kv=heads_kv,
            query_fp4_scratch=scratch["query_fp4_scratch"], query_scales_scratch=scratch["query_scales_scratch"],
            query_fp4_second_scratch=scratch["query_fp4_second_scratch"],
            query_scales_second_scratch=scratch["query_scales_second_scratch"], query_terms=2, rotation="hadamard",
            scale_mode=query_mode, tail_write=tail)

    quantized = quantize_step()
    kernel_args = bdfp4.DecodeArgs()
    decode_module._fill_args(
        kernel_args, rows=rows, heads_q=heads_q, heads_kv=heads_kv, page_count=w.regions[0].shape[0],
        query_fp4=quantized[0], query_scales=quantized[1], query_fp4_second=quantized[2],
        query_scales_second=quantized[3], query_padded_bf16=scratch["query_padded_scratch"],
        key_pages_fp4=w.regions[0], key_scales=w.regions[1], value_pages_fp4=w.regions[2], value_scales=w.regions[3],
        fp4_page_table=w.page_table, seqused_fp4=w.seqused_fp4, residual_key_pages_bf16=w.tail_key[0],
        residual_value_pages_bf16=w.tail_value[0], residual_page_ids=w.slot_ids,
        seqused_residual=w.seqused_residual, seqused_sink=w.seqused_sink, softmax_scale=128 ** -0.5,
        row_order=row_order, scale_format=scale_format, row_splits=row_splits)
    page_cost = decode_module.BF16_BLOCK_PAGE_COST if parts == splits and splits > 1 else 0
    if args.bf16_cost >= 0:
        page_cost = args.bf16_cost
    kernel_args.num_splits = splits
    kernel_args.bf16_split = int(parts > splits)
    kernel_args.bf16_page_cost = page_cost
    if splits > 1:
        kernel_args.partial_out = scratch["split_partial_scratch"].data_ptr()
        kernel_args.partial_lse = scratch["split_lse_scratch"].data_ptr()
    if splits == 1 or args.fused_merge:
        kernel_args.out, kernel_args.out_row_stride = out.data_ptr(), out.stride(0)
    if splits > 1 and args.fused_merge:  # the split launch merges its own partials
        kernel_args.merge_counters = scratch["split_merge_counters"].data_ptr()
    stream = bdfp4.current_stream(device)
    # the small workloads fit in L2: a write larger than L2 between steps sends their pages back to HBM
    small = algorithmic_bytes + long_bytes < (256 << 20)
    l2_scratch = torch.zeros(160 << 20, dtype=torch.uint8, device=device) if small else None

    def device_step(events=None):
        if l2_scratch is not None:
            flush_l2(l2_scratch)
        quantize_step()
        if events:
            events[0].record()
        bdfp4.decode(kernel_args, stream)
        if events:
            events[1].record()
        if splits > 1 and not args.fused_merge:
            bdfp4.combine(scratch["split_partial_scratch"], scratch["split_lse_scratch"], parts, rows, heads_q, out,
                          out.stride(0), stream)
        if long_step is not None:
            long_step()

    for _ in range(args.warmup):
        device_step()
    sampler = ClockSampler(local_rank)
    sampler.__enter__()  # samples through both timed regions; left at the end of the end-to-end arm
    resident = TimedRounds(args.steps, args.min_seconds, sampler, barrier, max_over_ranks)
    resident.run(device_step, lambda: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)))
    step_ms = max_over_ranks(resident.median_ms())
    kernel_ms = max_over_ranks(resident.median_kernel_ms())
    flush_ms = 0.0
    if l2_scratch is not None:  # the flush write is inside the step's events: measure it and take it out
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(20):
            flush_l2(l2_scratch)
        end.record()
        torch.cuda.synchronize()
        flush_ms = begin.elapsed_time(end) / 20
        step_ms -= flush_ms

    # ---- end-to-end arm: host buffers in, host buffer out, copies inside the timed region ------
    # The step's inputs (query, new K token, new V token of every row) sit in one pinned host record
    # and travel as one copy; the output comes back into a pinned host buffer.
    q_elems, kv_elems = w.query.numel(), new_key.numel()
    host_in = torch.empty(q_elems + 2 * kv_elems, dtype=torch.bfloat16).pin_memory()
    host_in[:q_elems] = w.query.cpu().reshape(-1)
    host_in[q_elems:q_elems + kv_elems] = new_key.cpu().reshape(-1)
    host_in[q_elems + kv_elems:] = new_value.cpu().reshape(-1)
    host_out = torch.empty(rows, heads_q, 128, dtype=torch.bfloat16).pin_memory()
    dev_in = torch.empty_like(host_in, device=device)
    dev_query = dev_in[:q_elems].view_as(w.query)
    dev_key = dev_in[q_elems:q_elems + kv_elems].view_as(new_key)
    dev_value = dev_in[q_elems + kv_elems:].view_as(new_value)

    def whole_step():
        dev_in.copy_(host_in, non_blocking=True)
        step(dev_query, dev_key, dev_value)
        host_out.copy_(out, non_blocking=True)

    # The whole step is captured once into a CUDA graph, as the serving engine captures its uniform
    # decode batches: the copy in, the plugin call and the copy out; a step is one replay and a
    # synchronise. The mixed step holds a collective, which is launched eagerly instead.
    graph = None
    if not mixed:
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            whole_step()
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            whole_step()

    def e2e_step(_events=None):
        if l2_scratch is not None:
            flush_l2(l2_scratch)
        if graph is not None:
            graph.replay()
        else:
            whole_step()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        e2e_step()
    end_to_end = TimedRounds(args.steps, args.min_seconds, sampler, barrier, max_over_ranks)
    end_to_end.run(e2e_step)
    sampler.__exit__(None, None, None)
    e2e_ms = max_over_ranks(end_to_end.median_ms()) - flush_ms
    h2d = host_in.numel() * 2
    d2h = host_out.numel() * 2

    # ---- quantize-on-write throughput (bulk page quantize, K and V) ---------------------------
    from nvfp4_decode_kernel.quantize_kv_kernel import KVCacheWriter

    q_pages = min(2048 * (128 // page_tokens), int((w.seqused_fp4 // page_tokens).sum()))
    quantize = None
    if q_pages >= 64:
        source_k = torch.randn(q_pages * page_tokens, heads_kv, 128, generator=gen, device=device).to(torch.bfloat16)
        source_v = torch.randn(q_pages * page_tokens, heads_kv, 128, generator=gen, device=device).to(torch.bfloat16)
        writer = KVCacheWriter(regions=w.regions, key_scale_mode=key_mode, value_scale_mode=value_mode, rotate_key=True)
        work_src = torch.arange(q_pages, dtype=torch.int32, device=device) * page_tokens
        used = torch.cat([w.page_table[r, :int(w.seqused_fp4[r]) // page_tokens] for r in range(rows)])
        work_dst = used[:q_pages].contiguous()
        for _ in range(3):
            writer(source_k, source_v, w.regions, work_src, work_dst)
        barrier()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(5):
            writer(source_k, source_v, w.regions, work_src, work_dst)
        end.record()
        barrier()
        quant_ms = begin.elapsed_time(end) / 5
        quant_bytes = q_pages * heads_kv * 2 * (page_tokens * 256 + page_tokens * (68 if mx else 72))
        quantize = {"ms": quant_ms, "bytes": quant_bytes, "gb_s": quant_bytes / (quant_ms * 1e-3) / 1e9,
                    "page_heads": q_pages * heads_kv * 2}

    # ---- parity at the benchmarked size, after and outside every timed region ------------------
    verified = None
    if args.verify:  # every rank takes the step (the mixed one holds a collective); rank 0 checks its own
        result = step(w.query, new_key, new_value)
        torch.cuda.synchronize()
    if args.verify and rank == 0:
        from oracle import tile_check

        torch.manual_seed(0)
        tiles = [(int(torch.randint(rows, (1,))), int(torch.randint(heads_kv, (1,)))) for _ in range(args.verify)]
        verified = tile_check.check_tiles(
            w, result, tiles, terms=2, scale_mode=query_mode, rotate=True, num_splits=splits, bf16_split=parts > splits,
            row_splits=row_parts if row_splits is not None else None,
            bf16_page_cost=decode_module.BF16_BLOCK_PAGE_COST if parts == splits and splits > 1 else 0)
        verified["tolerance"] = {"max_abs": 1e-2, "mean_rel": 1e-3}
        verified["against"] = "CPU oracle on sampled (row, KV head) tiles of this run's cache"

    live_copy = sustained_copy_gbs(device) if (rank == 0 and not args.no_live_copy) else None
    total_bytes = algorithmic_bytes
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, algorithmic_bytes)
        total_bytes = sum(gathered)
    peak, peak_kind = measured_peak_gbs()
    achieved = algorithmic_bytes / (kernel_ms * 1e-3) / 1e9
    clocks = sampler.summary()
    # DRAM traffic per launch is an estimate: algorithmic bytes times the ratio ncu measured on the
    # 8,192-token capture of the same kernel (639.8 / 630.3 MB with 64-token pages, 637.9 / 630.2 MB
    # with 128-token pages); traffic grows in proportion to the pages walked.
    traffic = algorithmic_bytes * ((639.8 / 630.3) if page_tokens == 64 else (637.9 / 630.2))
    if rank == 0:
        launches = (2 + (1 if splits > 1 and not args.fused_merge else 0) + (1 if small else 0) +
                    ((3 if args.exchange == "peer" else 5) if mixed else 0))
        config = common_config(spec, part["text"], page_tokens, args.scale_mode)
        line = {
            "metric": "decode_attn_us_per_step" if not mixed else "mixed_step_us",
            "value": step_ms * 1e3, "unit": "us/step", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": step_ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp4(e2m1)+ue8m0 / f32 accumulate" if mx else "fp4(e2m1)+ue4m3 / f32 accumulate",
            "data": "synthetic", "config": config,
            "launch": {"num_splits": splits, "parts": parts, "bf16_page_cost": page_cost,
                       "row_splits": None if row_splits is None else
                       {"min": min(row_parts), "max": max(row_parts), "ctas_with_work": sum(row_parts) * heads_kv},
                       "row_order": "longest first" if ragged else "index order",
                       "l2_flush_between_steps": small, "l2_flush_us_removed": flush_ms * 1e3},
            "timing": {"statistic": "median over rounds of K steps, max over ranks", "rounds": len(resident.rounds),
                       "timed_region_s": sum(r["ms_per_step"] for r in resident.rounds) * args.steps * 1e-3,
                       "clock_bins": resident.clock_bins(),
                       "us_x_median_sm_mhz": step_ms * 1e3 * (clocks["sm_mhz"] or 0)},
            "hbm_tb_s": (total_bytes + long_bytes * world) / (step_ms * 1e-3) / 1e12,
            "decode_kernel_us": kernel_ms * 1e3,
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "traffic_source": "estimated from the ncu capture under profiles/ (ratio to "
                                                      "algorithmic bytes 1.015 / 1.012), not measured in this run",
                "peak_kind": f"of {peak_kind}", "kernel": "decode_kernel",
                "algorithmic_bytes_per_launch": algorithmic_bytes,
                # context, not the denominator: the same copy measured back to back in this very run
                "copy_sustained_in_this_run_gb_s": None if live_copy is None else live_copy["gb_s"],
                "frac_of_copy_sustained_in_this_run": None if live_copy is None else achieved / live_copy["gb_s"],
            },
            "e2e": {"value": e2e_ms * 1e3, "unit": "us/step", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "how": "every step: one CUDA-graph replay of [H2D of the pinned input record, plugin call, D2H "
                           "into a pinned buffer], then synchronise" if graph is not None else
                           "every step: H2D of the pinned input record, plugin call (with its collective), D2H into "
                           "a pinned buffer, then synchronise"},
            "gpu_launches": args.steps * launches * len(resident.rounds),
            "clocks": clocks,
            "reference_gpu_kernel": REFERENCE_GPU_NOTE,
        }
        if quantize is not None:
            line["quantize_gb_s"] = quantize["gb_s"]
            line["roofline_quantize"] = {
                "bound": "hbm", "kernel": f"kv_page_kernel (K: Hadamard + {key_mode}, V: {value_mode})",
                "achieved": quantize["gb_s"], "peak": peak, "unit": "GB/s", "frac": quantize["gb_s"] / peak,
                "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_launch": quantize["bytes"],
                "units_per_launch": f"{quantize['page_heads']} page-heads x {page_tokens * 328} B "
                                    "(BF16 in, codes and scales out)", "traffic": None,
                "note": "the K role is instruction-bound (scale search + 7-level Hadamard), not HBM-bound",
            }
        if verified is not None:
            line["verified"] = verified
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_entry(cpu_step(spec, lengths, heads_kv, 12.0, page_tokens))
        print(json.dumps(line))
    if mixed:
        long_decoder.close()
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# MLA latent-cache decode (`--workload mla`): 128 query heads over one compressed KV of 512 NVFP4
# channels + 64 BF16 rope channels, batch 64, context 32,768, 64-token pages, rows over the ranks
# ---------------------------------------------------------------------------------------------

MLA_BATCH, MLA_HEADS, MLA_CONTEXT = 64, 128, 32768
MLA_SCALE = 576 ** -0.5
MLA_WORKLOAD = ("MLA-shaped latent-cache decode: 128 query heads, kv_lora_rank 512 (NVFP4, cached along channels "
                "and along tokens) + 64 BF16 rope, batch 64, context 32,768, page 64, shuffled block table")
MLA_TOKEN_BYTES = 416        # one latent copy (256 + 32) + rope 128: the single-copy figure the roofline uses
MLA_CACHE_TOKEN_BYTES = 704  # what this cache layout holds and the kernel reads per token


def mla_cpu_sample(tokens: int, heads: int, threads: int, seed: int = 0) -> float:
    """Seconds for one MLA decode step of (1 row, `heads` query heads, `tokens` tokens) on the CPU
    oracle, dequantizing both latent copies as a CPU path has to; the cache is quantized up front."""
    from oracle import mla_oracle

    torch.set_num_threads(threads)
    gen = torch.Generator().manual_seed(seed)
    pages = tokens // 64
    latent = torch.randn(tokens, 512, generator=gen)
    latent[:, torch.randperm(512, generator=gen)[:8]] *= torch.exp(1.5 * torch.randn(8, generator=gen))
    latent = latent.to(torch.bfloat16)
    rope = torch.randn(pages, 64, 64, generator=gen).to(torch.bfloat16)
    kc, ks, vc, vs = mla_oracle.quantize_pages(latent.reshape(pages, 64, 512))
    q_latent = torch.randn(1, heads, 512, generator=gen).to(torch.bfloat16)
    q_rope = torch.randn(1, heads, 64, generator=gen).to(torch.bfloat16)
    table = torch.arange(pages, dtype=torch.int32)[None]
    start = time.perf_counter()
    _, _, q_values = mla_oracle.quantize_query(q_latent)
    mla_oracle.decode_reference(q_values=q_values, q_rope=q_rope, key_codes=kc, key_scales=ks, value_codes=vc,
                                value_scales=vs, rope=rope, page_table=table, seq_lens=torch.tensor([tokens]),
                                softmax_scale=MLA_SCALE)
    return time.perf_counter() - start


def mla_cpu_baseline(rows_local: int, budget_s: float, sample_tokens: int = 4096, sample_heads: int = 128):
    threads = os.cpu_count() or 1
    mla_cpu_sample(512, sample_heads, threads)
    repeats, spent = 0, 0.0
    while spent < budget_s:
        spent += mla_cpu_sample(sample_tokens, sample_heads, threads, seed=repeats)
        repeats += 1
    seconds = spent / repeats
    units = rows_local * (MLA_HEADS / sample_heads) * (MLA_CONTEXT / sample_tokens)
    return seconds * units * 1e6, {
        "value": seconds * units * 1e6, "unit": "us/step", "cores": threads, "kind": "port",
        "sample": (f"MLA oracle (PyTorch CPU; the reference has no MLA path), {repeats} steps of 1 row x {sample_heads} "
                   f"heads x {sample_tokens} tokens, {seconds:.3f} s each on {threads} threads ({spent:.1f} s in all); "
                   f"scaled by {units:.0f} (rows x context ratio) to the rank's full step"),
    }


def run_mla_reference(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    rows_local = MLA_BATCH // args.gpus
    for _ in range(args.warmup):
        mla_cpu_sample(512, 128, os.cpu_count() or 1)
    values = []
    baseline = None
    for _ in range(args.steps):
        value, baseline = mla_cpu_baseline(rows_local, budget_s=2.0)
        values.append(value)
    value = sum(values) / len(values)
    baseline["value"] = value
    print(json.dumps({
        "impl": "reference", "metric": "mla_decode_attn_us_per_step", "value": value, "unit": "us/step",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": value / 1e3,
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp4(e2m1)+ue4m3 / f32 accumulate", "data": "synthetic",
        "config": {"workload": MLA_WORKLOAD, "rows_per_rank": rows_local},
        "cpu_baseline": baseline,
        "e2e": {"value": value, "unit": "us/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_mla(args) -> None:
    import torch.distributed as dist

    from nvfp4_decode_kernel import mla

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run, one rank per GPU")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    total_rows = args.batch or MLA_BATCH
    context = args.context if args.context != CONTEXT else MLA_CONTEXT
    if total_rows % world or context % 64:
        raise SystemExit("rows must divide over the ranks and the context be whole pages")
    rows = total_rows // world
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    # a CTA pair per (row, split): enough splits to give every SM a CTA, from the batch width only
    splits = args.splits or max(1, (sms // 2) // rows)

    gen = torch.Generator(device=device).manual_seed(4000 + rank)
    pages_per_row = context // 64
    total = rows * pages_per_row
    cache = mla.MLACache.allocate(total + 1, device)
    table = (torch.randperm(total, generator=gen, device=device) + 1).to(torch.int32).reshape(rows, pages_per_row)
    outliers = torch.randperm(512, generator=gen, device=device)[:8]
    factor = torch.exp(1.5 * torch.randn(8, generator=gen, device=device))
    source = torch.arange(pages_per_row, dtype=torch.int32, device=device) * 64
    # every step appends one token per row (quantize-on-write) before it attends: the rows sit one
    # token short of the context, their last page open in the appender's BF16 staging buffers
    appender = mla.MLAAppender(rows, device)
    open_latent = torch.zeros(rows, 64, 512, dtype=torch.bfloat16, device=device)
    open_rope = torch.zeros(rows, 64, 64, dtype=torch.bfloat16, device=device)
    for row in range(rows):
        latent = torch.randn(context, 512, generator=gen, device=device)
        latent[:, outliers] *= factor
        latent = latent.to(torch.bfloat16)
        rope = torch.randn(context, 64, generator=gen, device=device).to(torch.bfloat16)
        mla.write_pages(cache, latent, rope, source, table[row].contiguous())
        open_latent[row, :63], open_rope[row, :63] = latent[-64:-1], rope[-64:-1]
    appender.load_open_pages(open_latent, open_rope)
    new_latent, new_rope = latent[-1:].expand(rows, 512).contiguous(), rope[-1:].expand(rows, 64).contiguous()
    del latent, rope, open_latent, open_rope
    seq_lens = torch.full((rows,), context, dtype=torch.int32, device=device)
    lens_before = seq_lens - 1
    q_latent = torch.randn(rows, MLA_HEADS, 512, generator=gen, device=device).to(torch.bfloat16)
    q_rope = torch.randn(rows, MLA_HEADS, 64, generator=gen, device=device).to(torch.bfloat16)
    error = torch.zeros(1, dtype=torch.int32, device=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(value: float) -> float:
        if world == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    scratch = mla.MLAScratch(rows, MLA_HEADS, splits, device)
    result = torch.empty(rows, MLA_HEADS, 512, dtype=torch.bfloat16, device=device)

    def decode(ql, qr):
        appender.append(cache, new_latent, new_rope, lens_before, table, error_word=error)
        return mla.mla_decode(ql, qr, cache, table, seq_lens, softmax_scale=MLA_SCALE, num_splits=splits,
                              error_word=error, out=result, scratch=scratch)

    # ---- device-resident step: one-token append (3 launches), query quantize, decode (+ merge).
    # The launches are issued one by one so that CUDA events on the launching stream bracket the decode
    # kernel inside the very region the step time comes from.
    import bdfp4

    stream = torch.cuda.current_stream(device)
    codes, scales = scratch.codes, scratch.scales
    a = bdfp4.MlaDecodeArgs()
    a.rows, a.heads_q = rows, MLA_HEADS
    a.query_codes, a.query_scales, a.query_rope = codes.data_ptr(), scales.data_ptr(), q_rope.data_ptr()
    a.key_codes, a.key_scales = cache.key_codes.data_ptr(), cache.key_scales.data_ptr()
    a.value_codes, a.value_scales = cache.value_codes.data_ptr(), cache.value_scales.data_ptr()
    a.key_codes_pitch = a.key_scales_pitch = a.value_codes_pitch = a.value_scales_pitch = cache.pitch
    a.rope_pages, a.rope_pitch, a.pages = cache.rope.data_ptr(), cache.pitch, cache.pages
    a.page_table, a.page_table_stride, a.seq_lens = table.data_ptr(), table.stride(0), seq_lens.data_ptr()
    a.softmax_scale, a.p_scale_mode, a.p_scale_tau = MLA_SCALE, 2, 21.0 / 1024.0
    a.num_splits = splits
    a.error_word = error.data_ptr()
    if splits == 1:
        a.out = result.data_ptr()
    else:
        a.partial_out, a.partial_lse = scratch.partial_out.data_ptr(), scratch.partial_lse.data_ptr()

    def device_step(events=None):
        appender.append(cache, new_latent, new_rope, lens_before, table, error_word=error)
        mla.quantize_query(q_latent, out=(codes, scales))
        if events:
            events[0].record()
        bdfp4.mla_decode(a, stream.cuda_stream)
        if events:
            events[1].record()
        if splits > 1:
            bdfp4.mla_combine(scratch.partial_out, scratch.partial_lse, splits, rows, MLA_HEADS, result,
                              stream.cuda_stream)

    for _ in range(args.warmup):
        device_step()
    sampler = ClockSampler(local_rank)
    sampler.__enter__()
    resident = TimedRounds(args.steps, args.min_seconds, sampler, barrier, max_over_ranks)
    resident.run(device_step, lambda: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)))
    step_ms = max_over_ranks(resident.median_ms())
    kernel_ms = max_over_ranks(resident.median_kernel_ms())
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    # ---- end to end: pinned host query in, pinned host output back, every step
    host_q = torch.empty(rows, MLA_HEADS, 576, dtype=torch.bfloat16).pin_memory()
    host_q[..., :512].copy_(q_latent.cpu())
    host_q[..., 512:].copy_(q_rope.cpu())
    host_new = torch.empty(rows, 576, dtype=torch.bfloat16).pin_memory()  # the step's new token per row
    host_new[:, :512].copy_(new_latent.cpu())
    host_new[:, 512:].copy_(new_rope.cpu())
    device_new = torch.empty(rows, 576, dtype=torch.bfloat16, device=device)
    host_out = torch.empty(rows, MLA_HEADS, 512, dtype=torch.bfloat16).pin_memory()
    device_q = torch.empty(rows, MLA_HEADS, 576, dtype=torch.bfloat16, device=device)
    dense_latent = torch.empty(rows, MLA_HEADS, 512, dtype=torch.bfloat16, device=device)
    dense_rope = torch.empty(rows, MLA_HEADS, 64, dtype=torch.bfloat16, device=device)

    def e2e_step(_events=None):
        device_q.copy_(host_q, non_blocking=True)
        device_new.copy_(host_new, non_blocking=True)
        new_latent.copy_(device_new[:, :512])
        new_rope.copy_(device_new[:, 512:])
        dense_latent.copy_(device_q[..., :512])
        dense_rope.copy_(device_q[..., 512:])
        host_out.copy_(decode(dense_latent, dense_rope), non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        e2e_step()
    end_to_end = TimedRounds(args.steps, args.min_seconds, sampler, barrier, max_over_ranks)
    end_to_end.run(e2e_step)
    sampler.__exit__(None, None, None)
    e2e_ms = max_over_ranks(end_to_end.median_ms())

    tokens = rows * context
    algorithmic = tokens * MLA_TOKEN_BYTES + rows * MLA_HEADS * (576 + 512) * 2
    cache_bytes = tokens * MLA_CACHE_TOKEN_BYTES
    peak, peak_kind = measured_peak_gbs()
    achieved = algorithmic / (kernel_ms * 1e-3) / 1e9
    if rank == 0:
        line = {
            "metric": "mla_decode_attn_us_per_step", "value": step_ms * 1e3, "unit": "us/step", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp4(e2m1)+ue4m3 and bf16 rope / f32 accumulate",
            "data": "synthetic",
            "config": {
                "workload": MLA_WORKLOAD + ("" if (total_rows, context) == (MLA_BATCH, MLA_CONTEXT)
                                            else f" [shape overridden: batch {total_rows}, context {context}]"),
                "partition": f"{rows} of {total_rows} rows per rank, no collective", "num_splits": splits,
                "l2": "inputs (1.5 GB per step over all ranks) exceed the 126 MB L2; no flush needed",
                "step": "append one token per row (stage, re-quantize the open page, rope block), query quantize, decode (+ merge)",
                "e2e": "every step: H2D of the pinned query and new token, the step, D2H of the output into pinned memory, synchronise",
            },
            "timing": {"statistic": "median over rounds of K steps, max over ranks", "rounds": len(resident.rounds),
                       "timed_region_s": sum(r["ms_per_step"] for r in resident.rounds) * args.steps * 1e-3,
                       "clock_bins": resident.clock_bins()},
            "decode_kernel_us": kernel_ms * 1e3,
            "cache_read_gb_s": cache_bytes / (kernel_ms * 1e-3) / 1e9,
            "roofline_on_cache_bytes": {"achieved": cache_bytes / (kernel_ms * 1e-3) / 1e9, "peak": peak,
                                        "frac": cache_bytes / (kernel_ms * 1e-3) / 1e9 / peak,
                                        "note": "704 B per token: what this cache layout holds and the kernel reads"},
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                # DRAM traffic per launch: both latent copies are read (704 B per token); measured by ncu on
                # the 8,192-token case as 1.01 x the cache bytes walked
                "traffic": cache_bytes * 1.01, "peak_kind": f"of {peak_kind}", "kernel": "mla::decode_kernel",
                "algorithmic_bytes_per_launch": algorithmic,
                "note": "algorithmic bytes count one latent copy (416 B per token); this cache holds two (704 B)",
            },
            "e2e": {"value": e2e_ms * 1e3, "unit": "us/step", "h2d_bytes_per_step": (host_q.numel() + host_new.numel()) * 2,
                    "d2h_bytes_per_step": host_out.numel() * 2},
            "gpu_launches": args.steps * (5 if splits == 1 else 6) * len(resident.rounds),
            "clocks": sampler.summary(),
            "device_errors": int(error.item()),
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = mla_cpu_baseline(rows, budget_s=12.0)[1]
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()



# ---------------------------------------------------------------------------------------------
# One very long sequence split along the KV axis over the ranks (`--workload longseq`): 1,048,576
# tokens of the Qwen3-4B shape (32 query / 8 KV heads); the one path with a collective
# ---------------------------------------------------------------------------------------------

def run_longseq(args) -> None:
    import torch.distributed as dist

    from bdfp4.distributed import KvShardedDecoder
    from bdfp4.workload import build_workload

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run, one rank per GPU")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    total = args.context if args.context != CONTEXT else LONG_TOKENS
    shard = total // world // 128 * 128
    # every rank holds its shard as a cache of its own; the rolling tail (128 tokens here) and the sink
    # exist on every rank's workload but only their owners pass them on
    w = build_workload(rows=1, heads_q=HEADS_Q, heads_kv=HEADS_KV, seq_lens=[shard + 128], sink_tokens=SINK_ROWS,
                       seed=7000 + rank, device=device, key_scale_mode="four_six", value_scale_mode="amax6",
                       rotate=True, page_tokens=args.page_tokens)
    w.seqused_sink.clamp_(max=SINK_USED)
    zeros = torch.zeros_like(w.seqused_residual)
    owner_tail, owner_sink = rank == world - 1, rank == 0
    out = torch.empty(1, HEADS_Q, 128, dtype=torch.bfloat16, device=device)
    no_sink = torch.zeros_like(w.seqused_sink)
    decoder = KvShardedDecoder(
        *w.regions, w.page_table, w.seqused_fp4, heads_q=HEADS_Q, residual_key_pages_bf16=w.tail_key[0],
        residual_value_pages_bf16=w.tail_value[0], residual_page_ids=w.slot_ids,
        seqused_residual=w.seqused_residual if owner_tail else zeros,
        seqused_sink=w.seqused_sink if owner_sink else no_sink, query_terms=2, query_rotation="hadamard", out=out,
        num_splits=args.splits or None, exchange=args.exchange)

    def step():
        return decoder(w.query)

    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local_rank)
    sampler.__enter__()
    dist.barrier()
    torch.cuda.synchronize()
    sampler.open_window()
    begin.record()
    for _ in range(args.steps):
        step()
    end.record()
    torch.cuda.synchronize()
    dist.barrier()
    sampler.close_window()
    sampler.__exit__(None, None, None)
    t = torch.tensor([begin.elapsed_time(end) / args.steps], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_ms = float(t.item())
    shard_bytes = w.algorithmic_bytes()
    peak, peak_kind = measured_peak_gbs()
    if rank == 0:
        print(json.dumps({
            "metric": "kv_sharded_decode_us_per_step", "value": step_ms * 1e3, "unit": "us/step", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp4(e2m1)+ue4m3 / f32 accumulate", "data": "synthetic",
            "config": {"workload": f"one sequence of {shard * world + 128:,} tokens, 32 query / 8 KV heads, {args.page_tokens}-token "
                                   f"pages, split along the KV axis over {world} ranks; per step: query quantize, shard "
                                   "decode (split again inside the rank), then " +
                                   ("ONE kernel that folds the rank's parts, stores its [O | LSE] record into every "
                                    "rank's memory over NVLink, waits for the others' and merges"
                                    if args.exchange == "peer" else
                                    "local merge, one NCCL all-gather of [O | LSE] records, merge"),
                       "tokens_per_rank": shard, "exchange": args.exchange},
            "gpu_launches": args.steps * (3 if args.exchange == "peer" else 4),
            "hbm_tb_s": shard_bytes * world / (step_ms * 1e-3) / 1e12,
            "roofline": {"bound": "hbm", "achieved": shard_bytes / (step_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": shard_bytes / (step_ms * 1e-3) / 1e9 / peak, "traffic": None,
                         "peak_kind": f"of {peak_kind}", "kernel": "whole step (per rank)",
                         "algorithmic_bytes_per_launch": shard_bytes},
            "clocks": sampler.summary(),
        }))
    decoder.close()
    dist.destroy_process_group()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20, help="steps per timed round")
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--min-seconds", type=float, default=1.0,
                        help="rounds of --steps steps are repeated until this much device time has been measured")
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--context", type=int, default=CONTEXT, help="override the context length (profiling only)")
    parser.add_argument("--batch", type=int, default=0, help="override the batch (profiling only)")
    parser.add_argument("--heads-kv", type=int, default=0, help="override the KV head count (profiling only)")
    parser.add_argument("--heads-q", type=int, default=0, help="override the query head count (profiling only)")
    parser.add_argument("--splits", type=int, default=0, help="override the split-KV count")
    parser.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                        help="the exchange step of the KV-sharded sequence (longseq, mixed): 'peer' = one kernel "
                             "that stores the [O | LSE] records into the other ranks' memory and merges "
                             "(bdfp4_exchange_merge), 'nccl' = fold kernel + all-gather + merge kernel")
    parser.add_argument("--kv-groups", type=int, default=0,
                        help="ranks along the KV-head axis (default: as many as there are KV heads, then rows)")
    parser.add_argument("--bf16-cost", type=int, default=-1,
                        help="pages split 0 is charged for the tail and sink (default: the library's)")
    parser.add_argument("--scale-mode", default="nvfp4",
                        choices=["nvfp4", "mxfp4_ocp", "mxfp4_round_up", "mxfp4_search"],
                        help="cache and query format of the GQA workloads: NVFP4 (K four_six, V and Q amax6) or "
                             "MXFP4 with one E8M0 rule for all three (128-token pages only)")
    parser.add_argument("--page-tokens", type=int, default=64, choices=[64, 128],
                        help="tokens per cache page: 64 as the benchmark configuration names it, or the "
                             "reference's 128")
    parser.add_argument("--fused-merge", action="store_true",
                        help="merge split-KV partials inside the decode kernel instead of launching the merge "
                             "kernel (measured no faster)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-live-copy", action="store_true",
                        help="skip the sustained device-to-device copy measured for context beside the roofline")
    parser.add_argument("--verify", type=int, default=4, metavar="TILES",
                        help="after the timed regions, compare this many sampled (row, KV head) tiles of one decode "
                             "with the CPU oracle and report the errors (0: skip)")
    parser.add_argument("--workload", default="gqa", choices=["gqa", "cfg1", "cfg3", "mixed", "mla", "longseq"],
                        help="gqa: the headline Qwen3-4B-shaped step; cfg1: batch 4 with short contexts; cfg3: eight "
                             "query heads per KV head, 131,072 tokens; mixed: 256 Zipf-length sequences plus one "
                             "1M-token sequence split along the KV axis; mla: the latent-cache decode; longseq: the "
                             "1M-token sequence alone")
    args = parser.parse_args()
    if args.warmup < 3:
        print(f"bench.py: --warmup {args.warmup} is below the 3 warm-up steps a reportable number needs; "
              "running as asked", file=sys.stderr)
    if args.workload == "longseq":
        run_longseq(args)
    elif args.workload == "mla":
        run_mla_reference(args) if args.impl == "reference" else run_mla(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gqa(args)


if __name__ == "__main__":
    main()
