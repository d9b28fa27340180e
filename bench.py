#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on the LFM2-1.2B shape with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096]
                    [--layers L] [--impl ours|reference]

Prints ONE JSON line. ``value`` is decoded tokens per second at the given batch, timed on the
device over exactly K decode steps (each a CUDA-graph replay of the engine's own step, the
chosen token fed to the next step on the device). ``e2e`` is the same through the Python
entry point (``Engine.step``), token ids crossing the host in both directions every step.
``prefill`` is one 2,048-token prompt through the step function. ``roofline`` relates the
decode step to the bytes it has to read: every weight once and the cache of the live
requests. ``points`` holds decode at batch 1, 16, 32 and 64, at contexts of 512 and 32,768, and
for the LFM2-700M and LFM2-350M shapes.

Two more workloads, each printing one JSON line of its own (the default line is unchanged):

    python bench.py --case batching     continuous batching of 128 requests at the LFM2-700M shape
    python bench.py --case long         4 x 32,768-token prompts at the LFM2-350M shape, then decoding
    python bench.py --case lamisun      Lamisun beside LFM2 at equal width, depth and vocabulary:
                                        decode and prefill tokens/s, and the new kernels alone
    python bench.py --case tirudra      Tirudra beside Farorax at equal width, depth and vocabulary:
                                        decode and prefill tokens/s, and the new kernels alone
    python bench.py --case farorax      Farorax beside Galarax at equal width, depth and vocabulary:
                                        decode and prefill tokens/s, and the new kernels alone
    python bench.py --case galarax      Galarax beside LFM2 at equal width, depth and vocabulary:
                                        decode and prefill throughput, and its new kernels alone

Data: seeded uniform-random token ids and N(0, 0.02) weights (norms 1 + N(0, 0.1)); there
are no checkpoints offline. Working set per step (2.3 GB of weights) is far larger than L2,
so no flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# BASELINE.json configs[2]: LFM2-1.2B
LFM2_1_2B = dict(
    model_type="lfm2", num_hidden_layers=16,
    layer_types=["conv", "conv", "full_attention", "conv", "conv", "full_attention", "conv",
                 "conv", "full_attention", "conv", "full_attention", "conv", "full_attention",
                 "conv", "full_attention", "conv"],
    hidden_size=2048, num_attention_heads=32, num_key_value_heads=8,
    block_auto_adjust_ff_dim=True, block_ff_dim=12288, block_multiple_of=256,
    block_ffn_dim_multiplier=1.0, vocab_size=65536, rope_theta=1000000.0, conv_L_cache=3,
    conv_bias=False, tie_embedding=True, norm_eps=1e-5, max_position_embeddings=128000)


def _variant(**changes):
    return {**LFM2_1_2B, **changes}


# BASELINE.json configs[3] and configs[4]: same layer kinds, other widths
LFM2_700M = _variant(hidden_size=1536, num_attention_heads=24, block_ff_dim=10240)
LFM2_350M = _variant(hidden_size=1024, num_attention_heads=16, block_ff_dim=6656)
PAGE_SIZE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in data.items() if k in out})
            out["source"] = "measured"
            return out
        except (ValueError, TypeError):
            pass
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu=None):
        """``gpu``: what nvidia-smi's -i takes (index or UUID); None: the current CUDA device."""
        self.samples, self.times, self.reasons, self.max_mhz = [], [], set(), None
        self._process = None
        self._thread = None
        self.gpu = gpu

    def _current_gpu(self):
        if self.gpu is not None:
            return str(self.gpu)
        try:
            import torch
            return f"GPU-{torch.cuda.get_device_properties(torch.cuda.current_device()).uuid}"
        except Exception:           # noqa: BLE001
            return "0"

    def start(self):
        try:
            self._process = subprocess.Popen(
                ["nvidia-smi", "-i", self._current_gpu(), f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()

    def _read(self):
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self._process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                self.samples.append(float(parts[0]))
                self.max_mhz = float(parts[1])
            except ValueError:
                continue
            self.times.append(time.perf_counter())
            for name, value in zip(names, parts[2:6]):
                if value.lower().startswith("active"):
                    self.reasons.add(name)

    def stop(self, load_began=None, region=None):
        """``load_began``: when the GPU began to run the measured kind of step without a pause
        (samples before that describe an idle GPU and are left out of the median);
        ``region``: (begin, end) of the timed steps on the host's clock."""
        if self._process is not None:
            self._process.terminate()
            try:
                self._process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._process.kill()
        loaded = [s for s, t in zip(self.samples, self.times)
                  if load_began is None or t >= load_began + 0.06]
        inside = sum(1 for t in self.times if region and region[0] <= t <= region[1] + 0.06)
        return {"sm_mhz": statistics.median(loaded) if loaded else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples), "samples_under_load": len(loaded),
                "samples_in_timed_region": inside,
                "how": "nvidia-smi every 200 ms (a query can hold the GPU up for a millisecond, so "
                       "not more often) while the same decode steps run untimed for about a "
                       "second directly before the timed steps, and through them"}


def reference_arm():
    """The reference is Apple-MLX only: it pins mlx / mlx-metal wheels that exist for macOS
    on Apple silicon, and its model classes import mlx.nn. Nothing of it can run here."""
    reason = ("reference needs Apple MLX (mlx==0.32.2, mlx-metal; Metal GPU); no wheel exists "
              "for Linux/CUDA and none is in the offline wheelhouse")
    marker = ROOT / "baseline" / "_ref"
    if marker.is_dir():
        try:
            sys.path.insert(0, str(marker))
            import mlx.core  # noqa: F401
            reason = "mlx imported but the reference has no CUDA path; not run"
        except Exception as error:           # noqa: BLE001
            reason += f" (import mlx: {type(error).__name__})"
    print(json.dumps({"impl": "reference", "unavailable": reason}))
    return 0


def build_engine(config, layers, batch, context, steps_ahead, *, capacity=None, batching=None,
                 name="random-lfm2-1.2b"):
    import torch

    from mlx_one_b200 import BatchingConfig, CacheConfig, Engine
    from mlx_one_b200.config import get_architecture
    from mlx_one_b200.engine.loading import LoadedModel, build_model
    from mlx_one_b200.weights import random_tensors

    data = dict(config)
    if layers < data["num_hidden_layers"]:
        data["layer_types"] = data["layer_types"][:layers]
        data["num_hidden_layers"] = layers
    architecture = get_architecture(data["model_type"])
    typed = architecture.config_class.from_dict(data)
    spec = architecture.describe(typed)
    tensors = random_tensors(spec, seed=0, dtype=torch.bfloat16, device="cuda:0")
    model = build_model(spec, tensors, "bfloat16", "cuda:0")
    del tensors
    loaded = LoadedModel(Path(name), architecture, typed, spec, model)
    if capacity is None:
        capacity = batch * (-(-(context + steps_ahead + 128) // 64) * 64) + PREFILL_TOKENS + 64
    if batching is None:
        batching = BatchingConfig(max_sequences=batch, queue_size=batch + 1,
                                  prefill_chunk_size=2048, max_scheduled_tokens=4096,
                                  max_prefill_tokens=4096)
    return Engine(loaded, batching_config=batching,
                  cache_config=CacheConfig(block_size_tokens=PAGE_SIZE, capacity_tokens=capacity,
                                           max_requests=batch + 1))


def model_flops(spec, tokens):
    """Matrix-product and attention flops of one whole-prompt step (one logits row)."""
    from mlx_one_b200.parts.model import expected_tensors

    import re

    flops = 0
    used = {}                   # layer prefix -> share of its routed experts that a token uses
    for layer in spec.layers:
        part = layer.feed_forward
        if part is not None and part.kind == "routed":
            used[layer.prefix + part.prefix] = part["top"] / part["experts"]
    for name, tensor in expected_tensors(spec).items():
        if len(tensor.shape) == 2 and name != spec.embedding and name != spec.head \
                and not name.endswith(("conv.conv", ".conv", ".router", ".canon1", ".canon2")) \
                and name != "bigram" and name not in spec.vectors:
            share = 1.0
            found = re.match(r"(.*\.)e\d+\.(gate|up|down)$", name)
            if found and found.group(1) in used:
                share = used[found.group(1)]
            flops += int(2 * tokens * tensor.shape[0] * tensor.shape[1] * share)
    flops += 2 * spec.vocab_size * spec.hidden_size          # one row of logits
    for call in spec.order:
        mixer = spec.layers[call.layer].mixer
        mixers = [part for _, part, _ in mixer["branches"]] if mixer.kind == "parallel" else [mixer]
        for part in mixers:
            if part.kind == "attention":
                width = part["heads"] * part["head_dim"]
                window = part.get("window") or tokens
                kept = part.get("keep_first") or 0
                seen = sum(min(i + 1, window + min(kept, max(i + 1 - window, 0))) for i in range(tokens))
                flops += 4 * width * seen                       # causal (windowed) QK^T and PV
            elif part.kind == "latent_attention":
                # every head's query against the one row per token, and the weights' average of
                # the latents
                row = part["latent"] + part["rot_dim"]
                flops += 2 * part["heads"] * (row + part["latent"]) * tokens * (tokens + 1) // 2
            elif part.kind == "differential_attention":
                chunk = part.get("chunk") or tokens
                seen = sum(i % chunk + 1 for i in range(tokens))
                flops += 4 * part["heads"] * (part["head_dim"] + part["value_dim"]) * seen
            elif part.kind == "lightning":
                # 32-bit multiply-adds of the recurrence (not tensor-core work, but work)
                flops += 4 * tokens * part["heads"] * part["key_dim"] * part["value_dim"]
            elif part.kind == "mamba2":
                flops += 4 * tokens * part["heads"] * part["state"] * part["value_dim"]
    return flops


def random_prompts(vocab, count, length, seed):
    import torch

    generator = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=generator).tolist() for _ in range(count)]


def fill_requests(engine, prompts, ids):
    """Runs the prompts through the step function, several requests a step, and returns the
    first decoded token of each."""
    from mlx_one_b200.engine.runner import StepEntry

    runner, cache = engine.runner, engine.cache
    firsts = {}
    chunk = 1024
    for request_id in ids:
        cache.open(request_id)
    longest = max(len(p) for p in prompts)
    group = max(1, 4096 // chunk)
    for base in range(0, len(ids), group):
        members = list(range(base, min(base + group, len(ids))))
        for at in range(0, longest, chunk):
            entries = []
            for m in members:
                part = prompts[m][at:at + chunk]
                if part:
                    last = at + chunk >= len(prompts[m])
                    entries.append(StepEntry(ids[m], part, (len(part) - 1,) if last else ()))
            logits = runner.step(entries)
            if logits is not None:
                chosen = engine.model.ops.argmax(logits).tolist()
                for entry, token in zip([e for e in entries if e.want], chosen):
                    firsts[entry.request_id] = token
    return [firsts[i] for i in ids]


def time_decode(engine, batch, context, warmup, steps, seed, sampler=None):
    """Device-timed decode: ``steps`` graph replays after ``warmup``; contexts end at
    ``context``. Returns (seconds, clock record, mean context, kernels launched per step)."""
    import torch

    from mlx_one_b200.engine.runner import StepEntry

    vocab = engine.model.spec.vocab_size
    load_steps = 0
    if sampler:
        load_steps = max(min(2048, context - warmup - steps - 65), 0) // 64 * 64
    prompt_length = context - max(warmup, 3) - load_steps - steps - 2
    ids = [f"decode{batch}_{i}" for i in range(batch)]
    prompts = random_prompts(vocab, batch, prompt_length, seed)
    firsts = fill_requests(engine, prompts, ids)
    runner = engine.runner
    entries = [StepEntry(i, [t]) for i, t in zip(ids, firsts)]
    # the kernels of one decode step at this batch and context, counted where they are launched
    # (or captured): the first step, alone
    before = engine.model.ops.launches
    last = runner.decode_steps(entries, 1)[-1].tolist()
    launches_per_step = engine.model.ops.launches - before
    entries = [StepEntry(i, [t]) for i, t in zip(ids, last)]
    chosen = runner.decode_steps(entries, max(warmup, 3))
    torch.cuda.synchronize()
    last = chosen[-1].tolist()
    entries = [StepEntry(i, [t]) for i, t in zip(ids, last)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    load_began = None
    if sampler:
        # The timed region may last a few milliseconds, less than one sample of nvidia-smi. So the
        # clocks are sampled while the same steps run, untimed, for a second or more before it
        # (the prompts are that much shorter, so the timed steps end at ``context`` all the same).
        sampler.start()
        time.sleep(0.25)
        load_began = time.perf_counter()
        for _ in range(load_steps // 64):
            last = runner.decode_steps(entries, 64)[-1].tolist()
            entries = [StepEntry(i, [t]) for i, t in zip(ids, last)]
    torch.cuda.synchronize()
    began = time.perf_counter()
    # (the events are recorded around the steps' launches, after the host has packed the loop's
    # metadata: exactly `steps` steps lie between them)
    runner.decode_steps(entries, steps, events=(start, stop))
    torch.cuda.synchronize()
    ended = time.perf_counter()
    seconds = start.elapsed_time(stop) / 1e3
    clocks = sampler.stop(load_began, (began, ended)) if sampler else None
    if clocks is not None:
        clocks["untimed_load_steps"] = load_steps
    mean_context = context - 1 - steps / 2
    for request_id in ids:
        engine.cache.close(request_id)
    return seconds, clocks, mean_context, launches_per_step


def time_e2e(engine, batch, context, warmup, steps, seed):
    """Through Engine.step: host token ids in (pinned metadata copy) and out every step."""
    import torch

    from mlx_one_b200 import TextGenerationOptions

    vocab = engine.model.spec.vocab_size
    # prompts finish one after the other (long ones in several portions), so the first request
    # has decoded some tokens when the last one starts; `slack` keeps every request decoding
    # through the timed steps
    slack = batch * (context // PREFILL_TOKENS + 2) + 8
    prompt_length = context - max(warmup, 24) - steps - slack
    prompts = random_prompts(vocab, batch, prompt_length, seed + 1)
    options = TextGenerationOptions(max_tokens=max(warmup, 24) + steps + slack, ignore_eos=True)
    handles = [engine.submit_ids(p, options) for p in prompts]
    from mlx_one_b200.engine.scheduler import Phase
    while any(h.request.phase is not Phase.DECODE for h in handles):
        engine.step()
    # untimed steps until the pipeline of launches ahead is in its steady state (the step's graph
    # is captured at its second occurrence); at least the warm-up asked for
    for _ in range(max(warmup, 24)):
        engine.step()
    torch.cuda.synchronize()
    produced = sum(len(h.request.output) for h in handles)
    began = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - began
    produced = sum(len(h.request.output) for h in handles) - produced
    meta_bytes = engine.runner.last_meta_bytes
    report_bytes = 4 * engine.runner.last_report.numel()      # chosen tokens + the error flag
    assert produced == batch * steps, (produced, batch, steps)
    for handle in handles:
        handle.cancel()
    engine.step()
    return seconds, meta_bytes, report_bytes


def time_prefill(engine, tokens, warmup, repeats, seed):
    import torch

    from mlx_one_b200.engine.runner import StepEntry

    runner, cache = engine.runner, engine.cache
    prompts = random_prompts(engine.model.spec.vocab_size, warmup + repeats, tokens, seed)
    times = []
    for index, prompt in enumerate(prompts):
        request_id = f"prefill{index}"
        cache.open(request_id)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry(request_id, prompt, (tokens - 1,))])
        stop.record()
        torch.cuda.synchronize()
        if index >= warmup:
            times.append(start.elapsed_time(stop) / 1e3)
        cache.close(request_id)
    return statistics.median(times)


# --------------------------------------------------------------------------- other workloads


def batching_workload(vocab, requests, prompt_range, output_range, seed):
    """Seeded requests of the continuous-batching case: (prompt ids, new tokens) with lengths
    uniform in the given ranges (both ends included)."""
    import torch

    generator = torch.Generator().manual_seed(seed)
    draw = lambda low, high: int(torch.randint(low, high + 1, (1,), generator=generator))
    out = []
    for _ in range(requests):
        length, new = draw(*prompt_range), draw(*output_range)
        out.append((torch.randint(0, vocab, (length,), generator=generator).tolist(), new))
    return out


def run_batching(engine, workload):
    """Submits every request of ``workload`` at once and drives the engine until all are done.
    Returns (results in order, seconds on the host's clock around the run, the steps' records)."""
    from mlx_one_b200 import TextGenerationOptions

    import torch

    records = []
    engine.set_trace_sink(records.append)
    torch.cuda.synchronize()
    began = time.perf_counter()
    handles = [engine.submit_ids(prompt, TextGenerationOptions(max_tokens=new, ignore_eos=True))
               for prompt, new in workload]
    engine.run()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - began
    engine.set_trace_sink(None)
    return [handle.result() for handle in handles], seconds, records


def summarize_steps(records):
    """Step records by phase, and a histogram of their token counts."""
    phases = {}
    for record in records:
        entry = phases.setdefault(record["phase"], {"steps": 0, "tokens": 0, "prompt_tokens": 0,
                                                    "requests": 0})
        entry["steps"] += 1
        entry["tokens"] += record["tokens"]
        entry["prompt_tokens"] += record["prompt_tokens"]
        entry["requests"] += record["batch_size"]
    for entry in phases.values():
        entry["mean_tokens"] = round(entry["tokens"] / entry["steps"], 1)
        entry["mean_requests"] = round(entry.pop("requests") / entry["steps"], 1)
    edges = (1, 8, 32, 64, 128, 256, 512, 1024, 1 << 30)
    histogram = {}
    for record in records:
        top = next(e for e in edges if record["tokens"] <= e)
        label = f"<={top}" if top < 1 << 30 else ">1024"
        histogram[label] = histogram.get(label, 0) + 1
    return phases, histogram


def case_batching(args) -> int:
    """BASELINE.json configs[3]: continuous batching of 128 requests at the LFM2-700M shape,
    prompts uniform in [16, 3072] tokens, outputs uniform in [16, 512], prompt portions of 512
    tokens beside the running decodes. The protocol is the reference's for its decode runs
    (src/mlx_one/p1_decode.py:15-107): one warm-up repetition, then ``--repeats`` measured ones
    of the same requests, the median reported; the clock is the host's around submit + run."""
    import torch

    from mlx_one_b200 import BatchingConfig

    peak = peaks()
    requests, sequences = args.requests, args.sequences
    batching = BatchingConfig(max_sequences=sequences, queue_size=requests,
                              prefill_chunk_size=512, max_prefill_tokens=512,
                              max_scheduled_tokens=512 + sequences, timeout=0)
    capacity = sequences * (3072 + 512 + 64)
    engine = build_engine(LFM2_700M, args.layers, sequences, 0, 0, capacity=capacity,
                          batching=batching, name="random-lfm2-700m")
    spec = engine.model.spec
    workload = batching_workload(spec.vocab_size, requests, (16, 3072), (16, 512), seed=123)
    prompt_tokens = sum(len(p) for p, _ in workload)
    new_tokens = sum(n for _, n in workload)
    samples = []
    for repetition in range(args.repeats + 1):
        replays = engine.runner.graph_replays
        results, seconds, records = run_batching(engine, workload)
        assert [r.generation_tokens for r in results] == [n for _, n in workload]
        engine.model.ops.check_errors()
        stats = engine.runtime_stats()
        phases, histogram = summarize_steps(records)
        samples.append({"phase": "warmup" if repetition == 0 else "measured",
                        "seconds": round(seconds, 4), "steps": len(records),
                        "graph_replay_share": round((engine.runner.graph_replays - replays)
                                                    / max(len(records), 1), 3),
                        "by_phase": phases, "tokens_per_step": histogram,
                        "pages_low_water": stats["pages_low_water"][0],
                        "pages_total": stats["pages_total"][0],
                        "graphs_kept": stats["graphs"], "graph_captures_so_far":
                            stats["graph_captures"],
                        "graph_memory_gb": round(stats["graph_memory_bytes"] / 1e9, 2),
                        "device_memory_gb": round(torch.cuda.memory_reserved() / 1e9, 2)})
    measured = sorted(samples[1:], key=lambda sample: sample["seconds"])
    middle = measured[len(measured) // 2]
    line = {
        "case": "batching", "metric": "tokens/s of 128 requests batched continuously "
                                      "(LFM2-700M shape, bf16)",
        "value": round((prompt_tokens + new_tokens) / middle["seconds"], 1),
        "unit": "tokens/s (prompt + generated)",
        "generated_tokens_per_s": round(new_tokens / middle["seconds"], 1),
        "seconds_median": middle["seconds"],
        "seconds_all": [sample["seconds"] for sample in samples[1:]],
        "warmup_seconds": samples[0]["seconds"],
        "requests": requests, "prompt_tokens": prompt_tokens, "generated_tokens": new_tokens,
        "config": {"model": "LFM2-700M shape", "layers": args.layers, "hidden": spec.hidden_size,
                   "ffn_width": spec.layers[0].feed_forward["width"], "vocab": spec.vocab_size,
                   "max_sequences": sequences, "prefill_chunk_size": 512, "page_size": PAGE_SIZE,
                   "prompts": "uniform 16..3072", "outputs": "uniform 16..512",
                   "capacity_tokens": capacity, "peaks": peak["source"]},
        "median_run": middle, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), seeded uniform-random token ids",
    }
    print(json.dumps(line))
    return 0


def case_long(args) -> int:
    """BASELINE.json configs[4]: four requests of 32,768 prompt tokens at the LFM2-350M shape,
    prefilled in portions of 4,096 tokens, then 256 decode steps each. Prefill and decode are
    timed on the device through the step function (CUDA events); the same work is then run
    once more through the entry point on the host's clock."""
    import torch

    from mlx_one_b200 import BatchingConfig, TextGenerationOptions
    from mlx_one_b200.engine.runner import StepEntry

    peak = peaks()
    count, prompt_length, portion, decode = 4, args.context or 32768, 4096, args.steps
    batching = BatchingConfig(max_sequences=count, queue_size=count, prefill_chunk_size=portion,
                              max_prefill_tokens=portion, max_scheduled_tokens=portion + count,
                              timeout=0)
    per_request = -(-(prompt_length + decode + 16) // 64) * 64
    engine = build_engine(LFM2_350M, args.layers, count, 0, 0, capacity=count * per_request + 64,
                          batching=batching, name="random-lfm2-350m")
    model, spec, runner, cache = engine.model, engine.model.spec, engine.runner, engine.cache
    prompts = random_prompts(spec.vocab_size, count, prompt_length, seed=5)
    ids = [f"long{i}" for i in range(count)]
    attention_layers = sum(1 for layer in spec.layers if layer.mixer.kind == "attention")
    heads_width = spec.hidden_size
    linear_flops = model_flops(spec, 1) - 2 * spec.vocab_size * spec.hidden_size \
        - attention_layers * 4 * heads_width

    # prefill, portion by portion, each timed on the device
    portion_ms = []
    firsts = []
    for request_id, prompt in zip(ids, prompts):
        cache.open(request_id)
        for at in range(0, prompt_length, portion):
            part = prompt[at:at + portion]
            last = at + portion >= prompt_length
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            logits = runner.step([StepEntry(request_id, part, (len(part) - 1,) if last else ())])
            stop.record()
            torch.cuda.synchronize()
            if request_id != ids[0]:                          # the first request warms up
                portion_ms.append((at, start.elapsed_time(stop)))
            if last:
                firsts.append(int(model.ops.argmax(logits)[0]))
    pages_held = cache.get(ids[0]).live[0]
    timed_requests = count - 1
    prefill_seconds = sum(ms for _, ms in portion_ms) / 1e3
    prefill_tokens = timed_requests * prompt_length
    flops = timed_requests * sum(
        linear_flops * min(portion, prompt_length - at)
        + attention_layers * 4 * heads_width * sum(range(at + 1, min(at + portion, prompt_length) + 1))
        for at in range(0, prompt_length, portion))
    by_start = {}
    for at, ms in portion_ms:
        by_start.setdefault(at, []).append(ms)
    first_ms = statistics.median(by_start[0])
    last_start = max(by_start)
    last_ms = statistics.median(by_start[last_start])

    # decode: all four together, the chosen token fed back on the device
    entries = [StepEntry(i, [t]) for i, t in zip(ids, firsts)]
    chosen = runner.decode_steps(entries, 3)
    entries = [StepEntry(i, [t]) for i, t in zip(ids, chosen[-1].tolist())]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    runner.decode_steps(entries, decode)
    stop.record()
    torch.cuda.synchronize()
    decode_seconds = start.elapsed_time(stop) / 1e3
    model.ops.check_errors()
    mean_context = prompt_length + 3 + decode / 2
    kv_per_token = engine.cache_bytes_per_token()
    state_bytes = sum(g.storage[:, 0].numel() * g.storage.element_size() for g in cache.states)
    step_bytes = model.weight_bytes() + count * (mean_context * kv_per_token + 2 * state_bytes)
    achieved = step_bytes / (decode_seconds / decode) / 1e9
    for request_id in ids:
        cache.close(request_id)

    # the same through the entry point: submit four requests, run, host clock
    options = TextGenerationOptions(max_tokens=decode + 1, ignore_eos=True)
    records = []
    engine.set_trace_sink(records.append)
    torch.cuda.synchronize()
    began = time.perf_counter()
    handles = [engine.submit_ids(prompt, options) for prompt in prompts]
    engine.run()
    torch.cuda.synchronize()
    e2e_seconds = time.perf_counter() - began
    engine.set_trace_sink(None)
    results = [handle.result() for handle in handles]
    assert all(r.generation_tokens == decode + 1 for r in results)
    model.ops.check_errors()
    phases, histogram = summarize_steps(records)
    # decode through the entry point: the steps in which all four requests decode
    full = [r for r in records if r["phase"] == "decode" and r["batch_size"] == count]
    e2e_decode = None
    if len(full) > 2:
        e2e_decode = round(count * (len(full) - 1) / (full[-1]["committed_at"] - full[0]["committed_at"]), 1)
    stats = engine.runtime_stats()
    line = {
        "case": "long", "metric": "prefill and decode tokens/s at 4 x 32,768 tokens of context "
                                  "(LFM2-350M shape, bf16)",
        "prefill": {"value": round(prefill_tokens / prefill_seconds, 1), "unit": "tokens/s",
                    "tokens": prefill_tokens, "portion": portion,
                    "ms_first_portion": round(first_ms, 3),
                    "ms_last_portion": round(last_ms, 3),
                    "frac": round(flops / prefill_seconds / (peak["bf16_tflops"] * 1e12), 4),
                    "frac_last_portion": round(
                        (linear_flops * portion + attention_layers * 4 * heads_width
                         * sum(range(last_start + 1, last_start + portion + 1)))
                        / (last_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)},
        "decode": {"value": round(count * decode / decode_seconds, 1), "unit": "tokens/s",
                   "steps": decode, "ms_per_step": round(decode_seconds / decode * 1e3, 4),
                   "mean_context": mean_context},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peak["hbm_gbs"], 4),
                     "bytes_per_step": int(step_bytes)},
        "e2e": {"seconds": round(e2e_seconds, 4),
                "value": round(count * (prompt_length + decode + 1) / e2e_seconds, 1),
                "unit": "tokens/s (prompt + generated, host clock around submit + run)",
                "decode_tokens_per_s_all_four": e2e_decode, "by_phase": phases,
                "tokens_per_step": histogram},
        "pages_per_request": pages_held, "pages_low_water": stats["pages_low_water"][0],
        "pages_total": stats["pages_total"][0],
        "config": {"model": "LFM2-350M shape", "layers": args.layers, "hidden": spec.hidden_size,
                   "ffn_width": spec.layers[0].feed_forward["width"], "vocab": spec.vocab_size,
                   "requests": count, "prompt_tokens": prompt_length, "portion": portion,
                   "decode_steps": decode, "page_size": PAGE_SIZE, "peaks": peak["source"]},
        "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), seeded uniform-random token ids",
    }
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------- Galarax beside LFM2


def galarax_shape(width: int, layers: int, vocab: int = 65536) -> dict:
    """A Galarax of the sizes that a model of this width has: heads of 64 for the softmax branch
    (one key head per four query heads, half of a head rotated), heads of 128 x 128 for the delta
    rule (inner width = model width), a feed-forward four times the width."""
    left = {"heads": width // 64, "kv_heads": width // 256, "dim": 64, "vdim": 64,
            "scale": 0.125, "rot": {"base": 1000000.0, "dims": 32, "scaling": {
                "factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    right = {"heads": width // 128, "kv_heads": width // 256, "dim": 128, "vdim": 128, "conv": 4}
    layer = {"type": "parallel", "mixer": {"left": left, "right": right},
             "mlp": {"kind": "dense", "ff": 4 * width}}
    return {"architecture": "Galarax", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "layers": [layer] * layers}


def engine_of(data, batch, context, steps_ahead, name):
    """An engine over random weights for any registered architecture's config.json contents."""
    import torch

    from mlx_one_b200 import BatchingConfig, CacheConfig, Engine
    from mlx_one_b200.config import architecture_key, get_architecture
    from mlx_one_b200.engine.loading import LoadedModel, build_model
    from mlx_one_b200.weights import random_tensors

    architecture = get_architecture(architecture_key(data))
    typed = architecture.config_class.from_dict(data)
    spec = architecture.describe(typed)
    tensors = random_tensors(spec, seed=0, dtype=torch.bfloat16, device="cuda:0")
    model = build_model(spec, tensors, "bfloat16", "cuda:0")
    del tensors
    loaded = LoadedModel(Path(name), architecture, typed, spec, model)
    capacity = batch * (-(-(context + steps_ahead + 128) // 64) * 64) + PREFILL_TOKENS + 64
    batching = BatchingConfig(max_sequences=batch, queue_size=batch + 1, prefill_chunk_size=2048,
                              max_scheduled_tokens=4096, max_prefill_tokens=4096)
    return Engine(loaded, batching_config=batching,
                  cache_config=CacheConfig(block_size_tokens=PAGE_SIZE, capacity_tokens=capacity,
                                           max_requests=batch + 1))


def graph_seconds(fn, copies, inner):
    """Seconds per call of fn(i), i cycling over ``copies`` argument sets, inside a CUDA graph."""
    import torch

    for i in range(min(copies, 3)):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(inner):
            fn(i % copies)
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(5):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / 1e3 / (5 * inner)


def galarax_kernels(width, batch, peak):
    """The kernels that Galarax adds, alone, beside the like kernels of LFM2, for a decode step
    of ``batch`` tokens and a prompt of PREFILL_TOKENS tokens: algorithmic bytes / time against
    the measured copy bandwidth. Arguments rotate over copies that together exceed L2."""
    import torch

    from mlx_one_b200.kernels import default_ops
    from mlx_one_b200.parts import (FixedState, PagedKeyValues, PagedView, StateView,
                                    StepContext)
    from mlx_one_b200.parts.mixers import GatedDeltaRule

    ops, device = default_ops("cuda:0"), "cuda:0"
    ints = lambda values: torch.tensor(values, dtype=torch.int32, device=device)
    bf16 = lambda *shape: torch.randn(*shape, device=device).bfloat16()

    def ctx_of(portions, histories):
        positions, owner, starts = [], [], [0]
        for r, (n, before) in enumerate(zip(portions, histories)):
            positions += list(range(before, before + n))
            owner += [r] * n
            starts.append(starts[-1] + n)
        return StepContext(tokens=len(positions), requests=len(portions),
                           token_ids=ints([0] * len(positions)), positions=ints(positions),
                           token_request=ints(owner), request_start=ints(starts),
                           history=ints(histories), max_portion=max(portions),
                           max_context=max(p + h for p, h in zip(portions, histories)))

    H, G, D, V, taps = width // 128, width // 256, 128, 128, 4
    sizes = dict(heads=H, kv_heads=G, key_dim=D, value_dim=V, taps=taps)
    state_size = GatedDeltaRule.state_size({"heads": H, "kv_heads": G, "key_dim": D,
                                            "value_dim": V, "taps": taps})
    channels = 2 * G * D + H * V
    wide = channels + H * V + 2 * H
    out = {}
    for label, portions, histories in (("decode", [1] * batch, [2048] * batch),
                                       ("prefill", [PREFILL_TOKENS], [0])):
        ctx = ctx_of(portions, histories)
        tokens, requests = ctx.tokens, ctx.requests
        copies = max(2, min(24, int(200e6 // (requests * state_size * 4))))
        state = torch.zeros(copies * requests, state_size, device=device)
        views = [StateView(state, ints(list(range(c * requests, (c + 1) * requests))),
                           FixedState((state_size,), "float32")) for c in range(copies)]
        projected = [bf16(tokens, wide) for _ in range(copies)]
        constants = dict(conv=torch.randn(channels, taps, device=device) * 0.5,
                         a_log=torch.zeros(H, device=device), dt_bias=torch.zeros(H, device=device),
                         norm_weight=torch.ones(V, device=device), eps=1e-6, unit_eps=1e-6,
                         ctx=ctx, write=True, **sizes)
        seconds = graph_seconds(lambda i: ops.gated_delta_rule(projected[i], view=views[i],
                                                               **constants), copies, 2 * copies)
        moved = tokens * (wide + H * V) * 2 + 2 * requests * state_size * 4
        out[f"{label}_gated_delta"] = {
            "us": round(seconds * 1e6, 2), "gbs": round(moved / seconds / 1e9, 1),
            "hbm_frac": round(moved / seconds / 1e9 / peak["hbm_gbs"], 4),
            "gflops": round(6.0 * tokens * H * D * V / seconds / 1e9, 1)}
        # LFM2's like kernel: the gated short convolution with its slot
        conv_state = torch.zeros(copies * requests, 2, width, device=device).bfloat16()
        conv_views = [StateView(conv_state, views[c].slots, FixedState((2, width))) for c in range(copies)]
        bcx = [bf16(tokens, 3 * width) for _ in range(copies)]
        kernel = torch.randn(width, 3, device=device)
        seconds = graph_seconds(lambda i: ops.short_conv(bcx[i], kernel=kernel, bias=None, taps=3,
                                                         ctx=ctx, view=conv_views[i], write=True),
                                copies, 2 * copies)
        moved = tokens * 4 * width * 2 + 2 * requests * 2 * width * 2
        out[f"{label}_short_conv_lfm2"] = {
            "us": round(seconds * 1e6, 2), "gbs": round(moved / seconds / 1e9, 1),
            "hbm_frac": round(moved / seconds / 1e9 / peak["hbm_gbs"], 4)}
        # preparation of queries and keys with the page write: general form and LFM2's
        heads, kv_heads, head = width // 64, width // 256, 64
        pages = -(-(histories[0] + portions[0]) // PAGE_SIZE)
        table = ints([[r * pages + b for b in range(pages)] for r in range(requests)])
        kv = torch.zeros(2, requests * pages + 1, kv_heads, PAGE_SIZE, head, device=device).bfloat16()
        view = PagedView(kv, table, PAGE_SIZE, PagedKeyValues(kv_heads, head, None))
        qkv = [bf16(tokens, (heads + 2 * kv_heads) * head) for _ in range(copies)]
        inv_half = torch.rand(16, device=device)
        inv_full = torch.rand(32, device=device)
        ones = torch.ones(head, device=device)
        common = dict(heads=heads, kv_heads=kv_heads, head_dim=head, eps=1e-6, ctx=ctx, view=view,
                      write=True)
        moved = tokens * ((heads + 2 * kv_heads) * head * 2) * 2
        for name, extra in (("qk_prep_general", dict(q_weight=None, k_weight=None, rotary=(inv_half, 32),
                                                     value_dim=head, amplitude=1.2, norm_after=True)),
                            ("qk_prep_lfm2", dict(q_weight=ones, k_weight=ones, rotary=(inv_full, 64)))):
            seconds = graph_seconds(lambda i: ops.qk_norm_rope_store(qkv[i], **common, **extra),
                                    copies, 2 * copies)
            out[f"{label}_{name}"] = {"us": round(seconds * 1e6, 2),
                                      "gbs": round(moved / seconds / 1e9, 1),
                                      "hbm_frac": round(moved / seconds / 1e9 / peak["hbm_gbs"], 4)}
        # the mean of two normed branches into the stream, beside add + RMSNorm
        residual = [torch.zeros(tokens, width, device=device) for _ in range(copies)]
        a, b = [bf16(tokens, width) for _ in range(copies)], [bf16(tokens, width) for _ in range(copies)]
        weight = torch.ones(width, device=device)
        seconds = graph_seconds(lambda i: ops.normed_mean_add(residual[i], [a[i], b[i]],
                                                              [weight, weight], 1e-6), copies, 2 * copies)
        moved = tokens * width * (4 + 4 + 2 + 2)
        out[f"{label}_normed_mean_add"] = {"us": round(seconds * 1e6, 2),
                                           "hbm_frac": round(moved / seconds / 1e9 / peak["hbm_gbs"], 4)}
        seconds = graph_seconds(lambda i: ops.add_rmsnorm(residual[i], a[i], weight, 1e-6,
                                                          torch.bfloat16), copies, 2 * copies)
        moved = tokens * width * (4 + 4 + 2 + 2)
        out[f"{label}_add_rmsnorm_lfm2"] = {"us": round(seconds * 1e6, 2),
                                            "hbm_frac": round(moved / seconds / 1e9 / peak["hbm_gbs"], 4)}
        # the feed-forward's first product with its activation, beside the gated one of equal output
        up = [bf16(4 * width, width) * 0.02 for _ in range(copies)]
        gate_up = [bf16(8 * width, width) * 0.02 for _ in range(copies)]
        x = bf16(tokens, width)
        for name, fn, rows_w in (("up_relu2", lambda i: ops.linear_act(x, up[i], "relu2"), 4 * width),
                                 ("up_swiglu_lfm2", lambda i: ops.linear_swiglu(x, gate_up[i]), 8 * width)):
            seconds = graph_seconds(fn, copies, copies)
            entry = {"us": round(seconds * 1e6, 2)}
            if label == "decode":
                entry["hbm_frac"] = round(rows_w * width * 2 / seconds / 1e9 / peak["hbm_gbs"], 4)
            else:
                entry["tensor_frac"] = round(2.0 * tokens * rows_w * width / seconds / 1e12 /
                                             peak["bf16_tflops"], 4)
            out[f"{label}_{name}"] = entry
        del state, views, projected, conv_state, bcx, kv, qkv, residual, a, b, up, gate_up
        torch.cuda.empty_cache()
    return out


def case_galarax(args) -> int:
    """Galarax beside LFM2 at equal width, depth and vocabulary (random weights): decode tokens/s
    at ``--batch`` and ``--context`` (device-timed graph replays of the engine's step), prefill
    tokens/s of one 2,048-token prompt, each against its bound, and the new kernels alone."""
    import gc

    import torch

    peak = peaks()
    warmup, steps = max(args.warmup, 3), min(args.steps, 128)
    context = args.context or 2048
    layers = min(args.layers, 8)
    results = {}
    for width, twin in ((1024, LFM2_350M), (2048, LFM2_1_2B)):
        lfm2 = dict(twin)
        lfm2["layer_types"] = lfm2["layer_types"][:layers]
        lfm2["num_hidden_layers"] = layers
        for label, data in ((f"galarax_w{width}", galarax_shape(width, layers)),
                            (f"lfm2_w{width}", lfm2)):
            engine = engine_of(data, args.batch, context, warmup + steps, f"random-{label}")
            model, spec = engine.model, engine.model.spec
            weight_bytes = model.weight_bytes()
            kv_per_token = engine.cache_bytes_per_token()
            state_bytes = sum(g.storage[:, 0].numel() * g.storage.element_size()
                              for g in engine.cache.states)
            seconds, _, mean_context, launches = time_decode(engine, args.batch, context, warmup,
                                                             steps, seed=3)
            step_bytes = weight_bytes + args.batch * (mean_context * kv_per_token + 2 * state_bytes)
            prefill_seconds = time_prefill(engine, PREFILL_TOKENS, 2, 3, seed=5)
            flops = model_flops(spec, PREFILL_TOKENS)
            results[label] = {
                "layers": layers, "weight_mb": round(weight_bytes / 1e6, 1),
                "state_mb_per_request": round(state_bytes / 1e6, 2),
                "decode_tokens_per_s": round(args.batch * steps / seconds, 1),
                "decode_ms_per_step": round(seconds / steps * 1e3, 4),
                "decode_hbm_frac": round(step_bytes / (seconds / steps) / 1e9 / peak["hbm_gbs"], 4),
                "launches_per_step": launches,
                "prefill_tokens_per_s": round(PREFILL_TOKENS / prefill_seconds, 1),
                "prefill_ms": round(prefill_seconds * 1e3, 3),
                "prefill_tensor_frac": round(flops / prefill_seconds / (peak["bf16_tflops"] * 1e12), 4)}
            del engine, model
            gc.collect()
            torch.cuda.empty_cache()
        results[f"kernels_w{width}"] = galarax_kernels(width, args.batch, peak)
    print(json.dumps({"case": "galarax", "batch": args.batch, "context": context, "steps": steps,
                      "warmup": warmup, "dtype": "bf16", "peaks": peak["source"],
                      "data": "synthetic: random weights, seeded uniform-random token ids",
                      "results": results}))
    return 0


# --------------------------------------------------------------------------- Farorax beside Galarax


def farorax_shape(width: int, layers: int, vocab: int = 65536) -> dict:
    """A Farorax of the sizes that a model of this width has: one attention layer in four (heads
    of 64, one key head per four query heads, a window of 1024, the whole head rotated), the
    others lightning layers with heads of 128 x 128 (inner width = model width); feed-forwards in
    turn gated of four times the width and eight routed experts of the model's width of which a
    token uses two, beside a shared one."""
    attention = {"heads": width // 64, "kv_heads": width // 256, "dim": 64, "vdim": 64,
                 "scale": 0.125, "mask": {"size": 1024},
                 "rot": {"base": 1000000.0, "dims": 64, "scaling": {
                     "factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    heads = width // 128
    lightning = {"heads": heads, "dim": 128, "vdim": 128,
                 "decay": [1.0 - 2.0 ** (-3 - 5 * h / max(heads - 1, 1)) for h in range(heads)]}
    dense = {"kind": "dense", "ff": 4 * width}
    routed = {"kind": "moe", "expert": {"ff": width}, "shared": {"ff": width},
              "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 2}}}
    entries = []
    for index in range(layers):
        mixer = ("attention", attention) if index % 4 == 0 else ("lightning", lightning)
        entries.append({"type": mixer[0], "mixer": mixer[1], "mlp": routed if index % 2 else dense})
    return {"architecture": "Farorax", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "residual_mult": 0.5, "logit_softcap": 50.0, "layers": entries}


def farorax_kernels(width, batch, peak):
    """The kernels that Farorax adds, alone, beside the like kernels of Galarax, for a decode step
    of ``batch`` tokens and a prompt of PREFILL_TOKENS tokens: algorithmic bytes (or flops) /
    time against the measured peaks. Arguments rotate over copies that together exceed L2."""
    import torch

    from mlx_one_b200.kernels import default_ops
    from mlx_one_b200.parts import (FixedState, PagedKeyValues, PagedView, StateView,
                                    StepContext)
    from mlx_one_b200.parts.mixers import GatedDeltaRule

    ops, device = default_ops("cuda:0"), "cuda:0"
    ints = lambda values: torch.tensor(values, dtype=torch.int32, device=device)
    bf16 = lambda *shape: torch.randn(*shape, device=device).bfloat16()

    def ctx_of(portions, histories):
        positions, owner, starts = [], [], [0]
        for r, (n, before) in enumerate(zip(portions, histories)):
            positions += list(range(before, before + n))
            owner += [r] * n
            starts.append(starts[-1] + n)
        return StepContext(tokens=len(positions), requests=len(portions),
                           token_ids=ints([0] * len(positions)), positions=ints(positions),
                           token_request=ints(owner), request_start=ints(starts),
                           history=ints(histories), max_portion=max(portions),
                           max_context=max(p + h for p, h in zip(portions, histories)))

    def entry(seconds, moved=None, flops=None):
        out = {"us": round(seconds * 1e6, 2)}
        if moved is not None:
            out["gbs"] = round(moved / seconds / 1e9, 1)
            out["hbm_frac"] = round(moved / seconds / 1e9 / peak["hbm_gbs"], 4)
        if flops is not None:
            out["tflops"] = round(flops / seconds / 1e12, 2)
            out["tensor_frac"] = round(flops / seconds / 1e12 / peak["bf16_tflops"], 4)
        return out

    H, D, V = width // 128, 128, 128
    out = {}
    for label, portions, histories in (("decode", [1] * batch, [2048] * batch),
                                       ("prefill", [PREFILL_TOKENS], [0])):
        ctx = ctx_of(portions, histories)
        tokens, requests = ctx.tokens, ctx.requests
        # ---- lightning attention beside the gated delta rule, equal heads and sizes
        state_size = H * D * V
        copies = max(2, min(24, int(200e6 // (requests * state_size * 4))))
        state = torch.zeros(copies * requests, state_size, device=device)
        views = [StateView(state, ints(list(range(c * requests, (c + 1) * requests))),
                           FixedState((state_size,), "float32")) for c in range(copies)]
        wide = 2 * H * D + 2 * H * V
        projected = [bf16(tokens, wide) for _ in range(copies)]
        decay = torch.full((H,), 0.97, device=device)
        weight = torch.ones(H * V, device=device)
        seconds = graph_seconds(lambda i: ops.lightning_attention(
            projected[i], decay=decay, norm_weight=weight, eps=1e-6, ctx=ctx, view=views[i],
            write=True, heads=H, key_dim=D, value_dim=V), copies, 2 * copies)
        moved = tokens * (wide + H * V) * 2 + 2 * requests * state_size * 4
        out[f"{label}_lightning"] = entry(seconds, moved)
        out[f"{label}_lightning"]["gflops_fma"] = round(4.0 * tokens * H * D * V / seconds / 1e9, 1)
        G, taps = width // 256, 4
        sizes = dict(heads=H, kv_heads=G, key_dim=D, value_dim=V, taps=taps)
        delta_size = GatedDeltaRule.state_size({"heads": H, "kv_heads": G, "key_dim": D,
                                                "value_dim": V, "taps": taps})
        channels = 2 * G * D + H * V
        delta_wide = channels + H * V + 2 * H
        delta_state = torch.zeros(copies * requests, delta_size, device=device)
        delta_views = [StateView(delta_state, views[c].slots, FixedState((delta_size,), "float32"))
                       for c in range(copies)]
        delta_in = [bf16(tokens, delta_wide) for _ in range(copies)]
        constants = dict(conv=torch.randn(channels, taps, device=device) * 0.5,
                         a_log=torch.zeros(H, device=device), dt_bias=torch.zeros(H, device=device),
                         norm_weight=torch.ones(V, device=device), eps=1e-6, unit_eps=1e-6,
                         ctx=ctx, write=True, **sizes)
        seconds = graph_seconds(lambda i: ops.gated_delta_rule(delta_in[i], view=delta_views[i],
                                                               **constants), copies, 2 * copies)
        moved = tokens * (delta_wide + H * V) * 2 + 2 * requests * delta_size * 4
        out[f"{label}_gated_delta_galarax"] = entry(seconds, moved)
        del state, views, projected, delta_state, delta_views, delta_in
        # ---- attention over a window with sinks beside attention without
        heads, kv_heads, head, window = width // 64, width // 256, 64, 1024
        pages = -(-(histories[0] + portions[0]) // PAGE_SIZE)
        table = ints([[r * pages + b for b in range(pages)] for r in range(requests)])
        kv = (torch.randn(2, requests * pages + 1, kv_heads, PAGE_SIZE, head, device=device) * 0.3).bfloat16()
        view = PagedView(kv, table, PAGE_SIZE, PagedKeyValues(kv_heads, head, window))
        q = [bf16(tokens, heads, head) for _ in range(4)]
        sinks = torch.zeros(heads, device=device)
        seen = sum(min(h + i + 1, window) for n, h in zip(portions, histories) for i in range(n))
        moved = requests * min(histories[0] + portions[0], window + portions[0]) * kv_heads * head * 2 * 2 \
            + tokens * heads * head * 2 * 2
        flops = 4.0 * heads * head * seen
        for name, extra in (("attention_sinks", dict(sinks=sinks)), ("attention_plain_galarax", {})):
            seconds = graph_seconds(lambda i: ops.paged_attention(
                q[i], heads=heads, kv_heads=kv_heads, head_dim=head, scale=0.125, window=window,
                ctx=ctx, view=view, **extra), 4, 8)
            out[f"{label}_{name}"] = entry(seconds, moved, flops)
        del kv, q
        # ---- the routed feed-forward beside a gated one of the width a token uses
        experts, top, ff, shared = 8, 2, width, width
        copies = max(2, min(12, int(300e6 // ((experts * ff + shared) * width * 6))))
        stack = experts * ff + shared
        gate_up = [bf16(2 * stack, width) * 0.02 for _ in range(copies)]
        down = [bf16(width, stack) * 0.02 for _ in range(copies)]
        router = torch.randn(experts, width, device=device)
        x = bf16(tokens, width)
        routing = dict(experts=experts, top=top, groups=4, keep=2, group_score=2)

        at = experts * ff
        alone = [(torch.cat([g[at:at + shared], g[stack + at:stack + at + shared]]).contiguous(),
                  d[:, at:].contiguous()) for g, d in zip(gate_up, down)]

        def routed(i):                  # what the routed feed-forward part runs
            weights = ops.route_experts(x, router, **routing)
            if ops.sorts_experts(x, experts=experts, width=ff, top=top, stack=stack):
                return ops.routed_experts_sorted(x, weights, gate_up[i], down[i], experts=experts,
                                                 width=ff, top=top, shared_gate_up=alone[i][0],
                                                 shared_down=alone[i][1])
            gated = ops.linear_swiglu(x, gate_up[i])
            ops.scale_expert_columns(gated, weights, ff)
            return ops.linear(gated, down[i])
        used = top * ff + shared
        seconds = graph_seconds(routed, copies, 2 * copies)
        touched = min(experts, tokens * top) * ff + shared       # rows of weights a step must read
        out[f"{label}_routed_ff"] = entry(seconds, touched * width * 6 if label == "decode" else None,
                                          6.0 * tokens * used * width if label == "prefill" else None)
        dense_up = [bf16(2 * used, width) * 0.02 for _ in range(copies)]
        dense_down = [bf16(width, used) * 0.02 for _ in range(copies)]
        for name, kind in (("gated_ff_gelu", "gelu_tanh"), ("gated_ff_silu_galarax_lfm2", "silu")):
            seconds = graph_seconds(lambda i: ops.linear(ops.linear_gated(x, dense_up[i], kind),
                                                         dense_down[i]), copies, 2 * copies)
            out[f"{label}_{name}"] = entry(seconds, used * width * 6 if label == "decode" else None,
                                           6.0 * tokens * used * width if label == "prefill" else None)
        del gate_up, down, dense_up, dense_down
        # ---- what enters the stream before a pass: the mixing product beside the added vector
        residual = [torch.zeros(tokens, width, device=device) for _ in range(4)]
        delta = [bf16(tokens, width) for _ in range(4)]
        table_e = bf16(4096, width)
        ids = torch.randint(0, 4096, (tokens,), device=device, dtype=torch.int32)
        mix = bf16(width, 2 * width) * 0.02
        vector = torch.zeros(width, device=device)

        def enter(i):
            both = ops.concat_stream(residual[i], delta[i], ids, table_e, torch.bfloat16, delta_scale=0.5)
            return ops.linear(both, mix, vector, out_dtype=torch.float32)
        seconds = graph_seconds(enter, 4, 8)
        out[f"{label}_loop_entry_mix"] = entry(seconds, tokens * width * (4 + 2 + 2 + 4 + 4) + mix.numel() * 2)
        seconds = graph_seconds(lambda i: ops.add_vectors(residual[i], delta[i], ids, table_e, vector), 4, 8)
        out[f"{label}_loop_entry_add_galarax"] = entry(seconds, tokens * width * (4 + 2 + 2 + 4))
        seconds = graph_seconds(lambda i: ops.add_rmsnorm(residual[i], delta[i], vector, 1e-6,
                                                          torch.bfloat16, delta_scale=0.5), 4, 8)
        out[f"{label}_add_rmsnorm_scaled"] = entry(seconds, tokens * width * (4 + 4 + 2 + 2))
        del residual, delta
        torch.cuda.empty_cache()
    return out


def case_farorax(args) -> int:
    """Farorax beside Galarax (the closest of the engine's models: a recurrent mixer with a matrix
    state beside softmax attention) at equal width, depth and vocabulary, random weights: decode
    tokens/s at ``--batch`` and ``--context`` (device-timed graph replays of the engine's step),
    prefill tokens/s of one 2,048-token prompt, each against its bound, and the new kernels alone."""
    import gc

    import torch

    peak = peaks()
    warmup, steps = max(args.warmup, 3), min(args.steps, 128)
    context = args.context or 2048
    layers = min(args.layers, 8)
    results = {}
    for width in (1024, 2048):
        for label, data in ((f"farorax_w{width}", farorax_shape(width, layers)),
                            (f"galarax_w{width}", galarax_shape(width, layers))):
            engine = engine_of(data, args.batch, context, warmup + steps, f"random-{label}")
            model, spec = engine.model, engine.model.spec
            weight_bytes = model.weight_bytes()
            kv_per_token = engine.cache_bytes_per_token()
            state_bytes = sum(g.storage[:, 0].numel() * g.storage.element_size()
                              for g in engine.cache.states)
            seconds, _, mean_context, launches = time_decode(engine, args.batch, context, warmup,
                                                             steps, seed=3)
            step_bytes = weight_bytes + args.batch * (mean_context * kv_per_token + 2 * state_bytes)
            prefill_seconds = time_prefill(engine, PREFILL_TOKENS, 2, 3, seed=5)
            flops = model_flops(spec, PREFILL_TOKENS)
            results[label] = {
                "layers": layers, "weight_mb": round(weight_bytes / 1e6, 1),
                "state_mb_per_request": round(state_bytes / 1e6, 2),
                "decode_tokens_per_s": round(args.batch * steps / seconds, 1),
                "decode_ms_per_step": round(seconds / steps * 1e3, 4),
                "decode_hbm_frac": round(step_bytes / (seconds / steps) / 1e9 / peak["hbm_gbs"], 4),
                "launches_per_step": launches,
                "prefill_tokens_per_s": round(PREFILL_TOKENS / prefill_seconds, 1),
                "prefill_ms": round(prefill_seconds * 1e3, 3),
                "prefill_tensor_frac": round(flops / prefill_seconds / (peak["bf16_tflops"] * 1e12), 4)}
            del engine, model
            gc.collect()
            torch.cuda.empty_cache()
        results[f"kernels_w{width}"] = farorax_kernels(width, args.batch, peak)
    print(json.dumps({"case": "farorax", "batch": args.batch, "context": context, "steps": steps,
                      "warmup": warmup, "dtype": "bf16", "peaks": peak["source"],
                      "data": "synthetic: random weights, seeded uniform-random token ids",
                      "results": results}))
    return 0


# --------------------------------------------------------------------------- Tirudra beside Farorax


def tirudra_shape(width: int, layers: int, vocab: int = 65536) -> dict:
    """A Tirudra of the sizes that a model of this width has: state spaces in every other layer
    (heads of 64 values with states of 128, inner width = model width, four taps), between them in
    turn attention over a window of 1024 that keeps four tokens (heads of 64, one key head per
    four query heads, three taps, the whole head rotated) and attention whose values are its keys;
    eight routed experts of the model's width and two identity outputs of which a token uses
    three, beside a gated shared expert."""
    rot = {"base": 1000000.0, "dims": 64}
    attention = {"heads": width // 64, "kv_heads": width // 256, "dim": 64, "vdim": 64,
                 "scale": 0.125, "conv": 3, "mask": {"size": 1024, "keep_first": 4},
                 "rot": dict(rot, scaling={"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0})}
    shared = {"heads": width // 64, "kv_heads": width // 256, "dim": 64, "vdim": 64, "scale": 0.125,
              "rot": dict(rot, scaling={"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192})}
    space = {"heads": width // 64, "vdim": 64, "state": 128, "groups": 1, "conv": 4,
             "norm_groups": width // 256}
    routed = {"kind": "moe", "expert": {"ff": width}, "shared": {"ff": width},
              "router": {"experts": 8, "top": 3, "identity": 2}}
    entries = []
    for index in range(layers):
        mixer = (("mamba2", space), ("attention", attention), ("mamba2", space),
                 ("attention_2", shared))[index % 4]
        entries.append({"type": mixer[0], "mixer": mixer[1], "mlp": routed})
    return {"architecture": "Tirudra", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "logit_scale": 0.25, "layers": entries}


def tirudra_kernels(width, batch, peak):
    """The kernels that Tirudra adds, alone, beside the like kernels of Farorax, for a decode step
    of ``batch`` tokens and a prompt of PREFILL_TOKENS tokens: algorithmic bytes (or flops) /
    time against the measured peaks. Arguments rotate over copies that together exceed L2."""
    import torch

    from mlx_one_b200.kernels import default_ops
    from mlx_one_b200.parts import (FixedState, PagedKeyValues, PagedView, StateView,
                                    StepContext)

    ops, device = default_ops("cuda:0"), "cuda:0"
    ints = lambda values: torch.tensor(values, dtype=torch.int32, device=device)
    bf16 = lambda *shape: torch.randn(*shape, device=device).bfloat16()

    def ctx_of(portions, histories):
        positions, owner, starts = [], [], [0]
        for r, (n, before) in enumerate(zip(portions, histories)):
            positions += list(range(before, before + n))
            owner += [r] * n
            starts.append(starts[-1] + n)
        return StepContext(tokens=len(positions), requests=len(portions),
                           token_ids=ints([0] * len(positions)), positions=ints(positions),
                           token_request=ints(owner), request_start=ints(starts),
                           history=ints(histories), max_portion=max(portions),
                           max_context=max(p + h for p, h in zip(portions, histories)))

    def entry(seconds, moved=None, flops=None):
        out = {"us": round(seconds * 1e6, 2)}
        if moved is not None:
            out["gbs"] = round(moved / seconds / 1e9, 1)
            out["hbm_frac"] = round(moved / seconds / 1e9 / peak["hbm_gbs"], 4)
        if flops is not None:
            out["tflops"] = round(flops / seconds / 1e12, 2)
            out["tensor_frac"] = round(flops / seconds / 1e12 / peak["bf16_tflops"], 4)
        return out

    out = {}
    for label, portions, histories in (("decode", [1] * batch, [2048] * batch),
                                       ("prefill", [PREFILL_TOKENS], [0])):
        ctx = ctx_of(portions, histories)
        tokens, requests = ctx.tokens, ctx.requests
        # ---- the state space beside lightning attention, equal state sizes
        H, P, N = width // 64, 64, 128
        state_size = H * N * P
        copies = max(2, min(24, int(200e6 // (requests * state_size * 4))))
        state = torch.zeros(copies * requests, state_size, device=device)
        views = [StateView(state, ints(list(range(c * requests, (c + 1) * requests))),
                           FixedState((state_size,), "float32")) for c in range(copies)]
        channels = H * P + 2 * N
        mixed = [bf16(tokens, channels) for _ in range(copies)]
        raw = [bf16(tokens, H) for _ in range(copies)]
        constants = dict(a_log=torch.full((H,), -3.0, device=device),
                         dt_bias=torch.zeros(H, device=device), skip=torch.ones(H, device=device),
                         ctx=ctx, write=True, heads=H, value_dim=P, state_dim=N, groups=1)
        seconds = graph_seconds(lambda i: ops.state_space_scan(mixed[i], raw[i], view=views[i],
                                                               **constants), copies, 2 * copies)
        moved = tokens * ((channels + H) * 2 + H * P * 4) + 2 * requests * state_size * 4
        out[f"{label}_state_space"] = entry(seconds, moved)
        out[f"{label}_state_space"]["gflops_fma"] = round(4.0 * tokens * H * N * P / seconds / 1e9, 1)
        LH, D, V = width // 128, 128, 128
        wide = 2 * LH * D + 2 * LH * V
        projected = [bf16(tokens, wide) for _ in range(copies)]
        decay = torch.full((LH,), 0.97, device=device)
        weight = torch.ones(LH * V, device=device)
        seconds = graph_seconds(lambda i: ops.lightning_attention(
            projected[i], decay=decay, norm_weight=weight, eps=1e-6, ctx=ctx, view=views[i],
            write=True, heads=LH, key_dim=D, value_dim=V), copies, 2 * copies)
        moved = tokens * (wide + LH * V) * 2 + 2 * requests * state_size * 4
        out[f"{label}_lightning_farorax"] = entry(seconds, moved)
        out[f"{label}_lightning_farorax"]["gflops_fma"] = round(4.0 * tokens * LH * D * V / seconds / 1e9, 1)
        # ---- the convolution ahead of the state space; the gate and norm behind it
        taps = 4
        slots = torch.zeros(copies * requests, taps - 1, channels, device=device).bfloat16()
        conv_views = [StateView(slots, views[c].slots, FixedState((taps - 1, channels)))
                      for c in range(copies)]
        kernel, bias = torch.randn(channels, taps, device=device), torch.zeros(channels, device=device)
        seconds = graph_seconds(lambda i: ops.channel_conv(mixed[i], kernel, bias, taps=taps,
                                                           activation="silu", ctx=ctx,
                                                           view=conv_views[i], write=True),
                                copies, 2 * copies)
        out[f"{label}_channel_conv"] = entry(seconds, tokens * channels * 4 +
                                             2 * requests * (taps - 1) * channels * 2)
        y = [torch.randn(tokens, H * P, device=device) for _ in range(copies)]
        gate = [bf16(tokens, H * P) for _ in range(copies)]
        norm_weight = torch.ones(H * P, device=device)
        seconds = graph_seconds(lambda i: ops.gated_group_norm(y[i], gate[i], norm_weight,
                                                               groups=max(width // 256, 1), eps=1e-6,
                                                               dtype=torch.bfloat16), copies, 2 * copies)
        out[f"{label}_gated_group_norm"] = entry(seconds, tokens * H * P * (4 + 2 + 2))
        del state, views, mixed, raw, projected, slots, conv_views, y, gate
        # ---- attention over a window that keeps the first tokens beside a window alone
        heads, kv_heads, head, window, keep = width // 64, width // 256, 64, 1024, 4
        pages = -(-(histories[0] + portions[0]) // PAGE_SIZE)
        table = ints([[r * pages + b for b in range(pages)] for r in range(requests)])
        kv = (torch.randn(2, requests * pages + 1, kv_heads, PAGE_SIZE, head, device=device) * 0.3).bfloat16()
        q = [bf16(tokens, heads, head) for _ in range(4)]
        seen = sum(min(h + i + 1, window) for n, h in zip(portions, histories) for i in range(n))
        moved = requests * min(histories[0] + portions[0], window + portions[0]) * kv_heads * head * 2 * 2 \
            + tokens * heads * head * 2 * 2
        flops = 4.0 * heads * head * seen
        for name, kept in (("attention_kept_first", keep), ("attention_window_farorax", 0)):
            view = PagedView(kv, table, PAGE_SIZE, PagedKeyValues(kv_heads, head, window, keep_first=kept))
            seconds = graph_seconds(lambda i: ops.paged_attention(
                q[i], heads=heads, kv_heads=kv_heads, head_dim=head, scale=0.125, window=window,
                keep_first=kept, ctx=ctx, view=view), 4, 8)
            out[f"{label}_{name}"] = entry(seconds, moved, flops)
        mixed_heads = [bf16(tokens, heads * head) for _ in range(4)]
        gates = [bf16(tokens, heads * head) for _ in range(4)]
        seconds = graph_seconds(lambda i: ops.gate_heads(mixed_heads[i], gates[i], heads=heads,
                                                         row_dim=head, value_dim=head, per_head=False), 4, 8)
        out[f"{label}_gate_heads"] = entry(seconds, tokens * heads * head * 6)
        del kv, q, mixed_heads, gates
        # ---- the routed feed-forward with softmax scores, identity outputs and a gated shared
        # expert beside Farorax's
        experts, top, identity, ff, shared = 8, 3, 2, width, width
        copies = max(2, min(12, int(300e6 // ((experts * ff + shared) * width * 6))))
        stack = experts * ff + shared
        gate_up = [bf16(2 * stack, width) * 0.02 for _ in range(copies)]
        down = [bf16(width, stack) * 0.02 for _ in range(copies)]
        x = bf16(tokens, width)
        at = experts * ff
        alone = [(torch.cat([g[at:at + shared], g[stack + at:stack + at + shared]]).contiguous(),
                  d[:, at:].contiguous()) for g, d in zip(gate_up, down)]
        router = torch.randn(experts + identity + 1, width, device=device)
        correction = torch.zeros(experts + identity, device=device)

        def routed(i):                  # what the routed feed-forward part runs
            weights, others = ops.route_general(x, router, correction, experts=experts,
                                                identity=identity, top=top, scores="softmax",
                                                normalize=False, shared_gate=True)
            if ops.sorts_experts(x, experts=experts, width=ff, top=top, stack=stack):
                y = ops.routed_experts_sorted(x, weights, gate_up[i], down[i], experts=experts,
                                              width=ff, top=top, shared_gate_up=alone[i][0],
                                              shared_down=alone[i][1], shared_scale=others[1])
            else:
                gated = ops.linear_swiglu(x, gate_up[i])
                ops.scale_expert_columns(gated, weights, ff, tail=others[1])
                y = ops.linear(gated, down[i])
            ops.add_scaled_rows(y, x, others[0])
            return y

        def routed_farorax(i):
            weights = ops.route_experts(x, router[:experts], experts=experts, top=2, groups=4,
                                        keep=2, group_score=2)
            if ops.sorts_experts(x, experts=experts, width=ff, top=2, stack=stack):
                return ops.routed_experts_sorted(x, weights, gate_up[i], down[i], experts=experts,
                                                 width=ff, top=2, shared_gate_up=alone[i][0],
                                                 shared_down=alone[i][1])
            gated = ops.linear_swiglu(x, gate_up[i])
            ops.scale_expert_columns(gated, weights, ff)
            return ops.linear(gated, down[i])
        router_f = router[:experts].contiguous()
        for name, fn, used in (("routed_ff", routed, 2.4 * ff + shared),
                               ("routed_ff_farorax", routed_farorax, 2 * ff + shared)):
            if name.endswith("farorax"):
                router = router_f
            seconds = graph_seconds(fn, copies, 2 * copies)
            touched = min(experts, tokens * 3) * ff + shared
            out[f"{label}_{name}"] = entry(seconds, touched * width * 6 if label == "decode" else None,
                                           6.0 * tokens * used * width if label == "prefill" else None)
        del gate_up, down
        # ---- the norm of a part's output added into the stream beside add + norm
        residual = [torch.zeros(tokens, width, device=device) for _ in range(4)]
        delta = [bf16(tokens, width) for _ in range(4)]
        vector = torch.ones(width, device=device)
        seconds = graph_seconds(lambda i: ops.normed_mean_add(residual[i], [delta[i]], [vector], 1e-6), 4, 8)
        out[f"{label}_output_norm_add"] = entry(seconds, tokens * width * (4 + 4 + 2))
        seconds = graph_seconds(lambda i: ops.add_rmsnorm(residual[i], delta[i], vector, 1e-6,
                                                          torch.bfloat16), 4, 8)
        out[f"{label}_add_rmsnorm_farorax"] = entry(seconds, tokens * width * (4 + 4 + 2 + 2))
        del residual, delta
        torch.cuda.empty_cache()
    return out


def case_tirudra(args) -> int:
    """Tirudra beside Farorax (the closest of the engine's models: a recurrent mixer with a matrix
    state per head, softmax attention over a window, routed experts with a shared one) at equal
    width, depth and vocabulary, random weights: decode tokens/s at ``--batch`` and ``--context``
    (device-timed graph replays of the engine's step), prefill tokens/s of one 2,048-token prompt,
    each against its bound, and the new kernels alone."""
    import gc

    import torch

    peak = peaks()
    warmup, steps = max(args.warmup, 3), min(args.steps, 128)
    context = args.context or 2048
    layers = min(args.layers, 8)
    results = {}
    for width in (1024, 2048):
        for label, data in ((f"tirudra_w{width}", tirudra_shape(width, layers)),
                            (f"farorax_w{width}", farorax_shape(width, layers))):
            engine = engine_of(data, args.batch, context, warmup + steps, f"random-{label}")
            model, spec = engine.model, engine.model.spec
            weight_bytes = model.weight_bytes()
            kv_per_token = engine.cache_bytes_per_token()
            state_bytes = sum(g.storage[:, 0].numel() * g.storage.element_size()
                              for g in engine.cache.states)
            seconds, _, mean_context, launches = time_decode(engine, args.batch, context, warmup,
                                                             steps, seed=3)
            step_bytes = weight_bytes + args.batch * (mean_context * kv_per_token + 2 * state_bytes)
            prefill_seconds = time_prefill(engine, PREFILL_TOKENS, 2, 3, seed=5)
            flops = model_flops(spec, PREFILL_TOKENS)
            results[label] = {
                "layers": layers, "weight_mb": round(weight_bytes / 1e6, 1),
                "state_mb_per_request": round(state_bytes / 1e6, 2),
                "decode_tokens_per_s": round(args.batch * steps / seconds, 1),
                "decode_ms_per_step": round(seconds / steps * 1e3, 4),
                "decode_hbm_frac": round(step_bytes / (seconds / steps) / 1e9 / peak["hbm_gbs"], 4),
                "launches_per_step": launches,
                "prefill_tokens_per_s": round(PREFILL_TOKENS / prefill_seconds, 1),
                "prefill_ms": round(prefill_seconds * 1e3, 3),
                "prefill_tensor_frac": round(flops / prefill_seconds / (peak["bf16_tflops"] * 1e12), 4)}
            del engine, model
            gc.collect()
            torch.cuda.empty_cache()
        results[f"kernels_w{width}"] = tirudra_kernels(width, args.batch, peak)
    print(json.dumps({"case": "tirudra", "batch": args.batch, "context": context, "steps": steps,
                      "warmup": warmup, "dtype": "bf16", "peaks": peak["source"],
                      "data": "synthetic: random weights, seeded uniform-random token ids",
                      "results": results}))
    return 0


# --------------------------------------------------------------------------- Lamisun beside LFM2


def lamisun_shape(width: int, layers: int, vocab: int = 65536) -> dict:
    """A Lamisun of the sizes that a model of this width has: layers in turn with attention over
    latent rows (heads of 64 unrotated + a rotated part shared by the heads, a latent of a quarter
    of the width) and differential attention (two maps of 64 per head, one key head per four
    query heads, chunks of 1024 positions, as many score maps as LFM2 has heads), feed-forwards
    four times the width, four taps, a pair table of 65,536 buckets."""
    rot_dim, latent = (32, 256) if width <= 1024 else (64, 512)
    first = {"heads": width // 64, "dim": 64, "rot_dim": rot_dim, "vdim": 64, "kv_rank": latent,
             "scale": (64 + rot_dim) ** -0.5, "rot": {"base": 10000.0, "dims": rot_dim}}
    second = {"heads": width // 128, "kv_heads": width // 512, "dim": 64, "vdim": 64,
              "scale": 0.125, "diff": 0.2, "mask": {"size": 1024}}
    dense = {"kind": "dense", "ff": 4 * width}
    entries = [{"type": "attention", "mixer": second, "mlp": dense} if index % 2 else
               {"type": "latent_attention", "mixer": first, "mlp": dense} for index in range(layers)]
    return {"architecture": "Lamisun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0, "bigram": {"buckets": 65536, "mul_prev": 1000003,
                                                   "mul_cur": 31}},
            "canon": {"taps": 4}, "layers": entries}


def lamisun_kernels(width, batch, peak):
    """The kernels that Lamisun adds, alone, beside the like kernels of LFM2, for a decode step
    of ``batch`` tokens over 2,048 earlier ones and a prompt of PREFILL_TOKENS tokens:
    algorithmic bytes (or flops) / time against the measured peaks. Arguments rotate over copies
    that together exceed L2."""
    import torch

    from mlx_one_b200.kernels import default_ops
    from mlx_one_b200.parts import (FixedState, PagedKeyValues, PagedView, StateView,
                                    StepContext)

    ops, device = default_ops("cuda:0"), "cuda:0"
    ints = lambda values: torch.tensor(values, dtype=torch.int32, device=device)
    bf16 = lambda *shape: torch.randn(*shape, device=device).bfloat16()

    def ctx_of(portions, histories):
        positions, owner, starts = [], [], [0]
        for r, (n, before) in enumerate(zip(portions, histories)):
            positions += list(range(before, before + n))
            owner += [r] * n
            starts.append(starts[-1] + n)
        return StepContext(tokens=len(positions), requests=len(portions),
                           token_ids=ints([0] * len(positions)), positions=ints(positions),
                           token_request=ints(owner), request_start=ints(starts),
                           history=ints(histories), max_portion=max(portions),
                           max_context=max(p + h for p, h in zip(portions, histories)))

    def entry(seconds, moved=None, flops=None):
        out = {"us": round(seconds * 1e6, 2)}
        if moved is not None:
            out["gbs"] = round(moved / seconds / 1e9, 1)
            out["hbm_frac"] = round(moved / seconds / 1e9 / peak["hbm_gbs"], 4)
        if flops is not None:
            out["tflops"] = round(flops / seconds / 1e12, 2)
            out["tensor_frac"] = round(flops / seconds / 1e12 / peak["bf16_tflops"], 4)
        return out

    shape = lamisun_shape(width, 2)
    first, second = shape["layers"][0]["mixer"], shape["layers"][1]["mixer"]
    taps, vocab, buckets = 4, 65536, 65536
    out = {}
    for label, portions, histories in (("decode", [1] * batch, [2048] * batch),
                                       ("prefill", [PREFILL_TOKENS], [0])):
        ctx = ctx_of(portions, histories)
        tokens, requests = ctx.tokens, ctx.requests
        copies = 8 if label == "prefill" else 4
        slots = ints(list(range(requests)))
        # ---- the embedding with the pair table, beside LFM2's plain rows
        table, pairs = bf16(vocab, width), bf16(buckets + 1, width)
        ids = [torch.randint(0, vocab, (tokens,), device=device, dtype=torch.int32)
               for _ in range(copies)]
        last = StateView(torch.ones(requests, 1, dtype=torch.int32, device=device), slots,
                         FixedState((1,), "int32"))
        stream = [torch.zeros(tokens, width, device=device) for _ in range(copies)]
        seconds = graph_seconds(lambda i: ops.embedding_pairs(
            ids[i], table, 1.0, pairs, rule=(buckets, 1000003, 31), ctx=ctx, view=last,
            out=stream[i]), copies, 2 * copies)
        out[f"{label}_embedding_pairs"] = entry(seconds, tokens * width * (2 + 2 + 4))
        seconds = graph_seconds(lambda i: ops.embedding(ids[i], table), copies, 2 * copies)
        out[f"{label}_embedding_lfm2"] = entry(seconds, tokens * width * (2 + 2))
        del table, pairs
        # ---- what a sublayer reads: the stream plus its convolution over time, beside LFM2's
        # norm of the stream (both read 32-bit rows and write the compute dtype)
        kept = torch.zeros(requests, 2, taps - 1, width, device=device)
        inputs = StateView(kept, slots, FixedState((2, taps - 1, width), "float32"))
        kernel = torch.randn(width, taps, device=device) * 0.1
        seconds = graph_seconds(lambda i: ops.stream_conv(
            stream[i], kernel, taps=taps, ctx=ctx, view=inputs, sublayer=0, write=True,
            dtype=torch.bfloat16), copies, 2 * copies)
        out[f"{label}_stream_conv"] = entry(
            seconds, tokens * width * (4 + 2) + 2 * requests * (taps - 1) * width * 4)
        weight = torch.ones(width, device=device)
        seconds = graph_seconds(lambda i: ops.add_rmsnorm(stream[i], None, weight, 1e-6,
                                                          torch.bfloat16), copies, 2 * copies)
        out[f"{label}_rmsnorm_lfm2"] = entry(seconds, tokens * width * (4 + 2))
        # ---- a part's output, normed, into the stream, beside LFM2's add + norm
        delta = [bf16(tokens, width) for _ in range(copies)]
        seconds = graph_seconds(lambda i: ops.normed_mean_add(stream[i], [delta[i]], [weight],
                                                              1e-6), copies, 2 * copies)
        out[f"{label}_add_normed"] = entry(seconds, tokens * width * (4 + 4 + 2))
        seconds = graph_seconds(lambda i: ops.add_rmsnorm(stream[i], delta[i], weight, 1e-6,
                                                          torch.bfloat16), copies, 2 * copies)
        out[f"{label}_add_rmsnorm_lfm2"] = entry(seconds, tokens * width * (4 + 4 + 2 + 2))
        # ---- the weighted sum of the streams kept so far (after the eighth layer: nine of them)
        count = 9
        many = [torch.zeros(count + 1, tokens, width, device=device) for _ in range(2)]
        average = torch.full((count,), 1.0 / count, device=device)
        seconds = graph_seconds(lambda i: ops.stream_average(many[i], average, count,
                                                             many[i][count]), 2, 4)
        out[f"{label}_stream_average_9"] = entry(seconds, tokens * width * 4 * (count + 1))
        del many, stream, delta
        # ---- attention over latent rows: the preparation (latent norm, rotation, page write)
        # beside LFM2's (head norms, rotation, page write), then attention itself
        heads, nope, rot, latent = first["heads"], first["dim"], first["rot_dim"], first["kv_rank"]
        row = latent + rot
        span = histories[0] + portions[0]
        pages = -(-span // PAGE_SIZE)
        blocks = ints([[r * pages + b for b in range(pages)] for r in range(requests)])
        rows = (torch.randn(1, requests * pages + 1, 1, PAGE_SIZE, row, device=device) * 0.3).bfloat16()
        latent_view = PagedView(rows, blocks, PAGE_SIZE, PagedKeyValues(1, row, planes=1))
        wide = heads * (nope + rot) + row + heads * first["vdim"]
        projected = [bf16(tokens, wide) for _ in range(copies)]
        queries = [bf16(tokens, heads, row) * 0.3 for _ in range(copies)]
        inv_freq = torch.rand(rot // 2, device=device)
        norm_weight = torch.ones(latent, device=device)
        seconds = graph_seconds(lambda i: ops.latent_prepare(
            projected[i], queries[i], heads=heads, head_dim=nope, rot_dim=rot, latent=latent,
            norm_weight=norm_weight, eps=1e-6, rotary=(inv_freq, rot), neighbours=True, ctx=ctx,
            view=latent_view, write=True), copies, 2 * copies)
        out[f"{label}_latent_prepare"] = entry(
            seconds, tokens * ((heads * rot + row) * 2 + (heads * rot + row) * 2))
        lfm_heads, lfm_kv, head = width // 64, width // 256, 64
        kv = (torch.randn(2, requests * pages + 1, lfm_kv, PAGE_SIZE, head, device=device) * 0.3).bfloat16()
        view = PagedView(kv, blocks, PAGE_SIZE, PagedKeyValues(lfm_kv, head, None))
        qkv = [bf16(tokens, (lfm_heads + 2 * lfm_kv) * head) for _ in range(copies)]
        ones, inv_full = torch.ones(head, device=device), torch.rand(head // 2, device=device)
        seconds = graph_seconds(lambda i: ops.qk_norm_rope_store(
            qkv[i], heads=lfm_heads, kv_heads=lfm_kv, head_dim=head, q_weight=ones, k_weight=ones,
            eps=1e-6, rotary=(inv_full, head), ctx=ctx, view=view, write=True), copies, 2 * copies)
        out[f"{label}_qk_prep_lfm2"] = entry(seconds, tokens * (lfm_heads + 2 * lfm_kv) * head * 2 * 2)
        seen = sum(h + i + 1 for n, h in zip(portions, histories) for i in range(n))
        seconds = graph_seconds(lambda i: ops.latent_attention(
            queries[i], heads=heads, latent=latent, scale=first["scale"], ctx=ctx,
            view=latent_view), copies, 2 * copies)
        out[f"{label}_latent_attention"] = entry(
            seconds, requests * span * row * 2 + tokens * heads * row * 2 * 2,
            2.0 * heads * (row + latent) * seen)
        q = [bf16(tokens, lfm_heads, head) for _ in range(copies)]
        seconds = graph_seconds(lambda i: ops.paged_attention(
            q[i], heads=lfm_heads, kv_heads=lfm_kv, head_dim=head, scale=0.125, window=None,
            ctx=ctx, view=view), copies, 2 * copies)
        out[f"{label}_attention_lfm2"] = entry(
            seconds, requests * span * lfm_kv * head * 2 * 2 + tokens * lfm_heads * head * 2 * 2,
            4.0 * lfm_heads * head * seen)
        # ---- the products head by head around the attention (a library's batched product)
        up_k = bf16(heads, latent, nope) * 0.05
        up_v = bf16(heads, first["vdim"], latent) * 0.05
        seconds = graph_seconds(lambda i: ops.linear_heads(
            projected[i][:, :heads * (nope + rot)].view(tokens, heads, -1)[:, :, :nope], up_k,
            out=queries[i][:, :, :latent]), copies, 2 * copies)
        out[f"{label}_heads_up_k"] = entry(seconds, None, 2.0 * tokens * heads * latent * nope)
        out[f"{label}_heads_up_k"]["weights_gbs"] = round(up_k.numel() * 2 / seconds / 1e9, 1)
        seconds = graph_seconds(lambda i: ops.linear_heads(queries[i][:, :, :latent], up_v),
                                copies, 2 * copies)
        out[f"{label}_heads_up_v"] = entry(seconds, None, 2.0 * tokens * heads * latent * first["vdim"])
        out[f"{label}_heads_up_v"]["weights_gbs"] = round(up_v.numel() * 2 / seconds / 1e9, 1)
        # ---- the sigmoid gate on the heads' outputs
        inner = heads * first["vdim"]
        values = [bf16(tokens, inner) for _ in range(copies)]
        seconds = graph_seconds(lambda i: ops.sigmoid_gate(values[i], projected[i][:, wide - inner:]),
                                copies, 2 * copies)
        out[f"{label}_sigmoid_gate"] = entry(seconds, tokens * inner * 2 * 3)
        del rows, projected, queries, q, values
        # ---- differential attention: two maps per head within chunks, beside LFM2's heads over
        # every earlier key (from the fused projection to the mixed heads)
        dh, dkv, dim, chunk = second["heads"], second["kv_heads"], second["dim"], second["mask"]["size"]
        both = (torch.randn(2, requests * pages + 1, 2 * dkv, PAGE_SIZE, dim, device=device) * 0.3).bfloat16()
        maps_view = PagedView(both, blocks, PAGE_SIZE, PagedKeyValues(2 * dkv, dim, chunk=chunk))
        two = [bf16(tokens, (2 * dh + 4 * dkv) * dim) for _ in range(copies)]
        dim_ones = torch.ones(dim, device=device)
        seen_chunk = sum((h + i) % chunk + 1 for n, h in zip(portions, histories) for i in range(n))
        read = lambda kv_heads, size, keys: requests * keys * kv_heads * size * 2 * 2
        seconds = graph_seconds(lambda i: ops.qkv_attention(
            two[i], heads=2 * dh, kv_heads=2 * dkv, head_dim=dim, q_weight=dim_ones,
            k_weight=dim_ones, eps=1e-6, rotary=None, scale=0.125, window=None, chunk=chunk,
            ctx=ctx, view=maps_view, write=True), copies, 2 * copies)
        keys_read = min(span, (histories[0] % chunk) + portions[0]) if label == "decode" else span
        out[f"{label}_differential_maps"] = entry(
            seconds, read(2 * dkv, dim, keys_read) + tokens * (4 * dh + 4 * dkv) * dim * 2,
            4.0 * 2 * dh * dim * seen_chunk)
        seconds = graph_seconds(lambda i: ops.qkv_attention(
            qkv[i], heads=lfm_heads, kv_heads=lfm_kv, head_dim=head, q_weight=ones, k_weight=ones,
            eps=1e-6, rotary=(inv_full, head), scale=0.125, window=None, ctx=ctx, view=view,
            write=True), copies, 2 * copies)
        out[f"{label}_qkv_attention_lfm2"] = entry(
            seconds, read(lfm_kv, head, span) + tokens * (2 * lfm_heads + 2 * lfm_kv) * head * 2,
            4.0 * lfm_heads * head * seen)
        maps = [bf16(tokens, 2 * dh * dim) for _ in range(copies)]
        seconds = graph_seconds(lambda i: ops.differential_combine(
            maps[i], heads=dh, row_dim=dim, value_dim=dim, mix=0.3, eps=1e-6, factor=0.8),
            copies, 2 * copies)
        out[f"{label}_differential_combine"] = entry(seconds, tokens * dh * dim * 2 * 3)
        del both, two, maps, kv, qkv
        # ---- the feed-forward's first product with xielu, beside the gated one of LFM2
        ff = 4 * width
        wcopies = max(2, min(12, int(300e6 // (ff * width * 2))))
        up = [bf16(ff, width) * 0.02 for _ in range(wcopies)]
        gate_up = [bf16(2 * ff, width) * 0.02 for _ in range(wcopies)]
        x = bf16(tokens, width)
        for name, fn, rows_w in (
                ("up_xielu", lambda i: ops.linear_act(x, up[i], "xielu", (0.8, 0.8)), ff),
                ("up_swiglu_lfm2", lambda i: ops.linear_swiglu(x, gate_up[i]), 2 * ff)):
            seconds = graph_seconds(fn, wcopies, wcopies)
            out[f"{label}_{name}"] = entry(
                seconds, rows_w * width * 2 if label == "decode" else None,
                2.0 * tokens * rows_w * width if label == "prefill" else None)
        del up, gate_up
        torch.cuda.empty_cache()
    return out


def case_lamisun(args) -> int:
    """Lamisun beside LFM2 (the closest of the engine's models: softmax attention with normed
    queries and keys over paged keys, a convolution over time, a dense feed-forward) at equal
    width, depth and vocabulary, random weights: decode tokens/s at ``--batch`` and ``--context``
    (device-timed graph replays of the engine's step), prefill tokens/s of one 2,048-token
    prompt, each against its bound, and the new kernels alone."""
    import gc

    import torch

    peak = peaks()
    warmup, steps = max(args.warmup, 3), min(args.steps, 128)
    context = args.context or 2048
    layers = min(args.layers, 8)
    results = {}
    for width, twin in ((1024, LFM2_350M), (2048, LFM2_1_2B)):
        lfm2 = dict(twin)
        lfm2["layer_types"] = lfm2["layer_types"][:layers]
        lfm2["num_hidden_layers"] = layers
        for label, data in ((f"lamisun_w{width}", lamisun_shape(width, layers)),
                            (f"lfm2_w{width}", lfm2)):
            engine = engine_of(data, args.batch, context, warmup + steps, f"random-{label}")
            model, spec = engine.model, engine.model.spec
            weight_bytes = model.weight_bytes()
            kv_per_token = engine.cache_bytes_per_token()
            state_bytes = sum(g.storage[:, 0].numel() * g.storage.element_size()
                              for g in engine.cache.states)
            seconds, _, mean_context, launches = time_decode(engine, args.batch, context, warmup,
                                                             steps, seed=3)
            step_bytes = weight_bytes + args.batch * (mean_context * kv_per_token + 2 * state_bytes)
            prefill_seconds = time_prefill(engine, PREFILL_TOKENS, 2, 3, seed=5)
            flops = model_flops(spec, PREFILL_TOKENS)
            results[label] = {
                "layers": layers, "weight_mb": round(weight_bytes / 1e6, 1),
                "state_mb_per_request": round(state_bytes / 1e6, 2),
                "decode_tokens_per_s": round(args.batch * steps / seconds, 1),
                "decode_ms_per_step": round(seconds / steps * 1e3, 4),
                "decode_hbm_frac": round(step_bytes / (seconds / steps) / 1e9 / peak["hbm_gbs"], 4),
                "launches_per_step": launches,
                "prefill_tokens_per_s": round(PREFILL_TOKENS / prefill_seconds, 1),
                "prefill_ms": round(prefill_seconds * 1e3, 3),
                "prefill_tensor_frac": round(flops / prefill_seconds / (peak["bf16_tflops"] * 1e12), 4)}
            del engine, model
            gc.collect()
            torch.cuda.empty_cache()
        results[f"kernels_w{width}"] = lamisun_kernels(width, args.batch, peak)
    print(json.dumps({"case": "lamisun", "batch": args.batch, "context": context, "steps": steps,
                      "warmup": warmup, "dtype": "bf16", "peaks": peak["source"],
                      "data": "synthetic: random weights, seeded uniform-random token ids",
                      "results": results}))
    return 0


def decode_step_case(batch: int, context: int) -> int:
    """A few eager decode steps of the whole model at the benchmark's sizes, for a list of the
    step's launches (`ncu --metrics gpu__time_duration.sum`): the prompts are fed first, the last
    launches are the decode steps'."""
    import torch

    from mlx_one_b200.engine.runner import StepEntry

    engine = build_engine(LFM2_1_2B, LFM2_1_2B["num_hidden_layers"], batch, context, 16)
    engine.model.ops.set_dependent_launches(True)
    runner = engine.runner
    runner.use_graphs = False
    ids = [f"step{i}" for i in range(batch)]
    prompts = random_prompts(engine.model.spec.vocab_size, batch, context - 8, seed=3)
    firsts = fill_requests(engine, prompts, ids)
    before = engine.model.ops.launches
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    tokens = firsts
    for _ in range(4):
        runner.step([StepEntry(i, [t], (0,)) for i, t in zip(ids, tokens)], greedy=True)
        tokens = runner.last_greedy.tolist()
    stop.record()
    torch.cuda.synchronize()
    engine.model.ops.check_errors()
    print(json.dumps({"kernel": "decode_step", "batch": batch, "context": context,
                      "launches_per_step": (engine.model.ops.launches - before) // 4,
                      "eager_ms_per_step": round(start.elapsed_time(stop) / 4, 3)}))
    return 0


def decode_timeline_case(batch: int, context: int) -> int:
    """Where a decode step's time goes, kernel by kernel, as the step really runs (CUDA-graph
    replays with dependent launches): the device's own activity records, taken through
    torch.profiler, give every kernel's begin and end. A kernel's "exposed" time is the part of
    it after every earlier kernel of the step has ended, which is what it adds to the step (a
    kernel that starts early and waits for its predecessor shows a long duration and a short
    exposed time). Prints one JSON line; times under the profiler are for shares, the step's
    own time is the benchmark's."""
    import collections

    import torch
    from torch.profiler import ProfilerActivity, profile

    from mlx_one_b200.engine.runner import StepEntry

    engine = build_engine(LFM2_1_2B, LFM2_1_2B["num_hidden_layers"], batch, context, 64)
    engine.model.ops.set_dependent_launches(True)
    runner = engine.runner
    ids = [f"step{i}" for i in range(batch)]
    prompts = random_prompts(engine.model.spec.vocab_size, batch, context - 40, seed=3)
    firsts = fill_requests(engine, prompts, ids)
    last = runner.decode_steps([StepEntry(i, [t]) for i, t in zip(ids, firsts)], 16)[-1].tolist()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as record:
        runner.decode_steps([StepEntry(i, [t]) for i, t in zip(ids, last)], 8)
        torch.cuda.synchronize()
    engine.model.ops.check_errors()
    kernels = sorted(((e.name, e.time_range.start, e.time_range.end) for e in record.events()
                      if e.device_type.name == "CUDA" and "Memcpy" not in e.name
                      and "Memset" not in e.name), key=lambda k: k[1])
    # a step ends with the kernel that moves the chosen tokens on
    ends = [i for i, k in enumerate(kernels) if "decode_advance" in k[0]]
    if len(ends) < 6:
        print(json.dumps({"kernel": "decode_timeline", "error": "no steps in the record"}))
        return 1
    steps = [(ends[i] + 1, ends[i + 1] + 1) for i in range(2, len(ends) - 1)]
    calls, duration, exposed = collections.Counter(), collections.Counter(), collections.Counter()
    total = 0.0
    for begin, end in steps:
        horizon = kernels[begin][1]
        total += kernels[end - 1][2] - horizon
        for name, start, stop in kernels[begin:end]:
            short = name.replace("void (anonymous namespace)::", "").replace("void ", "")
            short = short.split("(")[0]
            calls[short] += 1
            duration[short] += stop - start
            exposed[short] += max(stop - max(horizon, start), 0.0) + max(start - horizon, 0.0)
            horizon = max(horizon, stop)
    count = len(steps)
    table = [{"kernel": name, "calls_per_step": calls[name] // count,
              "us_each": round(duration[name] / calls[name], 2),
              "exposed_us_each": round(exposed[name] / calls[name], 2),
              "exposed_us_per_step": round(exposed[name] / count, 1)}
             for name in sorted(exposed, key=exposed.get, reverse=True)]
    print(json.dumps({"kernel": "decode_timeline", "batch": batch, "context": context,
                      "steps_averaged": count, "us_per_step": round(total / count, 1),
                      "kernels": table}))
    return 0


def kernel_case(name: str, batch: int, context: int) -> int:
    """Runs one kernel of the step alone a few times at the benchmark's sizes and prints its
    time: the case that the ncu summaries under profiles/ were captured on."""
    import math

    import torch

    if name == "decode_step":
        return decode_step_case(batch, context)
    if name == "decode_timeline":
        return decode_timeline_case(batch, context)

    from mlx_one_b200.kernels import default_ops
    from mlx_one_b200.parts.base import PagedKeyValues, PagedView, StepContext

    ops, device = default_ops("cuda:0"), "cuda:0"
    ops.set_dependent_launches(True)
    hidden, width, heads, kv_heads, head_dim = 2048, 8192, 32, 8, 64
    torch.manual_seed(0)

    def weights(n, k, copies):          # several copies, so that no call finds its weights in L2
        return [(torch.randn(n, k, device=device) / math.sqrt(k)).bfloat16() for _ in range(copies)]

    def batch_context(portions, histories):
        as_int = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
        positions, owner, starts = [], [], [0]
        for r, (h, n) in enumerate(zip(histories, portions)):
            positions += list(range(h, h + n))
            owner += [r] * n
            starts.append(starts[-1] + n)
        blocks = [-(-(h + n) // PAGE_SIZE) for h, n in zip(histories, portions)]
        table = torch.full((len(portions), max(blocks)), -1, dtype=torch.int32)
        at = 0
        for r, count in enumerate(blocks):
            table[r, :count] = torch.arange(at, at + count)
            at += count
        ctx = StepContext(tokens=len(positions), requests=len(portions),
                          token_ids=as_int([0] * len(positions)), positions=as_int(positions),
                          token_request=as_int(owner), request_start=as_int(starts),
                          history=as_int(histories), max_portion=max(portions),
                          max_context=max(h + n for h, n in zip(histories, portions)))
        kv = torch.randn(2, at, kv_heads, PAGE_SIZE, head_dim, device=device).bfloat16()
        return ctx, PagedView(kv, table.to(device), PAGE_SIZE, PagedKeyValues(kv_heads, head_dim))

    if name == "skinny_swiglu":
        a = torch.randn(batch, hidden, device=device).bfloat16()
        w = weights(2 * width, hidden, 4)
        run = lambda i: ops.linear_swiglu(a, w[i % 4])
        work = f"{2 * width * hidden * 2 / 1e6:.1f} MB of weights"
    elif name == "skinny_in_proj":
        a = torch.randn(batch, hidden, device=device).bfloat16()
        w = weights(3 * hidden, hidden, 8)
        ops.skinny_max_rows = max(ops.skinny_max_rows, min(batch, 32))     # this kernel, not the library's
        run = lambda i: ops.linear(a, w[i % 8])
        work = f"{3 * hidden * hidden * 2 / 1e6:.1f} MB of weights"
    elif name == "skinny_down":
        a = torch.randn(batch, width, device=device).bfloat16()
        w = weights(hidden, width, 8)
        residual = torch.zeros(batch, hidden, device=device)
        run = lambda i: ops.linear_add(a, w[i % 8], None, residual)
        work = f"{hidden * width * 2 / 1e6:.1f} MB of weights"
    elif name == "decode_attention":
        ctx, view = batch_context([1] * batch, [context - 1] * batch)
        q = torch.randn(batch, heads, head_dim, device=device).bfloat16()
        run = lambda i: ops.paged_attention(q, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                            scale=head_dim ** -0.5, window=None, ctx=ctx, view=view)
        work = f"{batch * context * 2 * kv_heads * head_dim * 2 / 1e6:.1f} MB of keys and values"
    elif name == "prefill_attention":
        ctx, view = batch_context([PREFILL_TOKENS], [0])
        q = torch.randn(PREFILL_TOKENS, heads, head_dim, device=device).bfloat16()
        run = lambda i: ops.paged_attention(q, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                            scale=head_dim ** -0.5, window=None, ctx=ctx, view=view)
        work = f"{4 * heads * head_dim * PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2 / 1e9:.1f} GFLOP"
    elif name == "tcgen05_swiglu":
        a = torch.randn(PREFILL_TOKENS, hidden, device=device).bfloat16()
        w = weights(2 * width, hidden, 2)
        run = lambda i: ops.linear_swiglu(a, w[i % 2])
        work = f"{2 * PREFILL_TOKENS * 2 * width * hidden / 1e9:.1f} GFLOP"
    elif name == "swapped_swiglu":
        # the 33-to-128-row product with swapped operands (an option, off by default) on w13
        rows = max(batch, 33)
        a = torch.randn(rows, hidden, device=device).bfloat16()
        w = weights(2 * width, hidden, 4)
        ops.swapped_products = True
        run = lambda i: ops.linear_swiglu(a, w[i % 4])
        work = f"{2 * width * hidden * 2 / 1e6:.1f} MB of weights, {rows} rows"
    elif name == "mixed_attention":
        # attention of a mixed step at the LFM2-700M geometry (24 heads over 8 key heads): 63
        # decodes at `context` keys beside one 512-token portion after 1024 tokens
        heads, kv_heads = 24, 8
        singles = 63
        ctx, view = batch_context([1] * singles + [512], [context - 1] * singles + [1024])
        ctx.leading_single = singles
        q = torch.randn(singles + 512, heads, head_dim, device=device).bfloat16()
        run = lambda i: ops.paged_attention(q, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                            scale=head_dim ** -0.5, window=None, ctx=ctx, view=view)
        work = (f"{singles} single tokens over {context} keys "
                f"({singles * context * 2 * kv_heads * head_dim * 2 / 1e6:.1f} MB) + 512 tokens "
                f"after 1024")
    elif name == "sampling":
        vocab = LFM2_1_2B["vocab_size"]
        logits = [torch.randn(batch, vocab, device=device) * 3 for _ in range(4)]
        temperature = torch.full((batch,), 0.8, device=device)
        top_k = torch.full((batch,), 40, dtype=torch.int32, device=device)
        top_p = torch.full((batch,), 0.9, device=device)
        seed = torch.arange(batch, dtype=torch.int64, device=device)
        steps = torch.zeros(batch, dtype=torch.int32, device=device)
        run = lambda i: ops.sample(logits[i % 4], temperature, top_k, top_p, seed, steps)
        work = f"{batch} rows of {vocab} logits, temperature 0.8, top-k 40, top-p 0.9"
    elif name in ("delta_prefill", "delta_decode"):
        # the gated delta rule alone: 16 heads of 128 x 128, a prompt of 2048 tokens (prepare,
        # scan, finish) or `batch` single tokens (one kernel)
        from mlx_one_b200.parts import FixedState, StateView
        from mlx_one_b200.parts.mixers import GatedDeltaRule

        sizes = dict(heads=16, kv_heads=8, key_dim=128, value_dim=128, taps=4)
        slot = GatedDeltaRule.state_size(sizes)
        channels = 2 * 8 * 128 + 16 * 128
        wide = channels + 16 * 128 + 2 * 16
        portions = [PREFILL_TOKENS] if name == "delta_prefill" else [1] * batch
        ctx, _ = batch_context(portions, [0 if name == "delta_prefill" else context] * len(portions))
        state = torch.zeros(4 * len(portions), slot, device=device)
        views = [StateView(state, torch.arange(c * len(portions), (c + 1) * len(portions),
                                               dtype=torch.int32, device=device),
                           FixedState((slot,), "float32")) for c in range(4)]
        rows = [torch.randn(ctx.tokens, wide, device=device).bfloat16() for _ in range(4)]
        constants = dict(conv=torch.randn(channels, 4, device=device) * 0.5,
                         a_log=torch.zeros(16, device=device), dt_bias=torch.zeros(16, device=device),
                         norm_weight=torch.ones(128, device=device), eps=1e-6, unit_eps=1e-6,
                         ctx=ctx, write=True, **sizes)
        run = lambda i: ops.gated_delta_rule(rows[i % 4], view=views[i % 4], **constants)
        work = f"{ctx.tokens} tokens of {len(portions)} requests, 16 heads of 128 x 128, state {slot * 4 / 1e6:.1f} MB a request"
    elif name == "experts_sorted":
        # a routed feed-forward over 2,048 tokens sorted by expert: 8 experts of the model's width,
        # 2 a token, beside a shared one (sort, gather, two grouped tcgen05 products, the shared
        # expert's two products, combine)
        experts, top, ff, shared = 8, 2, hidden, hidden
        stack = experts * ff + shared
        gate_up = weights(2 * stack, hidden, 2)
        down = weights(hidden, stack, 2)
        at = experts * ff
        alone = [(torch.cat([g[at:at + shared], g[stack + at:stack + at + shared]]).contiguous(),
                  d[:, at:].contiguous()) for g, d in zip(gate_up, down)]
        router = torch.randn(experts, hidden, device=device)
        x = torch.randn(PREFILL_TOKENS, hidden, device=device).bfloat16()

        def run(i):
            routing = ops.route_experts(x, router, experts=experts, top=top, groups=4, keep=2,
                                        group_score=2)
            return ops.routed_experts_sorted(x, routing, gate_up[i % 2], down[i % 2], experts=experts,
                                             width=ff, top=top, shared_gate_up=alone[i % 2][0],
                                             shared_down=alone[i % 2][1])
        work = (f"{PREFILL_TOKENS} tokens, {experts} experts of {ff} x {hidden}, {top} a token, shared {shared}: "
                f"{6.0 * PREFILL_TOKENS * (top * ff + shared) * hidden / 1e9:.0f} GFLOP")
    elif name in ("lightning_prefill", "lightning_decode"):
        # lightning attention at the shape of a 2048-wide model: one 2,048-token prompt (segments:
        # build, chain, scan, then the norm and gate) or `batch` single tokens (scan, norm and gate)
        from mlx_one_b200.parts import FixedState, StateView

        heads, key_dim, value_dim = 16, 128, 128
        slot = heads * key_dim * value_dim
        wide = 2 * heads * key_dim + 2 * heads * value_dim
        portions = [PREFILL_TOKENS] if name == "lightning_prefill" else [1] * batch
        ctx, _ = batch_context(portions, [0 if name == "lightning_prefill" else context] * len(portions))
        state = torch.zeros(4 * len(portions), slot, device=device)
        views = [StateView(state, torch.arange(c * len(portions), (c + 1) * len(portions),
                                               dtype=torch.int32, device=device),
                           FixedState((slot,), "float32")) for c in range(4)]
        rows = [torch.randn(ctx.tokens, wide, device=device).bfloat16() for _ in range(4)]
        constants = dict(decay=torch.full((heads,), 0.97, device=device),
                         norm_weight=torch.ones(heads * value_dim, device=device), eps=1e-6, ctx=ctx,
                         write=True, heads=heads, key_dim=key_dim, value_dim=value_dim)
        run = lambda i: ops.lightning_attention(rows[i % 4], view=views[i % 4], **constants)
        work = f"{ctx.tokens} tokens of {len(portions)} requests, {heads} heads of {key_dim} x {value_dim}, state {slot * 4 / 1e6:.1f} MB a request"
    elif name in ("state_space_prefill", "state_space_decode", "channel_conv_prefill"):
        # a selective state space at the shape of a 2048-wide model: one 2,048-token prompt
        # (segments: build, chain, scan) or `batch` single tokens; and the convolution ahead of it
        from mlx_one_b200.parts import FixedState, StateView

        heads, value_dim, state_dim, taps = 32, 64, 128, 4
        slot = heads * state_dim * value_dim
        channels = heads * value_dim + 2 * state_dim
        portions = [1] * batch if name == "state_space_decode" else [PREFILL_TOKENS]
        ctx, _ = batch_context(portions, [context if name == "state_space_decode" else 0] * len(portions))
        slots = [torch.arange(c * len(portions), (c + 1) * len(portions), dtype=torch.int32,
                              device=device) for c in range(4)]
        rows = [torch.randn(ctx.tokens, channels, device=device).bfloat16() for _ in range(4)]
        if name == "channel_conv_prefill":
            kept = torch.zeros(4 * len(portions), taps - 1, channels, device=device).bfloat16()
            views = [StateView(kept, slots[c], FixedState((taps - 1, channels))) for c in range(4)]
            kernel, bias = torch.randn(channels, taps, device=device), torch.zeros(channels, device=device)
            run = lambda i: ops.channel_conv(rows[i % 4], kernel, bias, taps=taps, activation="silu",
                                             ctx=ctx, view=views[i % 4], write=True)
            work = f"{ctx.tokens} tokens, {channels} channels, {taps} taps"
        else:
            state = torch.zeros(4 * len(portions), slot, device=device)
            views = [StateView(state, slots[c], FixedState((slot,), "float32")) for c in range(4)]
            raw = [torch.randn(ctx.tokens, heads, device=device).bfloat16() for _ in range(4)]
            constants = dict(a_log=torch.full((heads,), -3.0, device=device),
                             dt_bias=torch.zeros(heads, device=device),
                             skip=torch.ones(heads, device=device), ctx=ctx, write=True, heads=heads,
                             value_dim=value_dim, state_dim=state_dim, groups=1)
            run = lambda i: ops.state_space_scan(rows[i % 4], raw[i % 4], view=views[i % 4], **constants)
            work = (f"{ctx.tokens} tokens of {len(portions)} requests, {heads} heads of {state_dim} x "
                    f"{value_dim}, state {slot * 4 / 1e6:.1f} MB a request")
    elif name in ("latent_prefill", "latent_decode"):
        # attention over latent rows at the sizes of a Lamisun 1024 wide: one 2,048-token prompt
        # (the kernel whose warps own 16 rows) or `batch` single tokens (key runs and their merge)
        mixer = lamisun_shape(1024, 1)["layers"][0]["mixer"]
        rot, latent = mixer["rot_dim"], mixer["kv_rank"]
        row = latent + rot
        portions = [PREFILL_TOKENS] if name == "latent_prefill" else [1] * batch
        ctx, plain = batch_context(portions, [0 if name == "latent_prefill" else context] * len(portions))
        pages = (torch.randn(1, int(plain.block_table.max()) + 1, 1, PAGE_SIZE, row, device=device)
                 * 0.3).bfloat16()
        view = PagedView(pages, plain.block_table, PAGE_SIZE, PagedKeyValues(1, row, planes=1))
        queries = [(torch.randn(ctx.tokens, mixer["heads"], row, device=device) * 0.3).bfloat16()
                   for _ in range(4)]
        run = lambda i: ops.latent_attention(queries[i % 4], heads=mixer["heads"], latent=latent,
                                             scale=mixer["scale"], ctx=ctx, view=view)
        work = (f"{ctx.tokens} tokens of {len(portions)} requests, {mixer['heads']} heads, rows of "
                f"{latent} + {rot}, keys {pages.numel() * 2 / 1e6:.1f} MB")
    else:
        print(f"unknown kernel case {name!r}")
        return 2
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(8):
        run(i)
    stop.record()
    torch.cuda.synchronize()
    ops.check_errors()
    print(json.dumps({"kernel": name, "us": round(start.elapsed_time(stop) * 1e3 / 8, 2),
                      "work": work, "batch": batch, "context": context}))
    return 0


def product_fractions(model, batch, peak):
    """The matrix products of the step alone, as the baseline's targets are stated for them:
    decode products against HBM bandwidth (bytes of weights / time), prefill products against
    the bf16 tensor peak. Each distinct product of the model is timed in a CUDA graph of
    back-to-back calls on several copies of its weights (so that none is found in L2)."""
    import torch

    ops, device = model.ops, "cuda:0"

    def graph_time(fn, copies, inner):
        for i in range(min(copies, 3)):
            fn(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(inner):
                fn(i % copies)
        graph.replay()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(5):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / 1e3 / (5 * inner)

    # (weight, kind, how many times a step runs it); kind picks the epilogue the engine uses
    seen: dict = {}
    for block in model.layers:
        mixer, ffn = block.mixer, block.feed_forward
        first = getattr(mixer, "qkv", None)
        first = first if first is not None else mixer.in_proj
        last = getattr(mixer, "out", None)
        last = last if last is not None else mixer.out_proj
        for weight, kind in ((first, "plain"), (last, "add"), (ffn.gate_up, "swiglu"),
                             (ffn.down, "add")):
            key = (tuple(weight.shape), kind)
            seen.setdefault(key, [weight, 0])[1] += 1
    decode_bytes = decode_seconds = prefill_flops = prefill_seconds = 0.0
    for (shape, kind), (weight, count) in seen.items():
        n, k = shape
        copies = max(2, min(16, int(300e6 // (n * k * 2))))
        weights = [weight] + [torch.randn_like(weight) * 0.02 for _ in range(copies - 1)]
        for rows in (batch, PREFILL_TOKENS):
            a = torch.randn(rows, k, device=device).bfloat16()
            residual = torch.zeros(rows, n, device=device)
            if kind == "plain":
                fn = lambda i: ops.linear(a, weights[i])
            elif kind == "swiglu":
                fn = lambda i: ops.linear_swiglu(a, weights[i])
            else:
                fn = lambda i: ops.linear_add(a, weights[i], None, residual)
            seconds = graph_time(fn, copies, copies * (2 if rows == batch else 1))
            if rows == batch:
                decode_bytes += count * n * k * 2
                decode_seconds += count * seconds
            else:
                prefill_flops += count * 2.0 * rows * n * k
                prefill_seconds += count * seconds
        del weights
    return {"decode_products_gbs": round(decode_bytes / decode_seconds / 1e9, 1),
            "decode_products_hbm_frac": round(decode_bytes / decode_seconds / 1e9 / peak["hbm_gbs"], 4),
            "prefill_products_tflops": round(prefill_flops / prefill_seconds / 1e12, 1),
            "prefill_products_frac": round(prefill_flops / prefill_seconds / 1e12 / peak["bf16_tflops"], 4)}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=None,
                        help="context length (default 4096; --case long: prompt tokens, 32768)")
    parser.add_argument("--case", default="decode", choices=["decode", "batching", "long", "galarax", "farorax", "lamisun", "tirudra"],
                        help="decode: the default line; batching: 128 requests batched "
                             "continuously (LFM2-700M shape); long: 4 x 32,768 tokens "
                             "(LFM2-350M shape)")
    parser.add_argument("--repeats", type=int, default=3, help="--case batching: measured runs")
    parser.add_argument("--requests", type=int, default=128, help="--case batching")
    parser.add_argument("--sequences", type=int, default=64,
                        help="--case batching: requests that run at a time")
    parser.add_argument("--layers", type=int, default=LFM2_1_2B["num_hidden_layers"])
    parser.add_argument("--skip-points", action="store_true", help="leave out the other batches and contexts")
    parser.add_argument("--kernel", default=None,
                        help="run one kernel alone instead of the benchmark: skinny_swiglu, "
                             "skinny_in_proj, skinny_down, decode_attention, prefill_attention, tcgen05_swiglu, "
                             "swapped_swiglu, mixed_attention, sampling, delta_prefill, delta_decode, lightning_prefill, "
                             "lightning_decode, experts_sorted, latent_prefill, latent_decode, state_space_prefill, "
                             "state_space_decode, channel_conv_prefill, decode_step (the "
                             "whole step, eager, for a launch list), decode_timeline (where "
                             "the graph-replayed step's time goes, kernel by kernel)")
    parser.add_argument("--dependent-launches", type=int, default=1,
                        help="1: kernels of a decode step may start while the one before ends")
    args = parser.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.case == "batching":
        return case_batching(args)
    if args.case == "long":
        return case_long(args)
    if args.case == "galarax":
        return case_galarax(args)
    if args.case == "farorax":
        return case_farorax(args)
    if args.case == "lamisun":
        return case_lamisun(args)
    if args.case == "tirudra":
        return case_tirudra(args)
    args.context = args.context or 4096
    if args.kernel:
        return kernel_case(args.kernel, args.batch, args.context)
    warmup = max(args.warmup, 3)

    import torch

    peak = peaks()
    largest = 64 if not args.skip_points else args.batch
    engine = build_engine(LFM2_1_2B, args.layers, max(largest, args.batch), args.context,
                          warmup + args.steps)
    model, spec = engine.model, engine.model.spec
    model.ops.set_dependent_launches(bool(args.dependent_launches))
    weight_bytes = model.weight_bytes()
    kv_per_token = engine.cache_bytes_per_token()
    state_bytes = sum(g.storage[:, 0].numel() * g.storage.element_size()
                      for g in engine.cache.states)

    sampler = ClockSampler()
    seconds, clocks, mean_context, launches_per_step = time_decode(
        engine, args.batch, args.context, warmup, args.steps, seed=1, sampler=sampler)
    value = args.batch * args.steps / seconds
    step_bytes = weight_bytes + args.batch * (mean_context * kv_per_token + 2 * state_bytes)
    achieved = step_bytes / (seconds / args.steps) / 1e9

    points = {}
    if not args.skip_points:
        for batch in (1, 16, 32, 64):
            s, _, _, _ = time_decode(engine, batch, args.context, warmup, args.steps, seed=2 + batch)
            points[f"decode_b{batch}"] = round(batch * args.steps / s, 1)
        # other context lengths at the default batch, as far as the pool made for batch 64 holds
        for context in (512, 32768):
            if context != args.context and args.batch * context <= 64 * args.context \
                    and context > warmup + args.steps + 66:
                s, _, _, _ = time_decode(engine, args.batch, context, warmup, args.steps,
                                         seed=100 + context)
                points[f"decode_b{args.batch}_context{context}"] = round(args.batch * args.steps / s, 1)

    e2e_seconds, h2d, d2h = time_e2e(engine, args.batch, args.context, warmup, args.steps, seed=7)
    e2e_value = args.batch * args.steps / e2e_seconds

    prefill_seconds = time_prefill(engine, PREFILL_TOKENS, 2, 3, seed=11)
    flops = model_flops(spec, PREFILL_TOKENS)
    products = None if args.skip_points else product_fractions(model, args.batch, peak)

    if not args.skip_points:
        # the two smaller shapes of the family at the default batch and context
        import gc
        del engine, model
        gc.collect()
        torch.cuda.empty_cache()
        for label, shape in (("lfm2_700m", LFM2_700M), ("lfm2_350m", LFM2_350M)):
            small = build_engine(shape, shape["num_hidden_layers"], args.batch, args.context,
                                 warmup + args.steps, name=f"random-{label}")
            small.model.ops.set_dependent_launches(bool(args.dependent_launches))
            s, _, _, _ = time_decode(small, args.batch, args.context, warmup, args.steps, seed=21)
            points[f"decode_b{args.batch}_{label}"] = round(args.batch * args.steps / s, 1)
            del small
            gc.collect()
            torch.cuda.empty_cache()

    line = {
        "metric": f"decode tok/s at batch {args.batch} (LFM2-1.2B shape, bf16, context {args.context})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(seconds / args.steps * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), seeded uniform-random token ids",
        "config": {
            "model": "LFM2-1.2B shape", "layers": args.layers,
            "layers_full_model": LFM2_1_2B["num_hidden_layers"],
            "hidden": spec.hidden_size, "heads": LFM2_1_2B["num_attention_heads"],
            "kv_heads": LFM2_1_2B["num_key_value_heads"],
            "head_dim": spec.hidden_size // LFM2_1_2B["num_attention_heads"],
            "ffn_width": spec.layers[0].feed_forward["width"], "vocab": spec.vocab_size,
            "conv_taps": LFM2_1_2B["conv_L_cache"], "attention_layers":
                sum(1 for l in spec.layers if l.mixer.kind == "attention"),
            "global_batch": args.batch, "seq_len": args.context, "page_size": PAGE_SIZE,
            "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (2.3 GB of weights per step)",
            "peaks": peak["source"],
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s",
                "ms_per_step": round(e2e_seconds / args.steps * 1e3, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_per_step * args.steps,
        "launches_per_step": launches_per_step,
        "prefill": {"value": round(PREFILL_TOKENS / prefill_seconds, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_seconds * 1e3, 3),
                    "frac": round(flops / prefill_seconds / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peak["hbm_gbs"], 4),
                     "bytes_per_step": int(step_bytes)},
        "points": points,
        "products": products,
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
