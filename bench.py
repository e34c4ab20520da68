#!/usr/bin/env python3
"""Benchmark of the engine on one B200.

    python bench.py --gpus 1 --steps K --warmup W          # this engine
    python bench.py --impl reference ...                   # the unmodified reference, if installed

The headline is decode tokens per second at batch 8 on the layer sizes of Qwen2.5-0.5B (24 layers,
context 4,096, random weights; ``--size`` picks 7b or 14b instead), timed on the device as R regions
of exactly K decode steps each; the median region is the value and the raw samples are listed.  The
same line carries: the same metric through the Python entry point with host tokens in and out
(``e2e``), a 2,048-token prefill, decode at batch 1 and 64, the fraction of the measured roofline
each reaches, and (unless ``--skip-sizes``) points for the 7B and 14B layer sizes: decode at batch
1 / 8 / 64, prefill, a mixed step of 8 decodes beside a 512-token prompt portion (7B), and a
continuous-batching run of 64 requests (14B); decode at contexts of 16k and 32k tokens and an 8k
prompt in 2,048-token portions (0.5B and 7B).  One JSON line is printed.

A step is one decode step of the whole batch.  Requests start from a prefix chosen so that the
timed steps are centred on a context of 3,072 tokens (a 2,048-token prefix growing to 4,096).
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL_SIZES = {
    "0.5b": dict(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_hidden_layers=24,
                 num_attention_heads=14, num_key_value_heads=2, max_position_embeddings=32768,
                 rms_norm_eps=1e-6, rope_theta=1000000.0, hidden_act="silu", tie_word_embeddings=True),
    "7b": dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
               num_attention_heads=28, num_key_value_heads=4, max_position_embeddings=32768,
               rms_norm_eps=1e-6, rope_theta=1000000.0, hidden_act="silu", tie_word_embeddings=False),
    "14b": dict(vocab_size=152064, hidden_size=5120, intermediate_size=13824, num_hidden_layers=48,
                num_attention_heads=40, num_key_value_heads=8, max_position_embeddings=32768,
                rms_norm_eps=1e-5, rope_theta=1000000.0, hidden_act="silu", tie_word_embeddings=False),
}
MODEL_NAMES = {"0.5b": "Qwen2.5-0.5B sizes", "7b": "Qwen2.5-7B sizes", "14b": "Qwen2.5-14B sizes"}
CONTEXT = 4096
CONTEXT_MEAN = 3072
PREFILL_TOKENS = 2048
BLOCK_SIZE = 16
REPEATS = 5
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def parse_args():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=32)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--size", choices=sorted(MODEL_SIZES), default="0.5b",
                        help="layer sizes of the headline: Qwen2.5-0.5B (default), 7B or 14B")
    parser.add_argument("--layers", type=int, default=None,
                        help="fewer layers than the model has (both numbers are reported)")
    parser.add_argument("--repeats", type=int, default=REPEATS, help="timed regions of --steps steps each")
    parser.add_argument("--skip-points", action="store_true", help="skip decode at batch 1 and 64")
    parser.add_argument("--skip-prefill", action="store_true")
    parser.add_argument("--skip-e2e", action="store_true")
    parser.add_argument("--skip-sizes", action="store_true", help="skip the points at the 7B and 14B layer sizes")
    parser.add_argument("--skip-long", action="store_true",
                        help="skip decode at contexts of 16k and 32k tokens and the 8k prompt in portions")
    parser.add_argument("--no-graphs", action="store_true", help="launch every kernel from the host (for profiling)")
    parser.add_argument("--no-arena", action="store_true",
                        help="place the weights without first touching one block of their total size (A/B)")
    parser.add_argument("--gemm", default=None, metavar="M,N,K[,swiglu]",
                        help="time this engine's bfloat16 product x[M,K] W[N,K]^T on one shape (weights rotate over "
                             "copies larger than L2) and print a small JSON record; nothing else runs")
    parser.add_argument("--context-mean", type=int, default=CONTEXT_MEAN,
                        help="context length the timed steps are centred on (default 3072)")
    return parser.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as handle:
                data = json.load(handle)
            return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                    "source": "measured"}
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks, utilisation and throttle reasons with nvidia-smi from start to stop; the
    summary is taken over the samples during which the GPU was busy."""

    QUERY = ("clocks.sm,clocks.max.sm,utilization.gpu,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self):
        self.process = None
        self.samples = []

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
        return self

    def __exit__(self, *exc):
        if self.process is None:
            return
        self.process.terminate()
        try:
            output, _ = self.process.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
            output, _ = self.process.communicate()
        for line in output.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 7 and parts[0].isdigit():
                self.samples.append(parts)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        busy = [s for s in self.samples if s[2].isdigit() and int(s[2]) >= 10] or self.samples
        reasons = [name for i, name in enumerate(self.NAMES) if any(s[3 + i].lower().startswith("active") for s in busy)]
        return {"sm_mhz": statistics.median(int(s[0]) for s in busy), "sm_max_mhz": int(busy[0][1]),
                "reasons": reasons, "samples": len(busy)}


def environment():
    """Where the number was taken: GPU, driver, CUDA, torch, and what source it was (the git head
    where the checkout has one, else a hash over the package's sources)."""
    import torch

    record = {"torch": torch.__version__, "cuda": torch.version.cuda, "python": sys.version.split()[0]}
    try:
        record["gpu"] = torch.cuda.get_device_name(0)
        record["sm_count"] = torch.cuda.get_device_properties(0).multi_processor_count
        record["driver"] = subprocess.run(["nvidia-smi", "--query-gpu=driver_version", "--format=csv,noheader"],
                                          capture_output=True, text=True, timeout=20).stdout.strip().splitlines()[0]
    except Exception:  # noqa: BLE001
        pass
    try:
        head = subprocess.run(["git", "-C", ROOT, "rev-parse", "--short=12", "HEAD"], capture_output=True, text=True,
                              timeout=20)
        if head.returncode == 0 and head.stdout.strip():
            record["git_head"] = head.stdout.strip()
    except Exception:  # noqa: BLE001
        pass
    digest = hashlib.sha256()
    package = os.path.join(ROOT, "mini_llm_runtime_b200")
    for folder, _, files in sorted(os.walk(package)):
        if "_build" in folder or "__pycache__" in folder:
            continue
        for name in sorted(files):
            if name.endswith((".py", ".cu", ".cuh", ".h")):
                with open(os.path.join(folder, name), "rb") as handle:
                    digest.update(name.encode() + handle.read())
    record["source_sha16"] = digest.hexdigest()[:16]
    return record


def model_numbers(config, layers):
    h, i, v = config.hidden_size, config.intermediate_size, config.vocab_size
    hq, hkv, d = config.num_attention_heads, config.num_key_value_heads, config.head_dim
    per_layer = (hq + 2 * hkv) * d * h + (hq + 2 * hkv) * d + h * hq * d + 3 * h * i + 2 * h
    head = v * h          # the head's matrix is read once per step, tied to the embedding or not
    return {"weight_bytes": 2 * (layers * per_layer + head + h),
            "kv_bytes_per_token": 2 * layers * hkv * d * 2,
            "linear_flops_per_token": 2 * layers * ((hq + 2 * hkv) * d * h + h * hq * d + 3 * h * i),
            "head_flops_per_row": 2 * head,
            # causal attention of `rows` new rows on top of `before` cached ones: QK^T and PV
            "attention_flops": lambda rows, before=0: layers * 4 * hq * d * (rows * before + rows * (rows + 1) // 2)}


def random_tokens(count, vocab, seed):
    import torch

    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=generator).tolist()


class Workbench:
    """One model of the given layer sizes with random weights drawn on the device, and runners on it."""

    def __init__(self, size, layers=None, arena=True):
        import torch

        from mini_llm_runtime_b200.config import Qwen2Config
        from mini_llm_runtime_b200.models import random_model

        self.size = size
        self.sizes = MODEL_SIZES[size]
        self.layers = layers or self.sizes["num_hidden_layers"]
        self.config = Qwen2Config(**dict(self.sizes, num_hidden_layers=self.layers))
        self.model = random_model(self.config, seed=0, dtype=torch.bfloat16, device="cuda:0", draw_on_device=True,
                                  arena=arena)
        self.numbers = model_numbers(self.config, self.layers)

    def runner(self, max_requests, tokens_per_request, pages=None):
        import torch

        from mini_llm_runtime_b200.cache import CacheManager
        from mini_llm_runtime_b200.engine import ModelRunner

        pages = pages or max_requests * -(-tokens_per_request // BLOCK_SIZE)
        cache = CacheManager(self.model.cache_needs(), page_size=BLOCK_SIZE, num_pages=pages,
                             max_requests=max_requests, max_tokens_per_request=tokens_per_request,
                             dtype=torch.bfloat16, device="cuda:0", max_step_tokens=PREFILL_TOKENS)
        return ModelRunner(self.model, cache)

    def close(self):
        import torch

        self.model = None
        torch.cuda.empty_cache()


def fill(runner, request_ids, prefix, vocab, real_prefill):
    """Bring every request's cache to ``prefix`` tokens: with real prefill steps, or (for the large
    sizes, where prefill of every request would take longer than everything timed) by declaring the
    length and filling the pools with random keys and values; a decode step reads the same bytes
    either way."""
    from mini_llm_runtime_b200.engine import StepEntry

    for index, rid in enumerate(request_ids):
        runner.cache.create_request(rid)
        if real_prefill:
            tokens = random_tokens(prefix, vocab, 1000 + index)
            for start in range(0, prefix, PREFILL_TOKENS):
                runner.step([StepEntry(rid, tokens[start:start + PREFILL_TOKENS], [])])
        else:
            runner.cache.adopt(rid, prefix)
    if not real_prefill:
        for group in runner.cache.groups:
            group.key.normal_(0.0, 0.5)
            group.value.normal_(0.0, 0.5)


def time_regions(run_region, repeats):
    """Device time (CUDA events) of ``repeats`` regions; returns the samples in ms."""
    import torch

    samples = []
    for _ in range(repeats):
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        run_region()
        end.record()
        torch.cuda.synchronize()
        samples.append(start.elapsed_time(end))
    return samples


def decode_point(bench, batch, steps, warmup, repeats, context_mean=CONTEXT_MEAN, graphs=True, real_prefill=True):
    """Median device time per decode step at this batch size, the raw samples, kernels launched in
    one region, and the bytes a step has to read."""
    import torch

    from mini_llm_runtime_b200.engine import StepEntry
    from mini_llm_runtime_b200.ops import cuda_ops

    total_steps = warmup + repeats * steps
    prefix = max(1, context_mean - total_steps // 2)
    runner = bench.runner(batch, max(CONTEXT, prefix + total_steps + 1))
    runner.use_graphs = runner.use_graphs and graphs
    ids = [f"d{i}" for i in range(batch)]
    fill(runner, ids, prefix, bench.config.vocab_size, real_prefill)
    entries = [StepEntry(rid, [0], [0]) for rid in ids]

    def one_step():
        # As the engine runs a decode step: tokens sampled on the device by slot, each request's input
        # taken from its slot record (feed), the step's own output buffers handed out (borrow).
        runner.step(entries, sample=True, borrow=True, feed=True)

    for _ in range(warmup):
        one_step()
    launches_before, replays_before = cuda_ops.launches, runner.graph_replays
    host_started = time.perf_counter()
    samples = time_regions(lambda: [one_step() for _ in range(steps)], repeats)
    host_ms = (time.perf_counter() - host_started) * 1e3
    launched = cuda_ops.launches - launches_before
    launched += (runner.graph_replays - replays_before) * runner.launches_per_replay(batch, True, True)
    runner.check_device()
    for rid in ids:
        runner.cache.release(rid)
    del runner
    torch.cuda.empty_cache()
    ms_per_step = statistics.median(samples) / steps
    step_bytes = bench.numbers["weight_bytes"] + batch * context_mean * bench.numbers["kv_bytes_per_token"]
    print(f"[bench] {bench.size} batch {batch}: {ms_per_step:.3f} ms/step (median of {repeats} x {steps} steps; "
          f"host {host_ms / (repeats * steps):.3f} ms/step)", file=sys.stderr)
    return {"ms_per_step": ms_per_step, "samples_ms_per_step": [round(s / steps, 4) for s in samples],
            "launches": launched // repeats, "prefix": prefix, "step_bytes": step_bytes,
            "tokens_per_s": batch / (ms_per_step / 1e3)}


def time_prefill(bench, repeats=REPEATS, warmup=3):
    import torch

    from mini_llm_runtime_b200.engine import StepEntry

    import numpy as np

    runner = bench.runner(2, PREFILL_TOKENS)
    # as the engine hands a prompt's portion to the step: an int32 array, not a list of Python integers
    tokens = np.asarray(random_tokens(PREFILL_TOKENS, bench.config.vocab_size, 99), dtype=np.int32)
    samples = []
    for attempt in range(warmup + repeats):
        runner.cache.create_request("p")
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry("p", tokens, [PREFILL_TOKENS - 1])])
        end.record()
        torch.cuda.synchronize()
        runner.cache.release("p")
        if attempt >= warmup:
            samples.append(start.elapsed_time(end))
    runner.check_device()
    del runner
    torch.cuda.empty_cache()
    ms = statistics.median(samples)
    flops = (PREFILL_TOKENS * bench.numbers["linear_flops_per_token"] + bench.numbers["head_flops_per_row"]
             + bench.numbers["attention_flops"](PREFILL_TOKENS))
    return ms, flops, samples


def time_portioned_prefill(bench, total=8192, portion=PREFILL_TOKENS, repeats=3, warmup=1):
    """A prompt of ``total`` tokens fed in portions of ``portion`` (each attends to the cached ones
    before it); returns the median time of the whole prompt and its flops."""
    import torch

    from mini_llm_runtime_b200.engine import StepEntry

    runner = bench.runner(2, total)
    tokens = random_tokens(total, bench.config.vocab_size, 98)
    samples = []
    for attempt in range(warmup + repeats):
        runner.cache.create_request("p")
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for first in range(0, total, portion):
            last = first + portion >= total
            runner.step([StepEntry("p", tokens[first:first + portion], [portion - 1] if last else [])])
        end.record()
        torch.cuda.synchronize()
        runner.cache.release("p")
        if attempt >= warmup:
            samples.append(start.elapsed_time(end))
    runner.check_device()
    del runner
    torch.cuda.empty_cache()
    flops = total * bench.numbers["linear_flops_per_token"] + bench.numbers["head_flops_per_row"] \
        + sum(bench.numbers["attention_flops"](min(portion, total - first), first) for first in range(0, total, portion))
    return statistics.median(samples), flops


def long_context_points(bench, peak, record, prefix):
    """Decode at batch 8 with contexts of 16k and 32k tokens, and an 8k prompt in 2,048-token portions."""
    detail = {}
    for context in (16384, 32768):
        point = decode_point(bench, 8, 8, 3, 3, context_mean=context - 64, real_prefill=False)
        achieved = point["step_bytes"] / (point["ms_per_step"] / 1e3) / 1e9
        name = f"{prefix}decode_b8_ctx{context // 1024}k"
        record["points"][name] = round(point["tokens_per_s"], 1)
        record["points"][name + "_hbm_frac"] = round(achieved / peak["hbm_gbs"], 4)
        detail[name] = {"ms": round(point["ms_per_step"], 3), "gb_per_step": round(point["step_bytes"] / 1e9, 2)}
    ms, flops = time_portioned_prefill(bench)
    record["points"][f"{prefix}prefill_8k_in_2k_portions"] = round(8192 / (ms / 1e3), 1)
    record["points"][f"{prefix}prefill_8k_in_2k_portions_frac"] = round(flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)
    detail[f"{prefix}prefill_8k"] = {"ms": round(ms, 3)}
    return detail


def time_mixed_step(bench, peak, decodes=8, portion=512, context=CONTEXT_MEAN, repeats=REPEATS, warmup=3):
    """One step of ``decodes`` decoded tokens (context ``context``) beside a ``portion``-token piece
    of a longer prompt that already has tokens cached."""
    import torch

    from mini_llm_runtime_b200.engine import StepEntry

    runner = bench.runner(decodes + 1, max(CONTEXT, portion * (3 + warmup + repeats)))
    ids = [f"m{i}" for i in range(decodes)]
    fill(runner, ids, context, bench.config.vocab_size, real_prefill=False)
    prompt = random_tokens(portion * (2 + warmup + repeats), bench.config.vocab_size, 5)
    runner.cache.create_request("prompt")
    runner.step([StepEntry("prompt", prompt[:portion], [])])
    samples, cursor = [], portion
    for attempt in range(warmup + repeats):
        entries = [StepEntry(rid, [1], [0]) for rid in ids] + [StepEntry("prompt", prompt[cursor:cursor + portion], [])]
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step(entries, sample=True, borrow=True)
        end.record()
        torch.cuda.synchronize()
        cursor += portion
        if attempt >= warmup:
            samples.append(start.elapsed_time(end))
    runner.check_device()
    del runner
    torch.cuda.empty_cache()
    ms = statistics.median(samples)
    before = portion * (1 + warmup + repeats // 2)            # tokens the prompt has cached at the median sample
    numbers = bench.numbers
    rows = decodes + portion
    flops = rows * numbers["linear_flops_per_token"] + decodes * numbers["head_flops_per_row"] \
        + numbers["attention_flops"](portion, before) + decodes * numbers["attention_flops"](1, context)
    step_bytes = numbers["weight_bytes"] + (decodes * context + before) * numbers["kv_bytes_per_token"]
    return {"ms": round(ms, 3), "tokens": rows, "hbm_frac": round(step_bytes / (ms / 1e3) / 1e9 / peak["hbm_gbs"], 4),
            "flops_frac": round(flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4),
            "samples_ms": [round(s, 3) for s in samples]}


def continuous_batching(bench, requests=64, budget=2048, seed=3):
    """The engine under load: ``requests`` requests arrive at once, prompt lengths uniform in
    [128, 2048], generation lengths cycling 32/64/128/256, at most ``budget`` tokens per step."""
    import random

    import torch

    from mini_llm_runtime_b200.engine import ContinuousBatchEngine

    rng = random.Random(seed)
    lengths = [rng.randint(128, 2048) for _ in range(requests)]
    generate = [(32, 64, 128, 256)[i % 4] for i in range(requests)]
    # The workload runs twice and the second run counts: the first also pays for what a server
    # pays once (first use of each shape, the allocator's growth).
    for run in range(2):
        engine = ContinuousBatchEngine.from_model(bench.model, block_size=BLOCK_SIZE, max_running_requests=requests,
                                                  max_batch_tokens=budget, max_model_len=2048 + 256, step_ahead=True)
        engine.generate([random_tokens(64, bench.config.vocab_size, 1)] * 2, max_new_tokens=4)     # warm-up
        torch.cuda.synchronize()
        started = time.perf_counter()
        for index in range(requests):
            engine.submit(f"c{index}", random_tokens(lengths[index], bench.config.vocab_size, 3000 + index),
                          max_new_tokens=generate[index])
        steps = engine.run()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - started
        timelines = [engine.metrics.get(f"c{index}") for index in range(requests)]
        tokens = sum(len(t.token_ids) for t in timelines)
        del engine
        torch.cuda.empty_cache()
    return {"tokens_per_s": round(tokens / seconds, 1), "seconds": round(seconds, 3), "steps": len(steps),
            "generated_tokens": tokens, "prompt_tokens": sum(lengths),
            "ttft_ms_median": round(statistics.median(t.ttft_ms for t in timelines), 2),
            "tpot_ms_median": round(statistics.median(t.median_tpot_ms for t in timelines), 3)}


def time_e2e(bench, batch, steps, warmup, repeats):
    """Decode tokens per second through ContinuousBatchEngine.step(): host token ids in at submit,
    host token ids out of every step; whatever a step has to send is copied from pinned memory, and
    its tokens are read back.  The bytes sent are counted by the runner, not assumed."""
    import torch

    from mini_llm_runtime_b200.engine import ContinuousBatchEngine

    total_steps = warmup + repeats * steps
    prefix = CONTEXT_MEAN - total_steps // 2
    # step_ahead: the engine launches each decode step behind the previous one (the device takes the
    # inputs from the slot records); every step() still returns that step's tokens on the host
    engine = ContinuousBatchEngine.from_model(bench.model, block_size=BLOCK_SIZE, max_running_requests=batch,
                                              max_batch_tokens=PREFILL_TOKENS, max_model_len=CONTEXT + 1024,
                                              step_ahead=True)
    # Requests that finish their prompt early decode while the others still prefill; leave room
    # for those extra tokens so that all of them are alive through the timed steps.
    slack = batch * (-(-prefix // PREFILL_TOKENS) + 1)
    for index in range(batch):
        engine.submit(f"e{index}", random_tokens(prefix, bench.config.vocab_size, 2000 + index),
                      max_new_tokens=total_steps + 1 + slack)
    while any(not engine.scheduler.get_request(f"e{i}").prompt_done for i in range(batch)):
        engine.step()
    for _ in range(warmup):
        engine.step()
    samples = []
    sent_before = engine.runner.bytes_sent
    for _ in range(repeats):
        torch.cuda.synchronize()
        started = time.perf_counter()
        for _ in range(steps):
            result = engine.step()
            assert len(result.outcome.emitted_tokens) == batch
        torch.cuda.synchronize()
        samples.append(time.perf_counter() - started)
    h2d = (engine.runner.bytes_sent - sent_before) / (repeats * steps)
    del engine
    torch.cuda.empty_cache()
    return (batch * steps / statistics.median(samples), round(h2d, 1), 4 * batch,
            [round(batch * steps / s, 1) for s in samples])


def headline_config(size, config, layers, batch, context_mean, peak_source):
    """The flat ``config`` both arms print (at most 20 keys)."""
    return {"model": MODEL_NAMES[size], "layers": layers, "layers_of_model": MODEL_SIZES[size]["num_hidden_layers"],
            "hidden": config.hidden_size, "q_heads": config.num_attention_heads,
            "kv_heads": config.num_key_value_heads, "head_dim": config.hidden_size // config.num_attention_heads,
            "intermediate": config.intermediate_size, "vocab": config.vocab_size,
            "tied_head": config.tie_word_embeddings, "global_batch": batch, "seq_len": CONTEXT,
            "context_mean": context_mean, "block_size": BLOCK_SIZE,
            "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (weights + KV > 1 GB)", "peaks": peak_source}


def size_points(size, args, peak, record):
    """Points at another model size: decode at batch 1 / 8 / 64, prefill of 2,048 tokens, and the
    workload named for that size (7B: a mixed step; 14B: continuous batching of 64 requests)."""
    bench = Workbench(size, arena=not args.no_arena)
    steps, repeats = min(args.steps, 16), 3
    detail = {"layers": bench.layers, "weight_gb": round(bench.numbers["weight_bytes"] / 1e9, 2)}
    for batch in (1, 8, 64):
        point = decode_point(bench, batch, steps, 3, repeats, real_prefill=False)
        achieved = point["step_bytes"] / (point["ms_per_step"] / 1e3) / 1e9
        record["points"][f"{size}_decode_b{batch}"] = round(point["tokens_per_s"], 1)
        record["points"][f"{size}_decode_b{batch}_hbm_frac"] = round(achieved / peak["hbm_gbs"], 4)
        detail[f"decode_b{batch}"] = {"ms": round(point["ms_per_step"], 3),
                                      "gb_per_step": round(point["step_bytes"] / 1e9, 2),
                                      "hbm_frac": round(achieved / peak["hbm_gbs"], 4),
                                      "samples_ms": point["samples_ms_per_step"]}
    ms, flops, samples = time_prefill(bench, repeats=3, warmup=2)
    frac = round(flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)
    record["points"][f"{size}_prefill_2048"] = round(PREFILL_TOKENS / (ms / 1e3), 1)
    record["points"][f"{size}_prefill_2048_frac"] = frac
    detail["prefill_2048"] = {"ms": round(ms, 3), "frac": frac, "samples_ms": [round(s, 3) for s in samples]}
    if size == "7b":
        detail["mixed_8_decodes_512_portion"] = time_mixed_step(bench, peak)
        record["points"]["7b_mixed_step_ms"] = detail["mixed_8_decodes_512_portion"]["ms"]
        if not args.skip_long:
            detail["long_contexts"] = long_context_points(bench, peak, record, "7b_")
    if size == "14b":
        detail["continuous_64_requests"] = continuous_batching(bench)
        record["points"]["14b_continuous_tokens_per_s"] = detail["continuous_64_requests"]["tokens_per_s"]
    bench.close()
    return detail


def run_gemm(args):
    """One product shape in isolation (for profiles of the GEMM kernels): CUDA events around
    ``--steps`` calls after ``--warmup``, the weight rotating over copies that together exceed L2."""
    import torch

    from mini_llm_runtime_b200 import ops

    fields = [int(v) for v in args.gemm.split(",")]
    M, N, K = fields[:3]
    swiglu = len(fields) > 3 and fields[3] != 0
    kernels = ops.current()
    x = (torch.randn(M, K, device="cuda:0") * 0.5).bfloat16()
    copies = max(2, min(16, int(400e6 // (N * K * 2)) + 1))
    weights = [(torch.randn(N, K, device="cuda:0") * 0.05).bfloat16() for _ in range(copies)]

    def call(i):
        w = weights[i % copies]
        return kernels.linear_swiglu(x, w, 64) if swiglu else kernels.linear(x, w)

    for i in range(args.warmup):
        call(i)
    samples = time_regions(lambda: [call(i) for i in range(args.steps)], args.repeats)
    kernels.raise_if_device_error()
    us = statistics.median(samples) / args.steps * 1e3
    peak = peaks()
    flops = 2.0 * M * N * K
    print(json.dumps({"gemm": [M, N, K], "swiglu": swiglu, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1),
                      "frac_of_burst": round(flops / us / 1e6 / peak["bf16_tflops"], 4),
                      "weight_gbs": round(N * K * 2 / us / 1e3, 1), "samples_us": [round(v / args.steps * 1e3, 2) for v in samples]}))
    return 0


def run_ours(args):
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    peak = peaks()
    with ClockSampler() as clocks:
        bench = Workbench(args.size, args.layers, arena=not args.no_arena)
        config, layers = bench.config, bench.layers
        small = args.size == "0.5b"
        head = decode_point(bench, args.batch, args.steps, args.warmup, args.repeats, args.context_mean,
                            not args.no_graphs, real_prefill=small)
        ms_per_step = head["ms_per_step"]
        achieved = head["step_bytes"] / (ms_per_step / 1e3) / 1e9
        record = {
            "metric": f"decode tokens/s (batch {args.batch}, context 4096)", "value": round(head["tokens_per_s"], 1),
            "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)", "impl": "ours",
            "config": headline_config(args.size, config, layers, args.batch, args.context_mean, peak["source"]),
            "prefix": head["prefix"], "repeats": args.repeats, "samples_ms_per_step": head["samples_ms_per_step"],
            "gpu_launches": head["launches"],
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / peak["hbm_gbs"], 4)},
        }
        if not args.skip_prefill:
            prefill_ms, flops, samples = time_prefill(bench)
            record["prefill"] = {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
                                 "ms": round(prefill_ms, 3),
                                 "frac": round(flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4),
                                 "samples_ms": [round(s, 3) for s in samples]}
        record["points"] = {}
        if not args.skip_points:
            for batch in (1, 64):
                point = decode_point(bench, batch, min(args.steps, 32), args.warmup, 3, real_prefill=small)
                record["points"][f"decode_b{batch}"] = round(point["tokens_per_s"], 1)
                record["points"][f"decode_b{batch}_hbm_frac"] = round(
                    point["step_bytes"] / (point["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"], 4)
        if not args.skip_long and small:
            record["long_contexts"] = long_context_points(bench, peak, record, "")
        if not args.skip_e2e:
            e2e, h2d, d2h, samples = time_e2e(bench, args.batch, args.steps, args.warmup, args.repeats)
            record["e2e"] = {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                             "d2h_bytes_per_step": d2h, "samples": samples}
        bench.close()
        if not args.skip_sizes and small:
            record["sizes"] = {}
            for size in ("7b", "14b"):
                try:
                    record["sizes"][size] = size_points(size, args, peak, record)
                except Exception as error:  # noqa: BLE001  (a point that fails must not lose the headline)
                    record["sizes"][size] = {"error": f"{type(error).__name__}: {error}"[:300]}
                    torch.cuda.empty_cache()
    record["clocks"] = clocks.summary()
    record["environment"] = environment()
    print(json.dumps(record))
    return 0


def run_reference(args):
    """The unmodified reference (installed into baseline/_ref) on the same workload: its
    ContinuousBatchEngine with its paged CUDA decode kernel, float16 (the only dtype that kernel
    takes), random weights of the same sizes, 8 requests decoding from the same prefix.  Its
    extension loader looks for csrc/ two levels above the installed package, i.e. baseline/csrc,
    which holds an untouched copy of the reference's csrc/ (the wheel does not ship it)."""
    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    sizes = MODEL_SIZES[args.size]
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "mini_llm_runtime")):
        return unavailable("baseline/_ref holds no installed reference (pip install --no-deps --target baseline/_ref)")
    if not os.path.isfile(os.path.join(ROOT, "baseline", "csrc", "paged_attention_cuda.cu")):
        return unavailable("baseline/csrc (the reference's kernel sources) is missing, its CUDA extension cannot be built")
    if not sizes["tie_word_embeddings"]:
        return unavailable("the reference rejects checkpoints with an untied head (qwen_config.py:43-44); "
                           "only the 0.5B sizes can run on it")
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        sys.path.insert(0, ref_root)
        from mini_llm_runtime.block_admission import PagedBlockAdmissionController
        from mini_llm_runtime.engine import ContinuousBatchEngine
        from mini_llm_runtime.paged_kv_manager import PagedKVCacheManager
        from mini_llm_runtime.qwen_config import QwenConfig
        from mini_llm_runtime.qwen_model_runner import QwenPrefillRunner
        from mini_llm_runtime.qwen_weights import QwenWeights
        from mini_llm_runtime.scheduler import RequestScheduler
    except Exception as error:  # noqa: BLE001
        return unavailable(f"the installed reference cannot be imported: {type(error).__name__}: {error}"[:300])

    try:
        device = torch.device("cuda:0")
        layers = args.layers
        config = QwenConfig(**dict(sizes, num_hidden_layers=layers))
        generator = torch.Generator(device=device).manual_seed(0)

        def rand(*shape, mean=0.0):
            return (torch.randn(*shape, generator=generator, device=device) * 0.02 + mean).half()

        h, i, kv = config.hidden_size, config.intermediate_size, config.num_key_value_heads * config.head_dim
        state = {"model.embed_tokens.weight": rand(config.vocab_size, h), "model.norm.weight": rand(h, mean=1.0)}
        for index in range(layers):
            p = f"model.layers.{index}."
            state.update({
                p + "input_layernorm.weight": rand(h, mean=1.0), p + "post_attention_layernorm.weight": rand(h, mean=1.0),
                p + "self_attn.q_proj.weight": rand(h, h), p + "self_attn.q_proj.bias": rand(h),
                p + "self_attn.k_proj.weight": rand(kv, h), p + "self_attn.k_proj.bias": rand(kv),
                p + "self_attn.v_proj.weight": rand(kv, h), p + "self_attn.v_proj.bias": rand(kv),
                p + "self_attn.o_proj.weight": rand(h, h), p + "mlp.gate_proj.weight": rand(i, h),
                p + "mlp.up_proj.weight": rand(i, h), p + "mlp.down_proj.weight": rand(h, i)})
        runner = QwenPrefillRunner(config, QwenWeights.from_state_dict(config, state), decode_attention_backend="paged_cuda")
        batch, steps, warmup = args.batch, args.steps, args.warmup
        prefix = max(1, args.context_mean - (steps + warmup) // 2)
        blocks = batch * -(-(prefix + steps + warmup + 2) // BLOCK_SIZE)
        manager = PagedKVCacheManager(total_blocks=blocks, block_size=BLOCK_SIZE, num_layers=layers,
                                      num_kv_heads=config.num_key_value_heads, head_dim=config.head_dim,
                                      dtype=torch.float16, device=device)
        admission = PagedBlockAdmissionController(manager)
        scheduler = RequestScheduler(max_running_requests=batch, max_batch_tokens=batch * prefix + batch,
                                     admission_callback=admission.try_admit)
        engine = ContinuousBatchEngine(scheduler=scheduler, runner=runner, admission=admission)
        for index in range(batch):
            engine.submit(f"r{index}", random_tokens(prefix, config.vocab_size, 2000 + index),
                          max_new_tokens=steps + warmup + 1)
        engine.step()                                    # packed prefill of all prompts
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler() as clocks:
            wall = time.perf_counter()
            start.record()
            for _ in range(steps):
                result = engine.step()
                assert len(result.update.emitted_tokens) == batch
            end.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - wall
        ms = start.elapsed_time(end)
    except Exception as error:  # noqa: BLE001
        return unavailable(f"the reference failed on this workload: {type(error).__name__}: {error}"[:300])

    value = batch * steps / (ms / 1e3)
    print(json.dumps({
        "metric": f"decode tokens/s (batch {batch}, context 4096)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms / steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp16 (the reference kernel's only dtype)",
        "data": "synthetic (random weights and token ids)", "impl": "reference",
        "path": "ContinuousBatchEngine + paged_cuda decode kernel",
        "config": headline_config(args.size, config, layers, batch, args.context_mean, peaks()["source"]),
        "prefix": prefix, "clocks": clocks.summary(),
        "e2e": {"value": round(batch * steps / wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": 8 * batch * 2,
                "d2h_bytes_per_step": 8 * batch},
    }))
    return 0


def main():
    args = parse_args()
    if args.layers is None:
        args.layers = MODEL_SIZES[args.size]["num_hidden_layers"]
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    if args.gemm:
        return run_gemm(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
