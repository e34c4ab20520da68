#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second at batch 8 (the headline value),
the same through the Python entry point with host tokens in and out (``e2e``), decode at batch 1
and 64, a 2,048-token prefill, and the fraction of the roofline each reaches.

    python bench.py --gpus 1 --steps K --warmup W          # this engine
    python bench.py --impl reference ...                   # the unmodified reference, if installed

The model has the layer sizes of Qwen2.5-0.5B (BASELINE.json configs[2]) with seeded random
weights; prompts are seeded uniform-random token ids.  A step is one decode step of the whole
batch.  Requests start from a prefix chosen so that the timed steps are centred on a context of
3,072 tokens (a 2,048-token prefix growing to 4,096).  One JSON line is printed.
"""

from __future__ import annotations

import argparse
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
SIZES = MODEL_SIZES["0.5b"]      # the default workload (BASELINE.json configs[2]); --size replaces it
CONTEXT = 4096
CONTEXT_MEAN = 3072
PREFILL_TOKENS = 2048
BLOCK_SIZE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def parse_args():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--size", choices=sorted(MODEL_SIZES), default="0.5b",
                        help="layer sizes: Qwen2.5-0.5B (default, the headline workload), 7B or 14B")
    parser.add_argument("--layers", type=int, default=None,
                        help="fewer layers than the model has (both numbers are reported)")
    parser.add_argument("--skip-points", action="store_true", help="skip decode at batch 1 and 64")
    parser.add_argument("--skip-prefill", action="store_true")
    parser.add_argument("--skip-e2e", action="store_true")
    parser.add_argument("--no-graphs", action="store_true", help="launch every kernel from the host (for profiling)")
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
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.process = None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
        return self

    def __exit__(self, *exc):
        self.samples = []
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
            if len(parts) == 6 and parts[0].isdigit():
                self.samples.append(parts)

    def summary(self):
        if not getattr(self, "samples", None):
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [name for i, name in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": statistics.median(int(s[0]) for s in self.samples),
                "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons}


def model_numbers(config, layers):
    h, i, v = config.hidden_size, config.intermediate_size, config.vocab_size
    hq, hkv, d = config.num_attention_heads, config.num_key_value_heads, config.head_dim
    per_layer = (hq + 2 * hkv) * d * h + (hq + 2 * hkv) * d + h * hq * d + 3 * h * i + 2 * h
    head = v * h          # the head's matrix is read once per step, tied to the embedding or not
    weight_bytes = 2 * (layers * per_layer + head + h)
    kv_bytes_per_token = 2 * layers * hkv * d * 2
    linear_flops_per_token = 2 * layers * ((hq + 2 * hkv) * d * h + h * hq * d + 3 * h * i)
    return {"weight_bytes": weight_bytes, "kv_bytes_per_token": kv_bytes_per_token,
            "linear_flops_per_token": linear_flops_per_token, "head_flops_per_row": 2 * head,
            "attention_flops_per_layer": lambda t: 2 * t * t * hq * d}


def build_runner(layers, max_requests, tokens_per_request):
    import torch

    from mini_llm_runtime_b200.cache import CacheManager
    from mini_llm_runtime_b200.config import Qwen2Config
    from mini_llm_runtime_b200.engine import ModelRunner
    from mini_llm_runtime_b200.models import random_model

    config = Qwen2Config(**dict(SIZES, num_hidden_layers=layers))
    model = random_model(config, seed=0, dtype=torch.bfloat16, device="cuda:0")
    pages = max_requests * -(-tokens_per_request // BLOCK_SIZE)
    cache = CacheManager(model.cache_needs(), page_size=BLOCK_SIZE, num_pages=pages, max_requests=max_requests,
                         max_tokens_per_request=tokens_per_request, dtype=torch.bfloat16, device="cuda:0",
                         max_step_tokens=PREFILL_TOKENS)
    return config, model, ModelRunner(model, cache)


def random_tokens(count, vocab, seed):
    import torch

    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=generator).tolist()


def fill(runner, request_ids, prefix, vocab):
    """Bring every request's cache to ``prefix`` tokens with real prefill steps."""
    from mini_llm_runtime_b200.engine import StepEntry

    for index, rid in enumerate(request_ids):
        runner.cache.create_request(rid)
        tokens = random_tokens(prefix, vocab, 1000 + index)
        for start in range(0, prefix, PREFILL_TOKENS):
            runner.step([StepEntry(rid, tokens[start:start + PREFILL_TOKENS], [])])


def time_decode(runner, request_ids, vocab, steps, warmup, clocks=None):
    """Device time of ``steps`` decode steps of the whole batch (CUDA events), after ``warmup``."""
    import torch

    from mini_llm_runtime_b200.engine import SamplingRows, StepEntry
    from mini_llm_runtime_b200.ops import cuda_ops

    batch = len(request_ids)
    sampling = SamplingRows([0.0] * batch, [0] * batch, [0] * batch)
    tokens = random_tokens(batch, vocab, 7)

    def one_step():
        # borrow: the step hands out its own output buffers (what the engine does too), no copies
        return runner.step([StepEntry(rid, [tokens[i]], [0]) for i, rid in enumerate(request_ids)], sampling, borrow=True)

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches_before = cuda_ops.launches
    replays_before = runner.graph_replays
    if clocks is not None:
        clocks.__enter__()            # sample clocks during the timed steps only
    host_started = time.perf_counter()
    start.record()
    for _ in range(steps):
        one_step()
    end.record()
    host_ms = (time.perf_counter() - host_started) * 1e3
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.__exit__(None, None, None)
    launched = cuda_ops.launches - launches_before
    launched += (runner.graph_replays - replays_before) * runner.launches_per_replay(batch, True)
    print(f"[bench] batch {batch}: device {start.elapsed_time(end) / steps:.3f} ms/step, host issue "
          f"{host_ms / steps:.3f} ms/step, graph replays {runner.graph_replays - replays_before}", file=sys.stderr)
    return start.elapsed_time(end), launched


def decode_point(layers, batch, steps, warmup, context_mean=CONTEXT_MEAN, graphs=True, clocks=None):
    import torch

    prefix = max(1, context_mean - (steps + warmup) // 2)
    config, model, runner = build_runner(layers, batch, CONTEXT)
    runner.use_graphs = runner.use_graphs and graphs
    ids = [f"d{i}" for i in range(batch)]
    fill(runner, ids, prefix, config.vocab_size)
    torch.cuda.synchronize()
    ms, launches = time_decode(runner, ids, config.vocab_size, steps, warmup, clocks)
    for rid in ids:
        runner.cache.release(rid)
    del runner, model
    torch.cuda.empty_cache()
    return ms, launches, prefix


def time_prefill(layers, repeats=5, warmup=3):
    import torch

    from mini_llm_runtime_b200.engine import StepEntry

    config, model, runner = build_runner(layers, 2, PREFILL_TOKENS)
    tokens = random_tokens(PREFILL_TOKENS, config.vocab_size, 99)
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
    del runner, model
    torch.cuda.empty_cache()
    return statistics.median(samples)


def time_e2e(layers, batch, steps, warmup):
    """Decode tokens per second through ContinuousBatchEngine.step(): host token ids in, host
    token ids out, every step copies its inputs from pinned memory and reads its tokens back."""
    import torch

    from mini_llm_runtime_b200.config import Qwen2Config
    from mini_llm_runtime_b200.engine import ContinuousBatchEngine
    from mini_llm_runtime_b200.models import random_model

    config = Qwen2Config(**dict(SIZES, num_hidden_layers=layers))
    model = random_model(config, seed=0, dtype=torch.bfloat16, device="cuda:0")
    prefix = CONTEXT_MEAN - (steps + warmup) // 2
    # step_ahead: the engine launches each decode step behind the previous one, fed on the device
    # with the tokens it chose; every step() still returns that step's tokens on the host
    engine = ContinuousBatchEngine.from_model(model, block_size=BLOCK_SIZE, max_running_requests=batch,
                                              max_batch_tokens=PREFILL_TOKENS, max_model_len=CONTEXT + 1024,
                                              step_ahead=True)
    # Requests that finish their prompt early decode while the others still prefill; leave room
    # for those extra tokens so that all of them are alive through the timed steps.
    slack = batch * (-(-prefix // PREFILL_TOKENS) + 1)
    for index in range(batch):
        engine.submit(f"e{index}", random_tokens(prefix, config.vocab_size, 2000 + index),
                      max_new_tokens=steps + warmup + 1 + slack)
    while any(not engine.scheduler.get_request(f"e{i}").prefilled for i in range(batch)):
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    started = time.perf_counter()
    for _ in range(steps):
        result = engine.step()
        assert len(result.update.emitted_tokens) == batch
    torch.cuda.synchronize()
    seconds = time.perf_counter() - started
    # per step: token ids, positions, segment table, slots, block tables ... (one packed buffer);
    # back: one int32 token per request
    table_width = -(-CONTEXT // BLOCK_SIZE)
    h2d = 4 * batch * 8 + 8 * batch + 4 * batch * table_width + 20 * batch
    del engine, model
    torch.cuda.empty_cache()
    return batch * steps / seconds, h2d, 4 * batch


def run_ours(args):
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    from mini_llm_runtime_b200.config import Qwen2Config

    peak = peaks()
    layers = args.layers
    config = Qwen2Config(**dict(SIZES, num_hidden_layers=layers))
    numbers = model_numbers(config, layers)

    clocks = ClockSampler()
    ms, launches, prefix = decode_point(layers, args.batch, args.steps, args.warmup, args.context_mean,
                                        not args.no_graphs, clocks)
    ms_per_step = ms / args.steps
    value = args.batch * args.steps / (ms / 1e3)
    step_bytes = numbers["weight_bytes"] + args.batch * args.context_mean * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9

    record = {
        "metric": f"decode tokens/s (batch {args.batch}, context 4096)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded random weights and token ids)", "impl": "ours",
        "config": {"model": MODEL_NAMES[args.size], "layers": layers, "layers_of_model": SIZES["num_hidden_layers"],
                   "hidden": config.hidden_size, "q_heads": config.num_attention_heads,
                   "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
                   "intermediate": config.intermediate_size, "vocab": config.vocab_size, "tied_head": config.tie_word_embeddings,
                   "global_batch": args.batch, "seq_len": CONTEXT, "context_mean": args.context_mean,
                   "prefix": prefix, "block_size": BLOCK_SIZE, "prefill_tokens": PREFILL_TOKENS,
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (weights + KV > 1 GB)",
                   "peaks": peak["source"]},
        "clocks": clocks.summary(),
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
    }
    if not args.skip_prefill:
        prefill_ms = time_prefill(layers)
        flops = PREFILL_TOKENS * numbers["linear_flops_per_token"] + numbers["head_flops_per_row"] \
            + layers * numbers["attention_flops_per_layer"](PREFILL_TOKENS)
        record["prefill"] = {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
                             "ms": round(prefill_ms, 3),
                             "frac": round(flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)}
    if not args.skip_points:
        points = {}
        for batch in (1, 64):
            steps = min(args.steps, 64)
            point_ms, _, _ = decode_point(layers, batch, steps, args.warmup)
            points[f"decode_b{batch}"] = round(batch * steps / (point_ms / 1e3), 1)
        record["points"] = points
    if not args.skip_e2e:
        e2e, h2d, d2h = time_e2e(layers, args.batch, args.steps, args.warmup)
        record["e2e"] = {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                         "d2h_bytes_per_step": d2h}
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

    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "mini_llm_runtime")):
        return unavailable("baseline/_ref holds no installed reference (pip install --no-deps --target baseline/_ref)")
    if not os.path.isfile(os.path.join(ROOT, "baseline", "csrc", "paged_attention_cuda.cu")):
        return unavailable("baseline/csrc (the reference's kernel sources) is missing, its CUDA extension cannot be built")
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
        config = QwenConfig(**dict(SIZES, num_hidden_layers=layers))
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
        "metric": "decode tokens/s (batch 8, context 4096)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms / steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp16 (the reference kernel's only dtype)",
        "data": "synthetic (random weights and token ids)", "impl": "reference",
        "config": {"model": MODEL_NAMES[args.size], "layers": layers, "layers_of_model": SIZES["num_hidden_layers"],
                   "global_batch": batch, "seq_len": CONTEXT, "context_mean": args.context_mean, "prefix": prefix,
                   "block_size": BLOCK_SIZE, "parallelism": "single GPU",
                   "path": "ContinuousBatchEngine + paged_cuda decode kernel"},
        "clocks": clocks.summary(),
        "e2e": {"value": round(batch * steps / wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": 8 * batch * 2,
                "d2h_bytes_per_step": 8 * batch},
    }))
    return 0


def main():
    global SIZES
    args = parse_args()
    SIZES = MODEL_SIZES[args.size]
    if args.layers is None:
        args.layers = SIZES["num_hidden_layers"]
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
