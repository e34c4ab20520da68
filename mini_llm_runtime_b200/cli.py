"""Command line of the engine: ``python -m mini_llm_runtime_b200 <command> ...``.

The reference ships no installed command; its entry points are runner scripts with argparse
options (experiments/continuous_batch_engine_runner.py:32-52, experiments/
paged_greedy_generation_runner.py:27-34, scripts/benchmark_batching_policy.py:59-75 there).  The
options below keep those names and meanings where the reference has them (``--model``,
``--block-size``, ``--max-new-tokens``, ``--request-count``, ``--generation-lengths``,
``--max-running-requests``, ``--max-batch-tokens``, ``--warmup``, ``--repeats``,
``--output-dir``).  ``--model`` is a local folder (no download), and prompts are token ids
(``--prompt-ids``) because tokenizers are outside this engine.

Commands:
  generate     one prompt through prefill and one-token steps (greedy or with a temperature)
  serve-batch  a burst of requests through the continuous-batching engine, with request metrics
  make-random  write a model folder with seeded random weights from a config.json
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path


def _int_list(raw: str) -> tuple[int, ...]:
    try:
        values = tuple(int(part.strip()) for part in raw.split(",") if part.strip())
    except ValueError as error:
        raise argparse.ArgumentTypeError("expected comma-separated integers") from error
    if not values:
        raise argparse.ArgumentTypeError("expected at least one integer")
    return values


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="mini_llm_runtime_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    commands = parser.add_subparsers(dest="command", required=True)

    def common(sub):
        sub.add_argument("--model", required=True, help="model folder: config.json + model.safetensors")
        sub.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
        sub.add_argument("--block-size", type=int, default=16, help="tokens per KV cache block")
        sub.add_argument("--total-blocks", type=int, default=None, help="KV cache blocks (default: enough for all)")
        sub.add_argument("--max-running-requests", type=int, default=4)
        sub.add_argument("--max-batch-tokens", type=int, default=2048)
        sub.add_argument("--max-mixed-prefill-tokens", type=int, default=None)
        sub.add_argument("--step-ahead", action="store_true",
                         help="launch each decode step before the previous one's tokens have reached the host")
        sub.add_argument("--max-model-len", type=int, default=None)
        sub.add_argument("--temperature", type=float, default=0.0, help="0 selects greedy")
        sub.add_argument("--seed", type=int, default=0)
        sub.add_argument("--eos-id", type=_int_list, default=None, help="comma-separated EOS token ids")
        sub.add_argument("--output-dir", type=Path, default=None, help="optional folder for result.json")
        sub.add_argument("--device", default="cuda:0")

    generate = commands.add_parser("generate", help="generate from one prompt")
    common(generate)
    generate.add_argument("--prompt-ids", type=_int_list, required=True, help="comma-separated token ids")
    generate.add_argument("--max-new-tokens", type=int, default=8)

    burst = commands.add_parser("serve-batch", help="run a burst of requests through the engine")
    common(burst)
    burst.add_argument("--request-count", type=int, default=8)
    burst.add_argument("--prompt-length", type=int, default=32, help="random prompt length per request")
    burst.add_argument("--prompt-ids", type=_int_list, default=None, help="use this prompt for every request")
    burst.add_argument("--generation-lengths", type=_int_list, default=(2, 4, 8, 12),
                       help="generation lengths, cycled over the requests")
    burst.add_argument("--warmup", type=int, default=0)
    burst.add_argument("--repeats", type=int, default=1)

    random_model = commands.add_parser("make-random", help="write a random-weights model folder")
    random_model.add_argument("--config", type=Path, required=True, help="a config.json to take the sizes from")
    random_model.add_argument("--seed", type=int, default=0)
    random_model.add_argument("--out", type=Path, required=True)
    random_model.add_argument("--storage-dtype", choices=("bfloat16", "float32"), default="bfloat16")
    return parser


def _engine(args):
    import torch

    from .engine import ContinuousBatchEngine

    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device is visible; this engine has no CPU path")
    return ContinuousBatchEngine.from_model_dir(
        args.model, dtype=args.dtype, device=args.device, block_size=args.block_size,
        total_blocks=args.total_blocks, max_running_requests=args.max_running_requests,
        max_batch_tokens=args.max_batch_tokens, max_mixed_prefill_tokens=args.max_mixed_prefill_tokens,
        max_model_len=args.max_model_len, step_ahead=args.step_ahead)


def _write(args, record: dict) -> None:
    print(json.dumps(record))
    if args.output_dir is not None:
        args.output_dir.mkdir(parents=True, exist_ok=True)
        (args.output_dir / "result.json").write_text(json.dumps(record, indent=2))


def command_generate(args) -> int:
    engine = _engine(args)
    started = time.perf_counter()
    engine.submit("cli", list(args.prompt_ids), max_new_tokens=args.max_new_tokens,
                  eos_token_ids=args.eos_id, temperature=args.temperature, seed=args.seed)
    engine.run()
    request = engine.scheduler.get_request("cli")
    _write(args, {"prompt_ids": list(args.prompt_ids), "generated_ids": list(request.generated_token_ids),
                  "finish_reason": request.finish_reason.value, "seconds": time.perf_counter() - started,
                  "metrics": engine.metrics.summary()})
    return 0


def command_serve_batch(args) -> int:
    import torch

    engine = _engine(args)
    vocab = engine.runner.vocab_size
    generator = torch.Generator().manual_seed(args.seed)
    runs = []
    for run in range(args.warmup + args.repeats):
        ids = []
        started = time.perf_counter()
        for index in range(args.request_count):
            prompt = list(args.prompt_ids) if args.prompt_ids else \
                torch.randint(0, vocab, (args.prompt_length,), generator=generator).tolist()
            rid = f"run{run}-req{index}"
            engine.submit(rid, prompt, max_new_tokens=args.generation_lengths[index % len(args.generation_lengths)],
                          eos_token_ids=args.eos_id, temperature=args.temperature, seed=args.seed + index)
            ids.append(rid)
        steps = engine.run()
        seconds = time.perf_counter() - started
        tokens = sum(len(engine.scheduler.get_request(rid).generated_token_ids) for rid in ids)
        if run >= args.warmup:
            runs.append({"seconds": seconds, "steps": len(steps), "generated_tokens": tokens,
                         "tokens_per_second": tokens / seconds,
                         "outputs": {rid: list(engine.scheduler.get_request(rid).generated_token_ids) for rid in ids}})
    _write(args, {"runs": runs, "metrics": engine.metrics.summary(),
                  "cache": engine.manager.stats().__dict__})
    return 0


def command_make_random(args) -> int:
    import torch

    from .config import config_from_dict
    from .models import write_random_model_dir

    config = config_from_dict(json.loads(args.config.read_text()))
    dtype = torch.bfloat16 if args.storage_dtype == "bfloat16" else torch.float32
    path = write_random_model_dir(args.out, config, args.seed, dtype)
    print(f"wrote {path}")
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return {"generate": command_generate, "serve-batch": command_serve_batch,
            "make-random": command_make_random}[args.command](args)


if __name__ == "__main__":
    sys.exit(main())
