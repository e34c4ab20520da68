"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and owns no model code: it loads the model through the architecture registry
and drives the same ``ModelRunner.step``, cache manager and kernels that generation uses.  The
reference has no such program; its nearest relative records ``engine.step()`` results of fixed
scenarios (scripts/check_engine_ragged_continuation.py:515-551 there).

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--block-size P]

Standard input carries one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch; ``want`` lists the places among an entry's tokens whose
logits are written, ``end`` the requests whose pages are given back after the step.  For a step
that wants something, ``<out>/<step>.f32`` receives little-endian float32 [wanted, vocab] in the
order of the entries and of their ``want``.  After every step a line ``done <step>`` is printed
and flushed.  The cache pool holds ``--max-tokens`` tokens per group of layers, so pages are
reused as requests end.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch


def parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    parser.add_argument("--out", required=True, help="folder that receives <step>.f32")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (pool size)")
    parser.add_argument("--block-size", type=int, default=16, help="tokens per cache page (default 16)")
    parser.add_argument("--max-requests", type=int, default=8, help="request slots (default 8)")
    parser.add_argument("--device", default="cuda:0")
    return parser.parse_args(argv)


def main(argv=None) -> int:
    args = parse_args(argv)
    if args.max_tokens <= 0 or args.block_size <= 0:
        print("trace_run: --max-tokens and --block-size must be positive", file=sys.stderr)
        return 2
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device is visible; this engine has no CPU path", file=sys.stderr)
        return 3

    from .cache import CacheManager
    from .engine import ModelRunner, StepEntry
    from .models import load_model

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    dtype = torch.float32 if args.dtype == "float32" else torch.bfloat16
    if dtype == torch.float32:
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
    config, model = load_model(args.model, dtype, args.device)
    pages = -(-args.max_tokens // args.block_size)
    per_request = min(args.max_tokens, model.spec.max_positions)
    cache = CacheManager(model.cache_needs(), page_size=args.block_size, num_pages=pages,
                         max_requests=args.max_requests, max_tokens_per_request=per_request,
                         dtype=dtype, device=args.device, max_step_tokens=per_request)
    runner = ModelRunner(model, cache)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            request_id = str(item["id"])
            if request_id not in cache.requests:
                cache.create_request(request_id)
            entries.append(StepEntry(request_id, [int(t) for t in item["tokens"]],
                                     [int(w) for w in item.get("want", [])]))
        if entries:
            logits = runner.step(entries)
            if logits.shape[0] > 0:
                host = logits.to("cpu", torch.float32).contiguous().numpy()
                host.astype("<f4", copy=False).tofile(out_dir / f"{step}.f32")
            else:
                torch.cuda.synchronize()
            runner.check_device()       # the host has just waited for the step: a kernel that gave up shows here
        for request_id in record.get("end", []):
            cache.release(str(request_id))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
