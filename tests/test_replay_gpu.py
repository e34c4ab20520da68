"""bin/trace_run driven as a user drives it: a model folder on disk, JSON steps on standard
input, ``done <step>`` awaited before the next step, logits read back from ``<step>.f32``.  The
same requests are replayed whole, with the last 32 tokens one by one, in changing portions and
mixed in a pool so small that pages are used again, in float32 and bfloat16, and every position
is compared with the plain implementation."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import scenarios
from harness import assert_close, random_prompt
from mini_llm_runtime_b200.models import write_random_model_dir
from mini_llm_runtime_b200.weights import read_checkpoint
from tiny_configs import TINY

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
TRACE_RUN = ROOT / "bin" / "trace_run"
LENGTHS = {"A": (5, 17, 33, 140), "B": (1, 9, 24, 40, 99), "C": (3, 70, 45, 97),
           "D": (2, 64, 65, 130, 300), "E": (7, 33, 128, 200)}


def run_trace(model_dir, dtype_name, out_dir, max_tokens, page, requests, steps):
    command = [sys.executable, str(TRACE_RUN), "--model", str(model_dir), "--dtype", dtype_name,
               "--out", str(out_dir), "--max-tokens", str(max_tokens), "--block-size", str(page)]
    process = subprocess.Popen(command, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for index, step in enumerate(steps):
            record = {"step": index,
                      "entries": [{"id": rid, "tokens": requests[rid][start:end], "want": list(range(end - start))}
                                  for rid, start, end in step["entries"]],
                      "end": step["end"]}
            process.stdin.write(json.dumps(record) + "\n")
            process.stdin.flush()
            answer = process.stdout.readline().strip()
            assert answer == f"done {index}", f"trace_run answered {answer!r} to step {index}"
        process.stdin.close()
        assert process.wait(timeout=120) == 0
    finally:
        if process.poll() is None:
            process.kill()


def collect(out_dir, vocab, requests, steps):
    pieces = {rid: [] for rid in requests}
    for index, step in enumerate(steps):
        data = np.fromfile(out_dir / f"{index}.f32", dtype="<f4").reshape(-1, vocab)
        row = 0
        for rid, start, end in step["entries"]:
            pieces[rid].append(torch.from_numpy(data[row:row + end - start].copy()))
            row += end - start
        assert row == data.shape[0]
    return {rid: torch.cat(parts) for rid, parts in pieces.items()}


@pytest.fixture(scope="module", params=list(TINY))
def folder(request, tmp_path_factory):
    name = request.param
    config, page = TINY[name]
    path = tmp_path_factory.mktemp(f"model_{name}")
    write_random_model_dir(path, config, seed=11)
    tensors = read_checkpoint(path)
    requests = {f"{name}{i}": random_prompt(config.vocab_size, length, 200 + i)
                for i, length in enumerate(LENGTHS[name])}
    with open(path / "config.json") as handle:
        config_dict = json.load(handle)
    want = {rid: plain.forward_logits(tensors, config_dict, tokens) for rid, tokens in requests.items()}
    return name, path, config, page, requests, want


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_replay(folder, tmp_path, dtype_name, cut):
    name, path, config, page, requests, want = folder
    steps = {"whole": scenarios.whole, "tail": scenarios.tail_one_by_one,
             "portions": scenarios.changing_portions,
             "mixed": lambda r: scenarios.mixed(r, seed=5)}[cut](requests)
    max_tokens = scenarios.pool_tokens(requests, steps)
    run_trace(path, dtype_name, tmp_path, max_tokens, page, requests, steps)
    got = collect(tmp_path, config.vocab_size, requests, steps)
    dtype = torch.float32 if dtype_name == "float32" else torch.bfloat16
    for rid in requests:
        assert_close(got[rid], want[rid], dtype, f"{name} {cut} {dtype_name} request {rid}")


def test_replay_writes_nothing_for_a_step_that_wants_nothing(folder, tmp_path):
    name, path, config, page, requests, want = folder
    rid = next(iter(requests))
    tokens = requests[rid]
    command = [sys.executable, str(TRACE_RUN), "--model", str(path), "--dtype", "float32", "--out", str(tmp_path),
               "--max-tokens", "256", "--block-size", str(page)]
    half = max(1, len(tokens) // 2)
    lines = [json.dumps({"step": 0, "entries": [{"id": rid, "tokens": tokens[:half], "want": []}], "end": []})]
    if half < len(tokens):
        lines.append(json.dumps({"step": 1, "entries": [{"id": rid, "tokens": tokens[half:], "want": [len(tokens) - half - 1]}], "end": [rid]}))
    done = subprocess.run(command, input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr
    assert done.stdout.split() == sum((["done", str(i)] for i in range(len(lines))), [])
    assert not (tmp_path / "0.f32").exists()
    if half < len(tokens):
        last = np.fromfile(tmp_path / "1.f32", dtype="<f4").reshape(-1, config.vocab_size)
        assert_close(torch.from_numpy(last), want[rid][-1:], torch.float32, "last position after an unobserved step")
