"""The command line as a user runs it: subprocesses of ``python -m mini_llm_runtime_b200``.
``make-random`` writes a model folder, ``generate`` must produce the plain implementation's greedy
tokens from it, ``serve-batch`` must report the same tokens for each request of its burst, whatever
else runs beside it.  The reference's runner script checks its own output in the same spirit
(experiments/continuous_batch_engine_runner.py:102-150 there)."""

import json
import os
import subprocess
import sys

import pytest

import plain_qwen2 as plain
from mini_llm_runtime_b200.weights import read_checkpoint
from tiny_configs import TINY

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_cli(*arguments, expect=0):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    done = subprocess.run([sys.executable, "-m", "mini_llm_runtime_b200", *arguments], capture_output=True,
                          text=True, env=env, timeout=600)
    assert done.returncode == expect, done.stderr[-2000:]
    return done.stdout


def test_make_random_generate_and_serve_batch(tmp_path):
    config, page = TINY["A"]
    (tmp_path / "config.json").write_text(json.dumps(config.to_dict()))
    model_dir = tmp_path / "model"
    out = run_cli("make-random", "--config", str(tmp_path / "config.json"), "--seed", "12", "--out", str(model_dir))
    assert "wrote" in out and (model_dir / "model.safetensors").is_file() and (model_dir / "config.json").is_file()
    tensors = read_checkpoint(model_dir)
    prompt = [5, 17, 3, 200, 41, 9, 9, 120]
    want = plain.greedy_tokens(tensors, config.to_dict(), prompt, 6)

    common = ["--model", str(model_dir), "--dtype", "float32", "--block-size", str(page), "--max-model-len", "128"]
    record = json.loads(run_cli("generate", *common, "--prompt-ids", ",".join(map(str, prompt)),
                                "--max-new-tokens", "6", "--output-dir", str(tmp_path / "gen")).splitlines()[-1])
    assert record["generated_ids"] == want and record["finish_reason"] == "max_tokens"
    assert json.loads((tmp_path / "gen" / "result.json").read_text())["generated_ids"] == want

    # a stop token ends generation early, and says so
    record = json.loads(run_cli("generate", *common, "--prompt-ids", ",".join(map(str, prompt)),
                                "--max-new-tokens", "6", "--eos-id", str(want[2])).splitlines()[-1])
    assert record["generated_ids"] == want[:want.index(want[2]) + 1] and record["finish_reason"] == "eos"

    record = json.loads(run_cli("serve-batch", *common, "--request-count", "5", "--prompt-ids",
                                ",".join(map(str, prompt)), "--generation-lengths", "2,6,3", "--max-running-requests", "2",
                                "--max-batch-tokens", "8", "--step-ahead").splitlines()[-1])
    run = record["runs"][0]
    assert run["generated_tokens"] == 2 + 6 + 3 + 2 + 6
    for index, (rid, tokens) in enumerate(sorted(run["outputs"].items())):
        assert tokens == want[:(2, 6, 3)[index % 3]], rid
    assert record["cache"]["live_requests"] == 0 and record["metrics"]["tokens"] == run["generated_tokens"]


def test_the_command_line_refuses_what_it_cannot_run(tmp_path):
    assert "config.json" in subprocess.run(
        [sys.executable, "-m", "mini_llm_runtime_b200", "generate", "--model", str(tmp_path), "--prompt-ids", "1"],
        capture_output=True, text=True, env=dict(os.environ, PYTHONPATH=ROOT), timeout=600).stderr
