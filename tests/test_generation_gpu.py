"""Generation through the Python entry point on the GPU: greedy tokens equal the plain
implementation's, temperature sampling is the plain sampler's and independent of the batch, and
toy parts defined by the test (a mixer with state, a routed feed-forward, another position
encoding) are registered, built and stepped on the device."""

import pytest
import torch

import plain_qwen2 as plain
import scenarios
from harness import assert_close, random_prompt
from mini_llm_runtime_b200.cache import CacheManager
from mini_llm_runtime_b200.config import register_architecture, unregister_architecture
from mini_llm_runtime_b200.engine import ContinuousBatchEngine, ModelRunner, StepEntry, greedy_generate
from mini_llm_runtime_b200.models import build_model, write_random_model_dir
from mini_llm_runtime_b200.weights import random_tensors, read_checkpoint
from tiny_configs import TINY

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


def greedy_with_margin(tensors, config_dict, prompt, steps):
    """Plain greedy tokens plus, per step, the gap between the best and the second-best logit."""
    sequence, tokens, gaps = list(prompt), [], []
    for _ in range(steps):
        logits = plain.forward_logits(tensors, config_dict, sequence)[-1]
        top = torch.topk(logits, 2).values
        tokens.append(int(torch.argmax(logits)))
        gaps.append(float(top[0] - top[1]))
        sequence.append(tokens[-1])
    return tokens, gaps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_greedy_generation_through_the_entry_point(name, dtype, tmp_path):
    config, page = TINY[name]
    write_random_model_dir(tmp_path, config, seed=31)
    tensors = read_checkpoint(tmp_path)
    engine = ContinuousBatchEngine.from_model_dir(tmp_path, dtype=dtype, device=DEVICE, block_size=page,
                                                  max_running_requests=4, max_batch_tokens=24, max_model_len=128)
    lengths = (5, 17, 33, 1, 50, 9)
    prompts = [random_prompt(config.vocab_size, n, 70 + i) for i, n in enumerate(lengths)]
    for i, prompt in enumerate(prompts):
        engine.submit(f"g{i}", prompt, max_new_tokens=8)
    results = engine.run()
    assert any(len(r.plan.prefill_request_ids) and len(r.plan.decode_request_ids) for r in results)
    for i, prompt in enumerate(prompts):
        want, gaps = greedy_with_margin(tensors, config.to_dict(), prompt, 8)
        got = list(engine.scheduler.get_request(f"g{i}").generated_token_ids)
        # bfloat16 may legitimately flip an argmax whose margin is below its rounding; compare
        # up to the first step whose margin is that small.
        limit = 1e-4 if dtype == "float32" else 2e-2
        sure = next((k for k, gap in enumerate(gaps) if gap < limit), len(gaps))
        assert got[:sure] == want[:sure], (name, dtype, i, got, want, gaps)
        assert len(got) == 8
    stats = engine.manager.stats()
    assert stats.live_requests == 0 and all(h == 0 for h in stats.held_pages)
    single = greedy_generate(engine.runner, prompts[1], max_new_tokens=4, return_step_logits=True)
    assert_close(torch.stack(single.step_logits)[:1],
                 plain.forward_logits(tensors, config.to_dict(), prompts[1])[-1:],
                 torch.float32 if dtype == "float32" else torch.bfloat16, "first step logits")


def test_temperature_sampling_on_the_device_is_the_plain_sampler_and_ignores_the_batch():
    config, page = TINY["B"]
    model = build_model(config, torch.float32)
    tensors = random_tensors(model.expected_tensors(), 33)
    model.load(tensors, DEVICE)
    prompts = [random_prompt(config.vocab_size, n, 80 + n) for n in (1, 9, 24, 40)]

    def run(order, budget):
        engine = ContinuousBatchEngine.from_model(model, block_size=page, max_running_requests=4,
                                                  max_batch_tokens=budget, max_model_len=128)
        for i in order:
            engine.submit(f"t{i}", prompts[i], max_new_tokens=12, temperature=0.7, seed=500 + i)
        engine.run()
        return {i: engine.scheduler.get_request(f"t{i}").generated_token_ids for i in order}

    together = run([0, 1, 2, 3], 64)
    assert together == run([3, 1, 0, 2], 9)
    sequence = list(prompts[2])
    for index, token in enumerate(together[2]):
        logits = plain.forward_logits(tensors, config.to_dict(), sequence)[-1]
        u = plain.uniform_from_seed(502, index)
        expected, cdf = plain.temperature_sample(logits, 0.7, u)
        if token != expected:
            low = float(cdf[token - 1]) if token > 0 else 0.0
            assert low - 1e-5 <= u <= float(cdf[token]) + 1e-5
        sequence.append(token)


@pytest.mark.parametrize("name,dtype,eventful", [("A", torch.float32, True), ("C", torch.float32, True),
                                                 ("D", torch.bfloat16, False), ("E", torch.bfloat16, False)])
def test_stepping_ahead_on_the_device(name, dtype, eventful):
    """The engine that launches the next decode step before it has read the current one's tokens
    (captured graphs, input ids fed from the device) returns, call by call, what the step-by-step
    engine returns.  In float32, where a row's result does not depend on its batch, with everything
    that changes the batches: a sampled request, a stop token in mid-flight, a late arrival.  In
    bfloat16 with requests that decode side by side to the end (there a step taken from the launch
    ahead and the same step launched in another batch may differ in rounding)."""
    config, page = TINY[name]
    model = build_model(config, dtype)
    model.load(random_tensors(model.expected_tensors(), 41), DEVICE)
    prompts = {rid: random_prompt(config.vocab_size, n, 300 + n) for rid, n in (("a", 5), ("b", 33), ("c", 70), ("late", 41))}
    stop_token = None
    if eventful:
        trial = ContinuousBatchEngine.from_model(model, block_size=page, max_running_requests=1, max_batch_tokens=128,
                                                 max_model_len=256)
        trial.submit("trial", prompts["c"], max_new_tokens=8)
        trial.run()
        stop_token = trial.scheduler.get_request("trial").generated_token_ids[5]
    histories = []
    for ahead in (False, True):
        engine = ContinuousBatchEngine.from_model(model, block_size=page, max_running_requests=4, max_batch_tokens=128,
                                                  max_model_len=256, step_ahead=ahead)
        if eventful:
            engine.submit("a", prompts["a"], max_new_tokens=40)
            engine.submit("b", prompts["b"], max_new_tokens=25, temperature=0.7, seed=11)
            engine.submit("c", prompts["c"], max_new_tokens=30, eos_token_ids=[stop_token])
        else:
            for rid in ("a", "b", "c"):
                engine.submit(rid, prompts[rid], max_new_tokens=30)
        history, steps = [], 0
        while engine.scheduler.has_unfinished_requests:
            if eventful and steps == 9:
                engine.submit("late", prompts["late"], max_new_tokens=12)
            result = engine.step()
            steps += 1
            history.append((result.outcome.emitted_tokens, result.outcome.finished_request_ids))
        engine.manager.check_consistency()
        assert not engine.manager.requests
        histories.append((history, engine.runner.graph_replays))
    assert histories[0][0] == histories[1][0]
    assert histories[1][1] > 0, "decode steps must have gone through captured graphs"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_parts_on_the_device(dtype):
    import toy_parts

    toy_parts.register_toys()
    register_architecture("ToyForCausalLM", toy_parts.ToyConfig.from_dict, toy_parts.toy_model_spec, replace=True)
    try:
        config = toy_parts.ToyConfig()
        model = build_model(config, dtype)
        tensors = random_tensors(model.expected_tensors(), 4, torch.bfloat16)
        for name in tensors:
            if "mix.weight" in name:
                tensors[name] = tensors[name] * 20
        model.load(tensors, DEVICE)
        cache = CacheManager(model.cache_needs(), page_size=8, num_pages=16, max_requests=3,
                             max_tokens_per_request=128, dtype=dtype, device=DEVICE)
        runner = ModelRunner(model, cache)
        requests = {"x": random_prompt(97, 45, 1), "y": random_prompt(97, 30, 2), "z": random_prompt(97, 7, 3)}
        pieces = {rid: [] for rid in requests}
        for step in scenarios.mixed(requests, seed=8, max_live=3, decode_tail=5):
            entries = []
            for rid, start, end in step["entries"]:
                if rid not in cache.requests:
                    cache.create_request(rid)
                entries.append(StepEntry(rid, requests[rid][start:end], list(range(end - start))))
            logits = runner.step(entries)
            row = 0
            for rid, start, end in step["entries"]:
                pieces[rid].append(logits[row:row + end - start])
                row += end - start
            for rid in step["end"]:
                cache.release(rid)
        for rid, tokens in requests.items():
            got = torch.cat(pieces[rid]).float().cpu()
            want = toy_parts.plain_toy_logits(tensors, config, tokens)
            if dtype == torch.float32:
                assert_close(got, want, dtype, f"toy {rid}")
            else:
                # The routed feed-forward takes a hard decision per row; bfloat16 rounding may flip
                # a near-tie, which changes that row (and, through the running mean, nudges later
                # ones).  Most rows must still agree to bfloat16 accuracy.
                assert torch.isfinite(got).all()
                rel = (got - want).norm(dim=-1) / want.norm(dim=-1)
                assert float(rel.median()) <= 2e-2 and float((rel <= 4e-2).float().mean()) >= 0.8, rel
    finally:
        unregister_architecture("ToyForCausalLM")


def test_stepping_ahead_with_events_in_bfloat16():
    """bfloat16, ``step_ahead`` on, and everything that changes the batches while steps are in
    flight: a sampled request, a stop token in mid-flight, a late arrival that prefills in portions
    beside the decodes.  A bfloat16 row may round differently in another batch, so the engine is
    not compared with its step-by-step twin but with the plain implementation: greedy requests up
    to the first step whose margin rounding could flip, the sampled request as long as its uniform
    number stays clear of a boundary of the cumulative distribution."""
    config, page = TINY["D"]
    model = build_model(config, torch.bfloat16)
    tensors = random_tensors(model.expected_tensors(), 43)
    model.load(tensors, DEVICE)
    cfg = config.to_dict()
    prompts = {rid: random_prompt(config.vocab_size, n, 900 + n) for rid, n in (("a", 5), ("b", 33), ("c", 70), ("late", 90))}
    want_c, gaps_c = greedy_with_margin(tensors, cfg, prompts["c"], 30)
    sure_c = next((k for k, gap in enumerate(gaps_c) if gap < 2e-2), len(gaps_c))
    assert sure_c >= 4, "the scenario needs a few sure steps to place a stop token in"
    stop_at = min(sure_c - 1, 6)
    stop_token = want_c[stop_at]
    if stop_token in want_c[:stop_at]:
        stop_at = want_c.index(stop_token)
    engine = ContinuousBatchEngine.from_model(model, block_size=page, max_running_requests=4, max_batch_tokens=32,
                                              max_model_len=256, step_ahead=True)
    engine.submit("a", prompts["a"], max_new_tokens=40)
    engine.submit("b", prompts["b"], max_new_tokens=25, temperature=0.7, seed=11)
    engine.submit("c", prompts["c"], max_new_tokens=30, eos_token_ids=[stop_token])
    steps = 0
    while engine.scheduler.has_unfinished_requests:
        if steps == 9:
            engine.submit("late", prompts["late"], max_new_tokens=12)
        engine.step()
        steps += 1
        engine.manager.check_consistency()
    assert not engine.manager.requests and engine.runner.graph_replays > 0
    got = {rid: list(engine.scheduler.get_request(rid).generated_token_ids) for rid in prompts}
    # the stop token ended c where the plain implementation says, and nothing came after it
    assert got["c"] == want_c[:stop_at + 1]
    assert engine.scheduler.get_request("c").finish_reason.value == "eos"
    for rid, count in (("a", 40), ("late", 12)):
        want, gaps = greedy_with_margin(tensors, cfg, prompts[rid], count)
        sure = next((k for k, gap in enumerate(gaps) if gap < 2e-2), len(gaps))
        assert len(got[rid]) == count and got[rid][:sure] == want[:sure], (rid, got[rid], want, gaps)
    # the sampled request: the plain sampler on the plain logits, while u is clear of a boundary
    assert len(got["b"]) == 25
    sequence = list(prompts["b"])
    for index, token in enumerate(got["b"]):
        logits = plain.forward_logits(tensors, cfg, sequence)[-1]
        u = plain.uniform_from_seed(11, index)
        expected, cdf = plain.temperature_sample(logits, 0.7, u)
        low = float(cdf[expected - 1]) if expected > 0 else 0.0
        if min(u - low, float(cdf[expected]) - u) < 2e-2:
            break                                   # too close to call in bfloat16
        assert token == expected, (index, token, expected)
        sequence.append(token)
