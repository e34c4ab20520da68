"""Everything above the kernels on the CPU, with the kernels replaced by their plain stand-ins
(``fake_ops.FakeOps``): the step function under several cuts, the engine loop with greedy and
temperature sampling, failure roll-back, and toy parts registered from outside the package."""

import pytest
import torch

import plain_qwen2 as plain
import scenarios
from fake_ops import FakeOps
from harness import TinyEngine, assert_close, random_prompt
from mini_llm_runtime_b200 import ops
from mini_llm_runtime_b200.cache import CacheManager
from mini_llm_runtime_b200.config import register_architecture, unregister_architecture
from mini_llm_runtime_b200.engine import (ContinuousBatchEngine, ModelRunner, StepEntry, greedy_generate)
from mini_llm_runtime_b200.models import build_model, random_model
from mini_llm_runtime_b200.weights import random_tensors
from tiny_configs import TINY


@pytest.fixture(autouse=True)
def stand_in_kernels():
    with ops.use(FakeOps()):
        yield


def test_the_package_never_computes_on_the_cpu_by_itself():
    config, page = TINY["A"]
    with ops.use(ops.CudaOps()):
        engine = TinyEngine(config, page, torch.float32, "cpu")
        with pytest.raises(ops.KernelError):
            engine.run_whole("a", [1, 2, 3])
        assert engine.cache.get("a").committed == 0 and not engine.cache.step_in_flight


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", list(TINY))
def test_step_function_under_mixed_cuts(name, dtype):
    """In bfloat16 the blocks fold their norms into the projections; the stand-in kernels claim the
    fused arrangement for steps of up to 16 rows, so both arrangements meet in one sequence."""
    config, page = TINY[name]
    engine = TinyEngine(config, page, dtype, "cpu", num_pages=24)
    assert all(block.folded == (dtype == torch.bfloat16) for block in engine.model.blocks)
    requests = {f"r{i}": random_prompt(config.vocab_size, n, i) for i, n in enumerate((3, 41, 18, 57, 9))}
    steps = scenarios.mixed(requests, seed=3)
    pieces = {rid: [] for rid in requests}
    for step in steps:
        entries = []
        for rid, start, end in step["entries"]:
            if rid not in engine.cache.requests:
                engine.cache.create_request(rid)
            entries.append(StepEntry(rid, requests[rid][start:end], list(range(end - start))))
        logits = engine.runner.step(entries)
        row = 0
        for rid, start, end in step["entries"]:
            pieces[rid].append(logits[row:row + end - start])
            row += end - start
        for rid in step["end"]:
            engine.cache.release(rid)
        engine.cache.check_consistency()
    for rid, tokens in requests.items():
        assert_close(torch.cat(pieces[rid]), engine.plain_logits(tokens), dtype, rid)


def test_step_validation():
    config, page = TINY["A"]
    engine = TinyEngine(config, page, torch.float32, "cpu", max_tokens=32)
    engine.cache.create_request("a")
    for bad in ([StepEntry("a", [], [])], [StepEntry("a", [config.vocab_size], [0])], [StepEntry("a", [-1], [0])],
                [StepEntry("a", [1, 2], [2])], [StepEntry("a", [1.5], [0])], []):
        with pytest.raises(ValueError):
            engine.runner.step(bad)
    with pytest.raises(KeyError):
        engine.runner.step([StepEntry("nobody", [1], [0])])
    assert engine.runner.step([StepEntry("a", [1, 2, 3], [])]).shape == (0, config.vocab_size)
    assert engine.cache.get("a").committed == 3


def test_attention_work_lists_of_one_portion_equal_the_general_construction():
    """A step of one prompt portion takes a short way to its attention work lists; they are the
    lists the general construction (cut every segment into tiles, heaviest first) gives."""
    import numpy as np

    from mini_llm_runtime_b200.ops import cuda_ops

    def general(count, start):
        lengths, starts = np.array([count], dtype=np.int32), np.array([start], dtype=np.int32)
        segments = np.array([0], dtype=np.int32)
        lists = {}
        for prefix, rows, order in (("tile", cuda_ops.GENERIC_TILE_ROWS, None), ("wide_tile", cuda_ops.MMA_TILE_ROWS, starts),
                                    ("big_tile", cuda_ops.TCGEN05_TILE_ROWS, starts)):
            lists[prefix + "_seg"], lists[prefix + "_row0"] = cuda_ops._tiles(lengths, segments, rows, order)
        return lists

    for count in (2, 3, 15, 16, 17, 63, 64, 65, 127, 128, 129, 777, 2048, 2049):
        for start in (0, 5, 1000):
            arrays, counts = cuda_ops.plan_attention([count], [start])
            for name, want in general(count, start).items():
                assert arrays[name].dtype == want.dtype and np.array_equal(arrays[name], want), (count, start, name)
                assert all(stride > 0 for stride in arrays[name].strides), "a tensor cannot be made from it"
            assert arrays["decode_seg"].shape == (0,) and counts["decode"] == 0
            assert (counts["tiles"], counts["wide"], counts["big"]) == tuple(
                len(arrays[name]) for name in ("tile_seg", "wide_tile_seg", "big_tile_seg"))


def test_a_captured_steps_context_limit_is_the_first_that_no_request_exceeds():
    """The limit a captured decode step plans its kernels against: the first of the runner's limits
    that holds every request's length after the step, limits at or beyond the cache's capacity per
    request do not count, and beyond the last one the capacity itself."""
    config, page = TINY["A"]
    engine = TinyEngine(config, page, torch.float32, "cpu", num_pages=64, max_requests=2, max_tokens=40 * page)
    runner, cache = engine.runner, engine.cache
    capacity = cache.max_pages_per_request * page
    runner.CONTEXT_LIMITS = (2 * page, 5 * page, 10 * capacity)
    cache.create_request("a")
    cache.create_request("b")
    runner.step([StepEntry("a", [1] * (2 * page - 1), []), StepEntry("b", [2, 3], [])])

    def limit_after(tokens_a, tokens_b):
        requests = cache.begin_step([("a", tokens_a), ("b", tokens_b)])
        try:
            return runner._context_limit(requests)
        finally:
            cache.abort_step()

    assert limit_after(1, 1) == 2 * page                    # a reaches exactly the first limit
    assert limit_after(2, 1) == 5 * page                    # one token more: the next
    assert limit_after(3 * page + 1, 1) == 5 * page
    assert limit_after(3 * page + 2, 1) == capacity         # beyond the last limit below the capacity
    assert limit_after(1, 5 * page) == capacity             # the longest request decides


def build_engine(name, **options):
    config, page = TINY[name]
    model = build_model(config, torch.float32)
    tensors = random_tensors(model.expected_tensors(), 21)
    model.load(tensors, "cpu")
    defaults = dict(block_size=page, max_running_requests=4, max_batch_tokens=24, max_model_len=128)
    defaults.update(options)
    return config, tensors, ContinuousBatchEngine.from_model(model, **defaults)


@pytest.mark.parametrize("name", list(TINY))
def test_continuous_batching_reproduces_plain_greedy_generation(name):
    config, tensors, engine = build_engine(name)
    prompts = {f"p{i}": random_prompt(config.vocab_size, n, 40 + i) for i, n in enumerate((5, 17, 33, 1, 50, 9))}
    for i, (rid, prompt) in enumerate(prompts.items()):
        engine.submit(rid, prompt, max_new_tokens=3 + i % 4)
    results = engine.run()
    assert any(len(r.plan.prefill_request_ids) and len(r.plan.decode_request_ids) for r in results)
    assert any(not item.emits for r in results for item in r.plan.items)     # some prompt was cut
    for i, (rid, prompt) in enumerate(prompts.items()):
        want = plain.greedy_tokens(tensors, config.to_dict(), prompt, 3 + i % 4)
        assert list(engine.scheduler.get_request(rid).generated_token_ids) == want, rid
    stats = engine.manager.stats()
    assert stats.live_requests == 0 and all(h == 0 for h in stats.held_pages) and all(p == 0 for p in stats.promised_pages)
    assert engine.metrics.summary()["tokens"] == sum(3 + i % 4 for i in range(6))


def test_eos_stops_a_request_and_frees_its_pages():
    config, tensors, engine = build_engine("A")
    prompt = random_prompt(config.vocab_size, 12, 5)
    want = plain.greedy_tokens(tensors, config.to_dict(), prompt, 6)
    engine.submit("e", prompt, max_new_tokens=6, eos_token_ids=[want[2]])
    engine.run()
    stop = want.index(want[2])
    assert list(engine.scheduler.get_request("e").generated_token_ids) == want[:stop + 1]
    assert engine.manager.stats().live_requests == 0


def test_temperature_sampling_does_not_depend_on_the_batch():
    config, tensors, _ = build_engine("B")
    prompts = [random_prompt(config.vocab_size, n, 60 + n) for n in (1, 9, 24, 40)]

    def run(order, budget):
        _, _, engine = build_engine("B", max_batch_tokens=budget)
        for i in order:
            engine.submit(f"t{i}", prompts[i], max_new_tokens=12, temperature=0.7, seed=1000 + i)
        engine.run()
        return {i: engine.scheduler.get_request(f"t{i}").generated_token_ids for i in order}

    together = run([0, 1, 2, 3], 64)
    assert together == run([3, 2, 1, 0], 7)
    assert {2: together[2]} == run([2], 64)
    # and the tokens are the plain sampler's, fed with the plain model's logits
    sequence = list(prompts[1])
    for index, token in enumerate(together[1]):
        logits = plain.forward_logits(tensors, config.to_dict(), sequence)[-1]
        u = plain.uniform_from_seed(1001, index)
        assert token == plain.temperature_sample(logits, 0.7, u)[0]
        sequence.append(token)
    assert len(set(together[1])) > 1


def test_a_failed_step_rolls_back_scheduler_and_cache_and_can_be_retried():
    config, tensors, engine = build_engine("A")
    engine.submit("a", random_prompt(config.vocab_size, 6, 1), max_new_tokens=3)
    engine.step()
    engine.submit("b", random_prompt(config.vocab_size, 4, 2), max_new_tokens=2)
    forward = engine.runner.model.forward
    calls = {"n": 0}

    def failing(ctx):
        calls["n"] += 1
        raise RuntimeError("injected failure between layers")

    engine.runner.model.forward = failing
    with pytest.raises(RuntimeError, match="injected"):
        engine.step()
    engine.runner.model.forward = forward
    assert calls["n"] == 1
    assert engine.scheduler.waiting_request_ids == ("b",) and engine.scheduler.running_request_ids == ("a",)
    assert "b" not in engine.manager.requests and engine.manager.get("a").committed == 6
    assert not engine.manager.step_in_flight
    engine.manager.check_consistency()
    result = engine.step()
    assert result.plan.index == 1 and set(result.plan.admitted_request_ids) == {"b"}
    engine.run()
    for rid, seed, length, count in (("a", 1, 6, 3), ("b", 2, 4, 2)):
        want = plain.greedy_tokens(tensors, config.to_dict(), random_prompt(config.vocab_size, length, seed), count)
        assert list(engine.scheduler.get_request(rid).generated_token_ids) == want


def test_greedy_generate_and_generate_entry_points():
    config, tensors, engine = build_engine("B")
    prompt = random_prompt(config.vocab_size, 24, 9)
    want = plain.greedy_tokens(tensors, config.to_dict(), prompt, 5)
    output = greedy_generate(engine.runner, prompt, max_new_tokens=5, return_step_logits=True)
    assert output.generated_token_ids == want and output.decode_steps == 4
    assert output.cache_length == len(prompt) + 4 and len(output.step_logits) == 5
    assert engine.manager.stats().live_requests == 0
    assert engine.generate([prompt, prompt[:3]], max_new_tokens=5)[0] == want
    with pytest.raises(ValueError):
        engine.submit("bad", [config.vocab_size], max_new_tokens=1)
    with pytest.raises(ValueError):
        engine.submit("long", [1] * 120, max_new_tokens=20)


def test_toy_parts_register_build_and_step_without_touching_the_package():
    import toy_parts

    toy_parts.register_toys()
    register_architecture("ToyForCausalLM", toy_parts.ToyConfig.from_dict, toy_parts.toy_model_spec, replace=True)
    try:
        config = toy_parts.ToyConfig()
        model = build_model(config, torch.float32)
        tensors = random_tensors(model.expected_tensors(), 4, torch.float32)
        for name in tensors:                      # larger weights so that routing and mixing matter
            if "router" in name or "mix.weight" in name:
                tensors[name] = tensors[name] * 20
        model.load(tensors, "cpu")
        needs = model.cache_needs()
        assert len(needs) == 3 and type(needs[1]).__name__ == "StateNeed"
        cache = CacheManager(needs, page_size=8, num_pages=16, max_requests=3, max_tokens_per_request=128,
                             dtype=torch.float32, device="cpu")
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
            assert_close(torch.cat(pieces[rid]), toy_parts.plain_toy_logits(tensors, config, tokens),
                         torch.float32, f"toy {rid}")
    finally:
        unregister_architecture("ToyForCausalLM")


def test_stepping_ahead_returns_the_same_results_step_by_step():
    """With ``step_ahead`` the next decode step is launched before the host has the tokens of the
    current one (fed on the device).  Every step() must return what it returns without it: tokens,
    finished requests, step after step - with a request that samples, one that stops on a stop
    token in mid-flight, one that reaches its token limit, and one submitted while others decode."""
    config, page = TINY["B"]
    histories = []
    for ahead in (False, True):
        with ops.use(FakeOps()):
            model = random_model(config, seed=3, dtype=torch.float32, device="cpu")
            engine = ContinuousBatchEngine.from_model(model, block_size=page, max_running_requests=4,
                                                      max_batch_tokens=48, step_ahead=ahead)
            engine.submit("a", [1, 2, 3, 4, 5], max_new_tokens=14)
            engine.submit("b", [9, 8, 7], max_new_tokens=9, temperature=0.8, seed=5)
            # a request that stops on the fourth token it generates (found with a trial run)
            trial = ContinuousBatchEngine.from_model(model, block_size=page, max_running_requests=1, max_batch_tokens=48)
            trial.submit("trial", [4, 4, 4, 4], max_new_tokens=6)
            trial.run()
            stop_token = trial.scheduler.get_request("trial").generated_token_ids[3]
            engine.submit("stops", [4, 4, 4, 4], max_new_tokens=12, eos_token_ids=[stop_token])
            history, steps = [], 0
            while engine.scheduler.has_unfinished_requests:
                if steps == 5:
                    engine.submit("late", list(range(20, 75)), max_new_tokens=4)
                result = engine.step()
                steps += 1
                history.append((result.outcome.emitted_tokens, result.outcome.finished_request_ids))
                engine.manager.check_consistency()
            assert not engine.manager.requests, "every finished request gave its pages back"
            tokens = {rid: engine.scheduler.get_request(rid).generated_token_ids for rid in ("a", "b", "stops", "late")}
            histories.append((history, tokens, engine.runner.steps_run))
    assert histories[0][0] == histories[1][0]
    assert histories[0][1] == histories[1][1]
    assert len(histories[1][1]["stops"]) < 12, "the stop token must have ended the request early"
    assert histories[1][2] > histories[0][2], "stepping ahead launches the dropped extra step of ended requests"


def test_a_device_error_ends_the_steps_requests_and_leaves_the_engine_usable():
    """A kernel whose bounded wait ran out reports through an error word that the engine reads where
    it waits for the step's tokens.  The requests of that step end with an error and give their
    pages back; a request that was still waiting runs afterwards and gets the right tokens."""
    from mini_llm_runtime_b200.engine import FinishReason

    config, tensors, engine = build_engine("A", max_running_requests=2)
    kernels = ops.current()
    prompts = {rid: random_prompt(config.vocab_size, n, seed) for rid, n, seed in (("a", 6, 1), ("b", 9, 2), ("c", 5, 3))}
    for rid, prompt in prompts.items():
        engine.submit(rid, prompt, max_new_tokens=4)
    engine.step()                                   # a and b prefill; c waits for a place
    kernels.error_code = 3
    with pytest.raises(ops.KernelError, match="bounded wait"):
        engine.step()
    for rid in ("a", "b"):
        request = engine.scheduler.get_request(rid)
        assert request.finish_reason is FinishReason.ERROR and len(request.generated_token_ids) == 1
    assert not engine.manager.requests and engine.scheduler.outstanding_plan is None
    engine.manager.check_consistency()
    assert engine.scheduler.waiting_request_ids == ("c",)
    engine.run()
    assert list(engine.scheduler.get_request("c").generated_token_ids) == \
        plain.greedy_tokens(tensors, config.to_dict(), prompts["c"], 4)
    # the single-request loop checks after each step too
    kernels.error_code = 5
    with pytest.raises(ops.KernelError):
        greedy_generate(engine.runner, prompts["a"], max_new_tokens=2)
    assert not engine.manager.requests


def test_slot_records_follow_the_requests():
    """What the device keeps per slot (length, last token, counter) after every step equals what the
    host knows of the request, through prompt portions, decodes fed from the records and slot reuse."""
    from mini_llm_runtime_b200.cache import read_record

    config, tensors, engine = build_engine("B", max_running_requests=2, max_batch_tokens=12)
    for i, n in enumerate((20, 3, 7)):
        engine.submit(f"r{i}", random_prompt(config.vocab_size, n, 80 + i), max_new_tokens=4 + i,
                      temperature=0.5 * i, seed=11 * i)
    while engine.scheduler.has_unfinished_requests:
        engine.step()
        for rid in engine.scheduler.running_request_ids:
            request, held = engine.scheduler.get_request(rid), engine.manager.get(rid)
            record = read_record(engine.manager.slot_state[held.slot].numpy())
            assert record["length"] == held.committed
            assert record["counter"] == len(request.generated_token_ids)
            assert record["temperature"] == request.temperature and record["seed"] == request.seed
            if request.generated_token_ids:
                assert record["last_token"] == request.generated_token_ids[-1]


def test_a_step_that_fails_after_a_stateful_mixer_ran_leaves_its_state_as_it_was():
    """The toy mixer overwrites its per-request state in place.  A failure later in the same step
    must not leave the half-advanced state behind: the retried step gives the logits of a run that
    never failed."""
    import toy_parts

    toy_parts.register_toys()
    register_architecture("ToyForCausalLM", toy_parts.ToyConfig.from_dict, toy_parts.toy_model_spec, replace=True)
    try:
        config = toy_parts.ToyConfig()
        model = build_model(config, torch.float32)
        tensors = random_tensors(model.expected_tensors(), 4, torch.float32)
        model.load(tensors, "cpu")
        cache = CacheManager(model.cache_needs(), page_size=8, num_pages=16, max_requests=2,
                             max_tokens_per_request=64, dtype=torch.float32, device="cpu")
        runner = ModelRunner(model, cache)
        tokens = random_prompt(97, 20, 6)
        cache.create_request("x")
        first = runner.step([StepEntry("x", tokens[:9], list(range(9)))])
        last_block = model.blocks[2]
        forward = last_block.forward

        def failing(*args, **kwargs):
            raise RuntimeError("injected failure after the stateful layers ran")

        last_block.forward = failing
        with pytest.raises(RuntimeError, match="injected"):
            runner.step([StepEntry("x", tokens[9:], list(range(11)))])
        last_block.forward = forward
        assert cache.get("x").committed == 9 and not cache.step_in_flight
        second = runner.step([StepEntry("x", tokens[9:], list(range(11)))])
        assert_close(torch.cat([first, second]), toy_parts.plain_toy_logits(tensors, config, tokens),
                     torch.float32, "toy after a failed step")
    finally:
        unregister_architecture("ToyForCausalLM")


def test_a_block_arrangement_with_further_parts_is_registered_from_outside():
    """A "sandwich" arrangement defined here: a norm after the mixer and after the feed-forward as
    well as before them.  The two further norms are named in the layer's spec, built by the model
    like any other part, checked by the loader by their tensor names, and found by the block."""
    from mini_llm_runtime_b200.config import LayerSpec, ModelSpec, PartSpec, RunStep
    from mini_llm_runtime_b200.parts import register_part
    from mini_llm_runtime_b200.parts.base import Block, unregister_part

    class Sandwich(Block):
        def forward(self, residual, pending, ctx, view, writes_cache):
            kernels = ops.current()
            if pending is not None:
                residual = kernels.add_inplace(residual, pending)
            mixed = self.mixer.forward(self.mixer_norm.forward(residual), ctx, view, writes_cache)
            residual = kernels.add_inplace(residual, self.extras["after_mixer"].forward(mixed))
            fed = self.feed_forward.forward(self.feed_forward_norm.forward(residual), ctx)
            return residual, self.extras["after_feed_forward"].forward(fed)

    register_part("block", "toy_sandwich", Sandwich, replace=True)
    try:
        h, vocab = 48, 61
        norm = {"size": h, "eps": 1e-5}
        attention = PartSpec("gqa_attention", {"hidden_size": h, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16,
                                               "qkv_bias": True, "out_bias": False, "window": None,
                                               "position": PartSpec("rope_half", {"head_dim": 16, "theta": 1e4})},
                             "model.layers.0.self_attn.")
        layer = LayerSpec("toy_sandwich", attention,
                          PartSpec("swiglu", {"hidden_size": h, "intermediate_size": 80}, "model.layers.0.mlp."),
                          PartSpec("rms_norm", norm, "model.layers.0.input_layernorm."),
                          PartSpec("rms_norm", norm, "model.layers.0.post_attention_layernorm."),
                          extra_parts=(("after_mixer", "norm", PartSpec("rms_norm", norm, "model.layers.0.after_mixer.")),
                                       ("after_feed_forward", "norm", PartSpec("rms_norm", norm, "model.layers.0.after_ffn."))))
        sizes = {"vocab_size": vocab, "hidden_size": h}
        spec = ModelSpec("ToySandwich", vocab, h, 128, PartSpec("token_embedding", sizes, "model.embed_tokens."),
                         (layer,), (RunStep(0, 0),), PartSpec("rms_norm", norm, "model.norm."),
                         PartSpec("tied_head", {**sizes, "tied_to": "model.embed_tokens.weight"}, "lm_head."))
        from mini_llm_runtime_b200.models import DecoderModel
        model = DecoderModel(spec, torch.float32)
        assert "model.layers.0.after_mixer.weight" in model.expected_tensors()
        tensors = random_tensors(model.expected_tensors(), 8, torch.float32)
        model.load(tensors, "cpu")
        cache = CacheManager(model.cache_needs(), page_size=8, num_pages=8, max_requests=2, max_tokens_per_request=64,
                             dtype=torch.float32, device="cpu")
        runner = ModelRunner(model, cache)
        tokens = random_prompt(vocab, 23, 4)
        cache.create_request("s")
        got = torch.cat([runner.step([StepEntry("s", tokens[:10], list(range(10)))]),
                         runner.step([StepEntry("s", tokens[10:], list(range(13)))])])
        # the same, plainly
        cfg = {"num_attention_heads": 3, "num_key_value_heads": 1, "hidden_size": h, "head_dim": 16, "rope_theta": 1e4}
        t = {k: v.float() for k, v in tensors.items()}
        x = t["model.embed_tokens.weight"][torch.tensor(tokens)]
        p = "model.layers.0"
        mixed = plain.attention_block(plain.rms_norm(x, t[p + ".input_layernorm.weight"], 1e-5), torch.arange(23), t, p, cfg)
        x = x + plain.rms_norm(mixed, t[p + ".after_mixer.weight"], 1e-5)
        fed = plain.swiglu_mlp(plain.rms_norm(x, t[p + ".post_attention_layernorm.weight"], 1e-5), t, p)
        x = x + plain.rms_norm(fed, t[p + ".after_ffn.weight"], 1e-5)
        want = plain.rms_norm(x, t["model.norm.weight"], 1e-5) @ t["model.embed_tokens.weight"].T
        assert_close(got, want, torch.float32, "sandwich block")
    finally:
        unregister_part("block", "toy_sandwich")
