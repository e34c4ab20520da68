"""The engine against the plain implementation, in float32 and bfloat16, for the tiny
configurations: each request alone and whole; most of it in one step and the last 32 tokens one by
one; in portions of changing size down to two tokens; mixed with other requests in a pool so small
that pages are used again; long decoding; the first tokens of a sequence.  Every position's logits
are compared with the plain implementation run on that request alone and whole."""

from __future__ import annotations

import pytest
import torch

import scenarios
from harness import TinyEngine, assert_close, random_prompt
from mini_llm_runtime_b200.engine import StepEntry
from tiny_configs import TINY

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
LENGTHS = {"A": (5, 17, 33, 150), "B": (1, 9, 24, 40, 131), "C": (3, 70, 45, 97, 160),
           "D": (2, 64, 65, 130, 300), "E": (7, 33, 128, 200)}


def make_requests(name, vocab):
    return {f"{name}{i}": random_prompt(vocab, length, 100 + i) for i, length in enumerate(LENGTHS[name])}


def replay(engine: TinyEngine, requests, steps):
    """Run ``steps`` through the runner; returns request id -> logits of all its positions."""
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
    return {rid: torch.cat(parts) for rid, parts in pieces.items()}


def check_all(engine, requests, results, dtype, what):
    for rid, tokens in requests.items():
        assert results[rid].shape[0] == len(tokens)
        assert_close(results[rid], engine.plain_logits(tokens), dtype, f"{what}, request {rid}")


@pytest.fixture(scope="module", params=[(n, d) for n in TINY for d in DTYPES],
                ids=lambda p: f"{p[0]}-{'f32' if p[1] == torch.float32 else 'bf16'}")
def setup(request):
    name, dtype = request.param
    config, page = TINY[name]
    engine = TinyEngine(config, page, dtype, DEVICE, num_pages=64, max_requests=4, max_tokens=512, seed=7)
    return name, dtype, engine, make_requests(name, config.vocab_size)


def test_whole(setup):
    name, dtype, engine, requests = setup
    check_all(engine, requests, replay(engine, requests, scenarios.whole(requests)), dtype, "whole")


def test_tail_one_by_one(setup):
    name, dtype, engine, requests = setup
    check_all(engine, requests, replay(engine, requests, scenarios.tail_one_by_one(requests)), dtype,
              "last 32 one by one")


def test_changing_portions(setup):
    name, dtype, engine, requests = setup
    check_all(engine, requests, replay(engine, requests, scenarios.changing_portions(requests)), dtype,
              "changing portions")


@pytest.mark.parametrize("seed", [1, 2])
def test_mixed_with_reused_pages(setup, seed):
    name, dtype, engine, requests = setup
    config, page = TINY[name]
    steps = scenarios.mixed(requests, seed)
    tokens = scenarios.pool_tokens(requests, steps)
    tight = TinyEngine(config, page, dtype, DEVICE, num_pages=-(-tokens // page), max_requests=4,
                       max_tokens=512, tensors=engine.tensors)
    handed_out = set()
    reused = False
    original_allocate = [g.allocator.allocate for g in tight.cache.groups]

    def watch(group_index):
        def allocate(count, **options):
            nonlocal reused
            ids = original_allocate[group_index](count, **options)
            reused = reused or any((group_index, i) in handed_out for i in ids)
            handed_out.update((group_index, i) for i in ids)
            return ids
        return allocate

    for index, group in enumerate(tight.cache.groups):
        group.allocator.allocate = watch(index)
    results = replay(tight, requests, steps)
    assert reused, "the scenario must hand out some page a second time"
    assert all(g.allocator.held_count == 0 for g in tight.cache.groups)
    check_all(tight, requests, results, dtype, f"mixed seed {seed}")


def test_long_decoding(setup):
    name, dtype, engine, requests = setup
    config, page = TINY[name]
    tokens = random_prompt(config.vocab_size, 300, 55)
    steps = [{"entries": [("long", 0, 4)], "end": []}]
    steps += [{"entries": [("long", p, p + 1)], "end": ["long"] if p == 299 else []} for p in range(4, 300)]
    results = replay(engine, {"long": tokens}, steps)
    assert_close(results["long"], engine.plain_logits(tokens), dtype, "long decoding")


def test_first_tokens(setup):
    name, dtype, engine, requests = setup
    config, page = TINY[name]
    for length in (1, 2, 3):
        tokens = random_prompt(config.vocab_size, length, 60 + length)
        got = engine.run_whole(f"first{length}", tokens)
        engine.cache.release(f"first{length}")
        assert_close(got, engine.plain_logits(tokens), dtype, f"first tokens, length {length}")
        one_by_one = engine.run_cuts(f"single{length}", tokens, list(range(1, length)))
        engine.cache.release(f"single{length}")
        assert_close(one_by_one, engine.plain_logits(tokens), dtype, f"first tokens one by one, length {length}")


def test_failed_step_leaves_no_trace(setup):
    """Out of pages: the step raises, nothing is held, and the same step succeeds once pages are free."""
    name, dtype, engine, requests = setup
    config, page = TINY[name]
    from mini_llm_runtime_b200.cache import OutOfPages
    small = TinyEngine(config, page, dtype, DEVICE, num_pages=3, max_requests=4, max_tokens=512,
                       tensors=engine.tensors)
    tokens = random_prompt(config.vocab_size, 3 * page, 70)
    small.cache.create_request("x")
    small.cache.create_request("y")
    first = small.runner.step([StepEntry("x", tokens[:2 * page], [2 * page - 1])])
    with pytest.raises(OutOfPages):
        small.runner.step([StepEntry("x", tokens[2 * page:], [0]), StepEntry("y", tokens[:page + 1], [page])])
    small.cache.check_consistency()
    assert small.cache.get("x").committed == 2 * page and small.cache.get("y").committed == 0
    rest = small.runner.step([StepEntry("x", tokens[2 * page:], list(range(page)))])
    want = small.plain_logits(tokens)
    assert_close(first, want[2 * page - 1:2 * page], dtype, "before the failed step")
    assert_close(rest, want[2 * page:], dtype, "after the failed step")


def test_decode_steps_replay_a_captured_graph(setup):
    """Decode-only steps of one batch size run through a CUDA graph after the first; the logits
    must not change because of it, whatever the requests' lengths and slots."""
    name, dtype, engine, requests = setup
    config, page = TINY[name]
    fresh = TinyEngine(config, page, dtype, DEVICE, num_pages=64, max_requests=4, max_tokens=256,
                       tensors=engine.tensors)
    assert fresh.runner.use_graphs
    prompts = {rid: random_prompt(config.vocab_size, n, 90 + n) for rid, n in (("u", 40), ("v", 27), ("w", 23))}
    steps = [{"entries": [(rid, 0, len(t) - 20) for rid, t in prompts.items()], "end": []}]
    for k in range(20):
        order = ["u", "v", "w"] if k % 2 == 0 else ["w", "u", "v"]
        steps.append({"entries": [(rid, len(prompts[rid]) - 20 + k, len(prompts[rid]) - 19 + k) for rid in order],
                      "end": list(prompts) if k == 19 else []})
    results = replay(fresh, prompts, steps)
    assert fresh.runner.graph_replays >= 18
    check_all(fresh, prompts, results, dtype, "graph replay")


def test_a_batch_size_is_captured_only_once_it_recurs(setup):
    """Capturing costs far more than one step, so a batch size that passes by (requests ending one
    after another) runs eagerly; the size that stays is captured at its third step.  The logits are
    the plain implementation's either way."""
    name, dtype, engine, requests = setup
    config, page = TINY[name]
    fresh = TinyEngine(config, page, dtype, DEVICE, num_pages=64, max_requests=4, max_tokens=256,
                       tensors=engine.tensors)
    fresh.runner.graph_capture_after = 3
    texts = {rid: random_prompt(config.vocab_size, n, 190 + n) for rid, n in (("u", 31), ("v", 22), ("w", 18))}
    # three live for two steps, two for two more, then "u" alone for six
    decoded = {"u": 10, "v": 2, "w": 4}
    prompts = {rid: text[:len(text) - 10 + decoded[rid]] for rid, text in texts.items()}
    steps = [{"entries": [(rid, 0, len(texts[rid]) - 10) for rid in texts], "end": []}]
    for k in range(10):
        live = [rid for rid in texts if k < decoded[rid]]
        steps.append({"entries": [(rid, len(texts[rid]) - 10 + k, len(texts[rid]) - 9 + k) for rid in live],
                      "end": [rid for rid in live if k == decoded[rid] - 1]})
    results = replay(fresh, prompts, steps)
    assert [key[:3] for key in fresh.runner._graphs] == [(1, False, False)]
    assert fresh.runner.graph_replays == 3          # of six steps: two eager, one captured, three replayed
    check_all(fresh, prompts, results, dtype, "captured late")


def test_captured_steps_follow_the_context_limit(setup):
    """A captured decode step plans against a context limit: a short one while every request is
    below it, the cache's capacity after that.  A request that grows across the limit moves from one
    captured step to the other; its logits stay the plain implementation's."""
    name, dtype, engine, requests = setup
    config, page = TINY[name]
    fresh = TinyEngine(config, page, dtype, DEVICE, num_pages=64, max_requests=2, max_tokens=256,
                       tensors=engine.tensors)
    fresh.runner.CONTEXT_LIMITS = (64,)
    text = random_prompt(config.vocab_size, 80, 311)
    steps = [{"entries": [("u", 0, 50)], "end": []}]
    steps += [{"entries": [("u", 50 + k, 51 + k)], "end": ["u"] if k == 29 else []} for k in range(30)]
    results = replay(fresh, {"u": text}, steps)
    limits = sorted(key[3] for key in fresh.runner._graphs)
    assert limits == [64, fresh.cache.max_pages_per_request * page], limits
    check_all(fresh, {"u": text}, results, dtype, "across the context limit")
