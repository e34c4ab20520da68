"""Claims that only a whole engine can break, on the GPU:

* float32 logits are the same *bits* however the tokens are cut into steps and batched;
* models with the layer sizes of real checkpoints (Qwen2.5-0.5B with 2 of its 24 layers, Qwen2.5-7B
  with 1 of its 28) agree with the plain implementation, run in float32 on the GPU, under the four
  ways of cutting;
* what the device keeps per slot follows the requests; a captured decode step stays right when a
  slot is taken over by a request with a shorter context; scratch memory that captured steps point
  at is never replaced; NVTX ranges can be switched on.
"""

from __future__ import annotations

import pytest
import torch

import plain_qwen2 as plain
import scenarios
from harness import TinyEngine, assert_close, random_prompt
from mini_llm_runtime_b200 import ops
from mini_llm_runtime_b200.cache import CacheManager, read_record
from mini_llm_runtime_b200.config import Qwen2Config
from mini_llm_runtime_b200.engine import ContinuousBatchEngine, ModelRunner, StepEntry
from mini_llm_runtime_b200.models import build_model
from mini_llm_runtime_b200.weights import random_tensors
from tiny_configs import TINY

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


def run_steps(engine, requests, steps, wanted=None):
    """Replay ``steps``; returns request id -> {position: logits row}.  ``wanted``: positions whose
    logits are asked for (default: all)."""
    rows: dict[str, dict[int, torch.Tensor]] = {rid: {} for rid in requests}
    for step in steps:
        entries, places = [], []
        for rid, start, end in step["entries"]:
            if rid not in engine.cache.requests:
                engine.cache.create_request(rid)
            want = [p - start for p in range(start, end) if wanted is None or p in wanted[rid]]
            entries.append(StepEntry(rid, requests[rid][start:end], want))
            places += [(rid, start + w) for w in want]
        logits = engine.runner.step(entries)
        for row, (rid, position) in enumerate(places):
            rows[rid][position] = logits[row].clone()
        for rid in step["end"]:
            engine.cache.release(rid)
    return rows


def four_ways(requests, seed=5):
    return {"whole": scenarios.whole(requests), "tail": scenarios.tail_one_by_one(requests),
            "portions": scenarios.changing_portions(requests), "mixed": scenarios.mixed(requests, seed)}


@pytest.mark.parametrize("name", list(TINY))
def test_float32_logits_are_the_same_bits_under_every_cut(name):
    config, page = TINY[name]
    engine = TinyEngine(config, page, torch.float32, DEVICE, num_pages=96, max_requests=4, max_tokens=512, seed=13)
    requests = {f"q{i}": random_prompt(config.vocab_size, n, 400 + i) for i, n in enumerate((3, 70, 45, 131, 18))}
    results = {way: run_steps(engine, requests, steps) for way, steps in four_ways(requests).items()}
    for way in ("tail", "portions", "mixed"):
        for rid, tokens in requests.items():
            for position in range(len(tokens)):
                assert torch.equal(results[way][rid][position], results["whole"][rid][position]), \
                    f"{name}: request {rid}, position {position}: '{way}' and 'whole' differ in float32"


REAL_SIZES = {
    # Qwen2.5-0.5B layer sizes, 2 of its 24 layers
    "0.5b-2-layers": (dict(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_hidden_layers=2,
                           num_attention_heads=14, num_key_value_heads=2, max_position_embeddings=32768,
                           rms_norm_eps=1e-6, rope_theta=1000000.0, hidden_act="silu", tie_word_embeddings=True),
                      (300, 2100)),
    # Qwen2.5-7B layer sizes (head_dim 128, seven query heads per kv head, untied head), 1 of its 28 layers
    "7b-1-layer": (dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=1,
                        num_attention_heads=28, num_key_value_heads=4, max_position_embeddings=32768,
                        rms_norm_eps=1e-6, rope_theta=1000000.0, hidden_act="silu", tie_word_embeddings=False),
                   (150, 700)),
}


@pytest.fixture(scope="module", params=list(REAL_SIZES))
def real_size(request):
    sizes, lengths = REAL_SIZES[request.param]
    config = Qwen2Config(**sizes)
    expected = build_model(config, torch.bfloat16).expected_tensors()
    tensors = random_tensors(expected, 17, torch.bfloat16)
    requests = {f"s{n}": random_prompt(config.vocab_size, n, 500 + n) for n in lengths}
    # logits of a few dozen positions per request: the first, page and tile edges, the last ones
    wanted = {}
    for rid, tokens in requests.items():
        n = len(tokens)
        wanted[rid] = sorted({0, 1, 15, 16, 17, 63, 64, 127, 128, 129, n // 2, n - 40} | set(range(n - 34, n))
                             | set(range(255, n, 509)))
        wanted[rid] = [p for p in wanted[rid] if 0 <= p < n]
    on_device = {name: tensor.to(DEVICE) for name, tensor in tensors.items()}
    with torch.inference_mode():
        oracle = {rid: plain.forward_logits(on_device, config.to_dict(), tokens, rows=wanted[rid]).cpu()
                  for rid, tokens in requests.items()}
    del on_device
    torch.cuda.empty_cache()
    yield request.param, config, tensors, requests, wanted, oracle


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_real_layer_sizes_under_the_four_ways_of_cutting(real_size, dtype):
    name, config, tensors, requests, wanted, oracle = real_size
    engine = TinyEngine(config, 16, dtype, DEVICE, num_pages=320, max_requests=4, max_tokens=2304,
                        max_step_tokens=2304, tensors=tensors)
    sets = {rid: set(places) for rid, places in wanted.items()}
    for way, steps in four_ways(requests).items():
        rows = run_steps(engine, requests, steps, sets)
        for rid in requests:
            got = torch.stack([rows[rid][p] for p in wanted[rid]])
            assert_close(got, oracle[rid], dtype, f"{name}, {way}, request {rid}")
        assert not engine.cache.requests
    del engine
    torch.cuda.empty_cache()


def test_slot_records_on_the_device_follow_the_requests():
    config, page = TINY["D"]
    model = build_model(config, torch.bfloat16)
    model.load(random_tensors(model.expected_tensors(), 23), DEVICE)
    engine = ContinuousBatchEngine.from_model(model, block_size=page, max_running_requests=3, max_batch_tokens=48,
                                              max_model_len=256, step_ahead=False)
    for i, n in enumerate((70, 9, 33, 5)):
        engine.submit(f"r{i}", random_prompt(config.vocab_size, n, 600 + i), max_new_tokens=6 + 3 * i,
                      temperature=0.4 * (i % 2), seed=100 + i)
    replays = 0
    while engine.scheduler.has_unfinished_requests:
        engine.step()
        state = engine.manager.slot_state.cpu().numpy()
        for rid in engine.scheduler.running_request_ids:
            request, held = engine.scheduler.get_request(rid), engine.manager.get(rid)
            record = read_record(state[held.slot])
            assert record["length"] == held.committed, rid
            assert record["counter"] == len(request.generated_token_ids), rid
            assert record["seed"] == request.seed and abs(record["temperature"] - request.temperature) < 1e-7
            if request.generated_token_ids:
                assert record["last_token"] == request.generated_token_ids[-1], rid
        with torch.inference_mode():                 # rows changed by this step's commit travel with the next step
            engine.runner._send_resident_updates()
        for group in engine.manager.groups:          # then the resident block tables mirror the host's
            assert torch.equal(group.device_table.cpu(), torch.from_numpy(group.table))
        replays = engine.runner.graph_replays
    assert replays > 0, "decode steps must have been replayed from captured graphs"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_a_captured_decode_step_after_its_slots_changed_hands(dtype):
    """Three requests decode through a captured graph; one ends, and a request with a much shorter
    context takes over its slot (and, the pool being small, its pages).  The same graph keeps being
    replayed; every position's logits still equal the plain implementation's."""
    config, page = TINY["D"]
    engine = TinyEngine(config, page, dtype, DEVICE, num_pages=24, max_requests=3, max_tokens=256, seed=29)
    assert engine.runner.use_graphs
    tokens = {rid: random_prompt(config.vocab_size, n, 700 + n) for rid, n in (("u", 150), ("v", 60), ("w", 90), ("x", 30))}
    steps = [{"entries": [(rid, 0, len(tokens[rid]) - 12) for rid in ("u", "v", "w")], "end": []}]
    for k in range(12):
        steps.append({"entries": [(rid, len(tokens[rid]) - 12 + k, len(tokens[rid]) - 11 + k) for rid in ("u", "v", "w")],
                      "end": ["u"] if k == 11 else []})
    # all three end; x, y and z take over their slots and pages with shorter contexts, in another order
    tokens["y"], tokens["z"] = random_prompt(config.vocab_size, 40, 801), random_prompt(config.vocab_size, 22, 802)
    steps[-1]["end"] = ["u", "v", "w"]
    steps.append({"entries": [(rid, 0, len(tokens[rid]) - 10) for rid in ("x", "y", "z")], "end": []})
    for k in range(10):
        steps.append({"entries": [(rid, len(tokens[rid]) - 10 + k, len(tokens[rid]) - 9 + k) for rid in ("z", "x", "y")],
                      "end": ["x", "y", "z"] if k == 9 else []})
    before = engine.runner.graph_replays
    rows = run_steps(engine, tokens, steps)
    assert engine.runner.graph_replays - before >= 20
    for rid, text in tokens.items():
        got = torch.stack([rows[rid][p] for p in range(len(text))])
        assert_close(got, engine.plain_logits(text), dtype, f"request {rid}")


def test_split_kv_scratch_is_never_replaced_under_captured_steps():
    """Captured launches keep the address of the split-KV scratch buffer.  A batch whose partial
    states would not fit must lower its split count instead of getting a new buffer, and the graph
    captured earlier must still give the right logits afterwards.  (The buffer is made to look small
    for the large batch; at its real size only batches of many thousands of heads reach the limit.)"""
    config, page = TINY["E"]          # head_dim 128, page 32: the bulk-copy decode kernel
    kernels = ops.current()
    space = kernels._workspace(torch.device(DEVICE))
    whole_buffer = space["attention_scratch"]
    engine = TinyEngine(config, page, torch.bfloat16, DEVICE, num_pages=64, max_requests=4, max_tokens=512, seed=31)
    tokens = {rid: random_prompt(config.vocab_size, n, 900 + n) for rid, n in (("a", 300), ("b", 120))}
    head = [{"entries": [(rid, 0, len(t) - 16) for rid, t in tokens.items()], "end": []}]
    first = [{"entries": [(rid, len(t) - 16 + k, len(t) - 15 + k) for rid, t in tokens.items()], "end": []} for k in range(8)]
    last = [{"entries": [(rid, len(t) - 8 + k, len(t) - 7 + k) for rid, t in tokens.items()],
             "end": list(tokens) if k == 7 else []} for k in range(8)]
    rows = run_steps(engine, tokens, head + first)
    assert engine.runner.graph_replays >= 6
    per_split = 64 * config.num_attention_heads * (config.head_dim + 2) * 4     # 64 rows
    try:
        space["attention_scratch"] = whole_buffer[: 3 * per_split + 64]        # room for three splits only
        kernels.decode_max_splits = 8                                          # and eight are asked for
        big = TinyEngine(config, page, torch.bfloat16, DEVICE, num_pages=200, max_requests=64, max_tokens=96,
                         tensors=engine.tensors)
        many = {f"m{i}": random_prompt(config.vocab_size, 70, 1000 + i) for i in range(64)}
        steps = [{"entries": [(rid, 0, 69) for rid in many], "end": []},
                 {"entries": [(rid, 69, 70) for rid in many], "end": list(many)}]
        got = run_steps(big, many, steps, {rid: {69} for rid in many})
        for rid in ("m0", "m63"):
            assert_close(got[rid][69][None], big.plain_logits(many[rid])[-1:], torch.bfloat16, rid)
        assert space["attention_scratch"].data_ptr() == whole_buffer.data_ptr()
        with pytest.raises(ops.KernelError, match="scratch"):
            space["attention_scratch"] = whole_buffer[: per_split // 2]         # not even one split fits: refused
            run_steps(big, many, steps[:1] + [dict(steps[1], end=[])], {rid: set() for rid in many})
    finally:
        kernels.decode_max_splits = None
        space["attention_scratch"] = whole_buffer
    more = run_steps(engine, tokens, last)
    for rid, text in tokens.items():
        rows[rid].update(more[rid])
        got = torch.stack([rows[rid][p] for p in range(len(text))])
        assert_close(got, engine.plain_logits(text), torch.bfloat16, f"request {rid}")


def test_nvtx_ranges_can_be_switched_on():
    config, page = TINY["A"]
    model = build_model(config, torch.float32)
    tensors = random_tensors(model.expected_tensors(), 37)
    model.load(tensors, DEVICE)
    engine = ContinuousBatchEngine.from_model(model, block_size=page, max_running_requests=2, max_batch_tokens=16,
                                              max_model_len=64, enable_nvtx=True, step_ahead=True)
    prompt = random_prompt(config.vocab_size, 21, 3)
    assert engine.generate([prompt], max_new_tokens=5)[0] == plain.greedy_tokens(tensors, config.to_dict(), prompt, 5)
