"""The scheduler's decisions on the CPU with made-up tokens: decode priority, strict FIFO,
portions under the token budget, the mixed-step budget, static policy, page budgets and what
happens when pages run out, atomic write-back, abort."""

import pytest
import torch

from mini_llm_runtime_b200.cache import CacheManager
from mini_llm_runtime_b200.engine import (BatchingPolicy, CacheGate, FinishReason, RequestScheduler, RequestStatus,
                                          WorkKind)
from mini_llm_runtime_b200.parts import KVCacheNeed


def scheduler(**options):
    defaults = dict(max_running_requests=4, max_batch_tokens=16)
    defaults.update(options)
    return RequestScheduler(**defaults)


def finish_step(s, token=1):
    batch = s.outstanding_plan
    return s.apply_step_results({rid: token for rid in batch.emitting_request_ids})


def costs(batch):
    return [(i.request_id, i.kind.value, len(i.tokens), i.emits) for i in batch.items]


def test_decode_first_then_fifo_admission():
    s = scheduler()
    s.submit("a", [1, 2, 3], max_new_tokens=3)
    s.submit("b", [4, 5], max_new_tokens=2)
    batch = s.schedule_step()
    assert costs(batch) == [("a", "prefill", 3, True), ("b", "prefill", 2, True)]
    assert batch.token_count == 5 and batch.admitted_request_ids == ("a", "b")
    finish_step(s, 7)
    s.submit("c", [6], max_new_tokens=1)
    batch = s.schedule_step()
    assert costs(batch) == [("a", "decode", 1, True), ("b", "decode", 1, True), ("c", "prefill", 1, True)]
    assert batch.items[0].tokens == (7,)
    update = finish_step(s, 8)
    assert set(update.finished_request_ids) == {"b", "c"}
    assert s.get_request("b").finish_reason is FinishReason.MAX_TOKENS
    assert s.running_request_ids == ("a",) and s.get_request("c").status is RequestStatus.FINISHED


def test_a_long_prompt_is_cut_into_portions_and_emits_once():
    s = scheduler(max_batch_tokens=8, max_running_requests=2)
    s.submit("long", list(range(19)), max_new_tokens=2)
    s.submit("next", [1, 2], max_new_tokens=1)
    first = s.schedule_step()
    assert costs(first) == [("long", "prefill", 8, False)]
    assert first.emitting_request_ids == ()
    s.apply_step_results({})
    assert s.get_request("long").cursor == 8 and not s.get_request("long").prompt_done
    second = s.schedule_step()
    assert costs(second) == [("long", "prefill", 8, False)]
    assert second.items[0].tokens == tuple(range(8, 16)) and not second.items[0].admitted
    s.apply_step_results({})
    third = s.schedule_step()          # the rest of the prompt, then the next request in what is left
    assert costs(third) == [("long", "prefill", 3, True), ("next", "prefill", 2, True)]
    finish_step(s, 5)
    fourth = s.schedule_step()
    assert costs(fourth) == [("long", "decode", 1, True)]


def test_decodes_keep_their_place_when_portions_fill_the_budget():
    s = scheduler(max_batch_tokens=6, max_running_requests=3)
    s.submit("a", [1], max_new_tokens=5)
    s.schedule_step()
    finish_step(s)
    s.submit("b", list(range(20)), max_new_tokens=1)
    batch = s.schedule_step()
    assert costs(batch) == [("a", "decode", 1, True), ("b", "prefill", 5, False)]
    assert batch.token_count == 6


def test_whole_prompt_mode_is_the_reference_behaviour():
    s = scheduler(max_batch_tokens=8, chunked_prefill=False)
    with pytest.raises(ValueError):
        s.submit("too-long", list(range(9)), max_new_tokens=1)
    s.submit("a", list(range(6)), max_new_tokens=2)
    s.submit("b", list(range(5)), max_new_tokens=2)
    s.submit("c", [1], max_new_tokens=2)
    batch = s.schedule_step()
    assert costs(batch) == [("a", "prefill", 6, True)]    # b does not fit; c must not overtake it
    assert s.waiting_request_ids == ("b", "c")


def test_mixed_budget_limits_prompt_tokens_beside_decodes_only():
    s = scheduler(max_batch_tokens=16, max_mixed_prefill_tokens=4)
    s.submit("a", list(range(10)), max_new_tokens=4)
    first = s.schedule_step()
    assert costs(first) == [("a", "prefill", 10, True)]    # no decode in the step: no mixed limit
    finish_step(s)
    s.submit("b", list(range(9)), max_new_tokens=1)
    second = s.schedule_step()
    assert costs(second) == [("a", "decode", 1, True), ("b", "prefill", 4, False)]


def test_static_policy_does_not_refill_a_running_cohort():
    s = scheduler(batching_policy=BatchingPolicy.STATIC, max_running_requests=2)
    s.submit("a", [1], max_new_tokens=2)
    s.submit("b", [1], max_new_tokens=1)
    s.submit("c", [1], max_new_tokens=1)
    assert len(s.schedule_step().items) == 2
    finish_step(s)                                  # b finishes, a still runs
    assert costs(s.schedule_step()) == [("a", "decode", 1, True)]
    finish_step(s)
    assert costs(s.schedule_step()) == [("c", "prefill", 1, True)]


def test_eos_wins_over_the_length_limit_and_results_are_checked_first():
    s = scheduler()
    s.submit("a", [1], max_new_tokens=1, eos_token_ids=[9])
    s.submit("b", [1], max_new_tokens=3, eos_token_ids=9)
    s.schedule_step()
    with pytest.raises(ValueError):
        s.apply_step_results({"a": 9})               # b is missing: nothing may change
    with pytest.raises(ValueError):
        s.apply_step_results({"a": 9, "b": -1})
    assert s.get_request("a").generated_token_ids == ()
    update = s.apply_step_results({"a": 9, "b": 9})
    assert s.get_request("a").finish_reason is FinishReason.EOS
    assert s.get_request("b").finish_reason is FinishReason.EOS
    assert update.finished_request_ids == ("a", "b") and not s.has_unfinished_requests
    with pytest.raises(RuntimeError):
        s.apply_step_results({})


def test_abort_puts_new_requests_back_in_front_and_keeps_the_step_index():
    s = scheduler(max_running_requests=3)
    s.submit("a", [1], max_new_tokens=3)
    s.schedule_step()
    finish_step(s)
    s.submit("b", [1, 2], max_new_tokens=1)
    s.submit("c", [3], max_new_tokens=1)
    batch = s.schedule_step()
    assert batch.index == 1 and batch.admitted_request_ids == ("b", "c")
    s.submit("d", [4], max_new_tokens=1)            # arrives while the batch is out
    with pytest.raises(RuntimeError):
        s.schedule_step()
    s.abort_step()
    assert s.waiting_request_ids == ("b", "c", "d") and s.running_request_ids == ("a",)
    assert s.get_request("b").status is RequestStatus.WAITING
    again = s.schedule_step()
    assert again.index == 1 and [i.request_id for i in again.items] == ["a", "b", "c"]


def test_submit_validation():
    s = scheduler()
    for bad in (dict(request_id="", prompt_token_ids=[1], max_new_tokens=1),
                dict(request_id="x", prompt_token_ids=[], max_new_tokens=1),
                dict(request_id="x", prompt_token_ids=[-1], max_new_tokens=1),
                dict(request_id="x", prompt_token_ids=[True], max_new_tokens=1),
                dict(request_id="x", prompt_token_ids=[1], max_new_tokens=0),
                dict(request_id="x", prompt_token_ids=[1], max_new_tokens=1, temperature=-1.0),
                dict(request_id="x", prompt_token_ids=[1], max_new_tokens=1, seed=-1)):
        with pytest.raises(ValueError):
            s.submit(**bad)
    s.submit("x", [1], max_new_tokens=1)
    with pytest.raises(ValueError):
        s.submit("x", [1], max_new_tokens=1)
    with pytest.raises(ValueError):
        RequestScheduler(max_running_requests=5, max_batch_tokens=4)
    assert s.get_request("x").lifetime_tokens == 1


def page_limited(pages, page=4, tokens=64, **options):
    manager = CacheManager([KVCacheNeed(1, 8, None)], page_size=page, num_pages=pages, max_requests=4,
                           max_tokens_per_request=tokens, dtype=torch.float32, device="cpu",
                           allocate_device_memory=False)
    return manager, scheduler(gate=CacheGate(manager), **options)


def test_when_pages_run_out_the_head_of_the_queue_waits_and_blocks_those_behind_it():
    manager, s = page_limited(pages=4)
    s.submit("a", list(range(8)), max_new_tokens=5)      # 12 tokens -> 3 pages
    s.submit("b", list(range(5)), max_new_tokens=4)      # 8 tokens -> 2 pages: must wait
    s.submit("c", [1], max_new_tokens=1)                 # 1 page would fit, but may not overtake b
    batch = s.schedule_step()
    assert [i.request_id for i in batch.items] == ["a"]
    assert manager.get("a").promised == [3] and batch.items[0].slot == manager.get("a").slot
    assert manager.groups[0].allocator.promised == 3 and "b" not in manager.requests
    for _ in range(4):
        finish_step(s)
        assert [i.request_id for i in s.schedule_step().items] == ["a"]
    update = finish_step(s)                               # a's fifth token: finished, and its pages are back
    assert update.finished_request_ids == ("a",) and "a" in update.freed
    assert manager.groups[0].allocator.promised == 0 and "a" not in manager.requests
    batch = s.schedule_step()
    assert [i.request_id for i in batch.items] == ["b", "c"]


def test_a_request_that_can_never_fit_is_an_error_not_a_wait():
    manager, s = page_limited(pages=2)
    s.submit("huge", list(range(9)), max_new_tokens=1)    # 3 pages, the pool has 2
    with pytest.raises(ValueError):
        s.schedule_step()
    manager, s = page_limited(pages=100, tokens=16)
    s.submit("long", list(range(16)), max_new_tokens=2)   # 17 tokens, requests are capped at 16
    with pytest.raises(ValueError):
        s.schedule_step()


def test_an_aborted_step_gives_slots_and_promises_back():
    manager, s = page_limited(pages=8)
    s.submit("a", [1, 2], max_new_tokens=2)
    s.submit("b", [3], max_new_tokens=2)
    s.schedule_step()
    assert manager.stats().live_requests == 2
    s.abort_step()
    assert manager.stats().live_requests == 0 and manager.groups[0].allocator.promised == 0
    assert s.waiting_request_ids == ("a", "b") and s.get_request("a").slot is None
    with pytest.raises(RuntimeError):
        s.abort_step()


def test_failed_requests_end_with_an_error_and_free_everything():
    manager, s = page_limited(pages=8)
    s.submit("a", [1, 2], max_new_tokens=4)
    s.submit("b", [3], max_new_tokens=4)
    s.schedule_step()
    finish_step(s)
    s.submit("c", [5], max_new_tokens=1)
    s.schedule_step()                                     # a and b decode, c is admitted
    assert s.fail_requests(["a", "c"]) == ("a", "c")
    assert s.get_request("a").finish_reason is FinishReason.ERROR
    assert s.get_request("c").status is RequestStatus.FINISHED and s.outstanding_plan is None
    assert set(manager.requests) == {"b"} and s.running_request_ids == ("b",)
    assert [i.request_id for i in s.schedule_step().items] == ["b"]     # the engine goes on with the rest
