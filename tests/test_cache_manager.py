"""The cache manager on the CPU (no device memory): pages are never lost, held twice or freed
twice, under random orders of requests; transactions; windows; promises; slots."""

import random

import pytest
import torch

from mini_llm_runtime_b200.cache import CacheManager, OutOfPages, PoolAllocator
from mini_llm_runtime_b200.parts import KVCacheNeed, StateNeed

FULL = KVCacheNeed(2, 16, None)
WINDOW = KVCacheNeed(2, 16, 20)


def manager(needs=(FULL, FULL), pages=8, page=4, requests=4, tokens=64, step=16):
    return CacheManager(list(needs), page_size=page, num_pages=pages, max_requests=requests,
                        max_tokens_per_request=tokens, dtype=torch.float32, device="cpu",
                        max_step_tokens=step, allocate_device_memory=False)


def test_allocator_is_atomic_ordered_and_detects_double_free():
    pool = PoolAllocator(5)
    assert pool.allocate(3) == [0, 1, 2]
    with pytest.raises(OutOfPages):
        pool.allocate(3)
    assert pool.free_count == 2
    pool.free([1])
    assert pool.allocate(2) == [1, 3]      # lowest free id first
    with pytest.raises(ValueError):
        pool.free([4])                     # never handed out
    pool.free([0, 3])
    with pytest.raises(ValueError):
        pool.free([0])                     # double free
    with pytest.raises(ValueError):
        pool.free([1, 1])
    assert pool.held == frozenset({1, 2})
    assert pool.promise(5) and not pool.promise(1)
    pool.unpromise(2)
    assert pool.promised == 3
    with pytest.raises(ValueError):
        pool.unpromise(4)


def test_layers_with_equal_needs_share_a_group_and_windows_get_their_own():
    m = manager(needs=(FULL, WINDOW, FULL, StateNeed((3,)), WINDOW, None))
    assert [g.entries for g in m.groups] == [[0, 2], [1, 4]]
    assert m.entry_group == {0: (0, 0), 2: (0, 1), 1: (1, 0), 4: (1, 1)}
    assert m.groups[1].window == 20


def test_step_transaction_commit_abort_and_address_map():
    m = manager()
    m.create_request("a")
    m.begin_step([("a", 6)])
    request = m.get("a")
    assert request.pending == (0, 6) and request.committed == 0 and request.pages[0] == [0, 1]
    assert m.slot_mapping(m.groups[0], request, 0, 6).tolist() == [0, 1, 2, 3, 4, 5]
    m.abort_step()
    assert request.pages[0] == [] and m.groups[0].allocator.free_count == 8 and request.committed == 0
    m.begin_step([("a", 6)])
    m.commit_step()
    assert request.committed == 6
    m.create_request("b")
    m.begin_step([("b", 3), ("a", 3)])
    assert m.get("b").pages[0] == [2] and request.pages[0] == [0, 1, 3]
    assert m.slot_mapping(m.groups[0], request, 6, 3).tolist() == [6, 7, 12]
    m.abort_step()                       # only the pages this step took go back
    assert request.pages[0] == [0, 1] and m.get("b").pages[0] == []
    m.check_consistency()
    with pytest.raises(RuntimeError):
        m.commit_step()


def test_out_of_pages_changes_nothing():
    m = manager(pages=3)
    m.create_request("a")
    m.create_request("b")
    m.begin_step([("a", 8)])
    m.commit_step()
    with pytest.raises(OutOfPages):
        m.begin_step([("a", 1), ("b", 5)])          # a's page would fit, b's two do not
    assert not m.step_in_flight and m.get("a").pages[0] == [0, 1] and m.get("b").pages[0] == []
    assert m.groups[0].allocator.free_count == 1
    m.check_consistency()
    m.begin_step([("a", 1)])
    m.commit_step()
    assert m.release("a")[0] == [0, 1, 2]
    m.begin_step([("b", 5)])                        # freed pages are used again, lowest first
    assert m.get("b").pages[0] == [0, 1]


def test_step_rules():
    m = manager()
    m.create_request("a")
    with pytest.raises(ValueError):
        m.begin_step([("a", 1), ("a", 1)])
    with pytest.raises(ValueError):
        m.begin_step([("a", 0)])
    with pytest.raises(KeyError):
        m.begin_step([("zz", 1)])
    with pytest.raises(ValueError):
        m.begin_step([("a", 65)])                   # beyond max_tokens_per_request
    with pytest.raises(ValueError):
        m.create_request("a")
    m.begin_step([("a", 1)])
    with pytest.raises(RuntimeError):
        m.begin_step([("a", 1)])
    with pytest.raises(RuntimeError):
        m.release("a")                              # part of the step in flight


def test_window_gives_pages_back_once_passed():
    m = manager(needs=(FULL, WINDOW), pages=32, page=4, tokens=128, step=16)
    m.create_request("a")
    m.begin_step([("a", 16)])
    m.commit_step()                                 # next position 16 sees keys > -4: nothing to free
    assert m.get("a").pages[1] == [0, 1, 2, 3]
    m.begin_step([("a", 13)])
    released = m.commit_step()                      # next position 29 sees keys >= 10: pages 0, 1 go
    assert released == {"a": {1: [0, 1]}}
    assert m.get("a").pages[1][:2] == [-1, -1] and m.get("a").pages[0][:2] == [0, 1]
    assert (m.groups[1].table[m.get("a").slot, :2] == -1).all()
    m.check_consistency()
    for _ in range(40):
        m.begin_step([("a", 1)])
        m.commit_step()
        m.check_consistency()
    held = m.get("a").held(1)
    assert held <= m.pages_for_lifetime(m.groups[1], 128)
    assert m.get("a").held(0) == -(-69 // 4)
    m.release("a")
    assert all(g.allocator.free_count == g.num_pages for g in m.groups)


def test_promises_guarantee_a_running_request_its_pages():
    m = manager(needs=(FULL, WINDOW), pages=[6, 6], page=4, tokens=24, step=4)
    assert m.lifetime_pages(24) == (6, min(6, -(-(19 + 4) // 4) + 1))
    assert m.create_request("a", lifetime_tokens=12) is not None       # 3 pages
    assert m.create_request("b", lifetime_tokens=12) is not None       # 3 pages
    assert m.create_request("c", lifetime_tokens=4) is None            # nothing left to promise
    assert "c" not in m.requests and m.slots.free_count == 2
    with pytest.raises(ValueError):
        m.create_request("d", lifetime_tokens=25)                      # can never fit
    for _ in range(3):
        m.begin_step([("a", 4), ("b", 4)])
        m.commit_step()
    with pytest.raises(OutOfPages):
        m.begin_step([("a", 1)])                                       # beyond its promise
    m.release("a")
    assert m.groups[0].allocator.promised == 3
    assert m.create_request("c", lifetime_tokens=12) is not None
    m.check_consistency()


def test_slots_and_state_are_per_request():
    m = CacheManager([FULL, StateNeed((2, 3))], page_size=4, num_pages=4, max_requests=2,
                     max_tokens_per_request=16, dtype=torch.float32, device="cpu")
    a = m.create_request("a")
    b = m.create_request("b")
    assert {a.slot, b.slot} == {0, 1} and m.state[1].shape == (2, 2, 3)
    with pytest.raises(OutOfPages):
        m.create_request("c")
    m.state[1][a.slot] += 5
    m.release("a")
    again = m.create_request("c")
    assert again.slot == a.slot and float(m.state[1][again.slot].abs().sum()) == 0.0   # zeroed on reuse
    assert m.stats().free_slots == 0 and m.stats().live_requests == 2


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_share_a_page(seed):
    rng = random.Random(seed)
    m = manager(needs=(FULL, WINDOW, FULL), pages=[24, 10], page=4, requests=5, tokens=80, step=12)
    live: dict[str, int] = {}
    counter = 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            counter += 1
            m.create_request(f"r{counter}")
            live[f"r{counter}"] = 0
        elif action < 0.35 and live:
            rid = rng.choice(sorted(live))
            m.release(rid)
            del live[rid]
        elif live:
            chosen = rng.sample(sorted(live), rng.randint(1, len(live)))
            entries = [(rid, rng.randint(1, 12)) for rid in chosen if live[rid] < 68]
            if not entries:
                continue
            before = {g.index: g.allocator.free_count for g in m.groups}
            try:
                m.begin_step(entries)
            except OutOfPages:
                assert {g.index: g.allocator.free_count for g in m.groups} == before
                m.check_consistency()
                continue
            if rng.random() < 0.2:
                m.abort_step()
                assert {g.index: g.allocator.free_count for g in m.groups} == before
            else:
                m.commit_step()
                for rid, count in entries:
                    live[rid] += count
        m.check_consistency()
        for rid, tokens in live.items():
            request = m.get(rid)
            assert request.committed == tokens
            assert request.held(0) == -(-tokens // 4)
            lowest = max(0, tokens - 20 + 1) // 4
            assert all(p >= 0 for p in request.pages[1][lowest:]) and all(p < 0 for p in request.pages[1][:lowest])
    for rid in list(live):
        m.release(rid)
    assert all(g.allocator.free_count == g.num_pages and g.allocator.promised == 0 for g in m.groups)
    assert m.slots.free_count == 5


def test_requests_without_a_promise_cannot_take_what_is_promised_to_others():
    """A request admitted with a promise and one created without (replay, greedy_generate) on one
    manager: the second may only take pages that no promise covers."""
    m = manager(needs=(FULL,), pages=6, page=4, tokens=24, step=8)
    assert m.create_request("promised", lifetime_tokens=16) is not None      # 4 of the 6 pages
    m.create_request("free-rider")
    m.begin_step([("free-rider", 8)])                                        # the 2 uncovered pages
    m.commit_step()
    with pytest.raises(OutOfPages):
        m.begin_step([("free-rider", 1)])                                    # a third would cut into the promise
    for _ in range(4):                                                       # the promise is honoured to its end
        m.begin_step([("promised", 4)])
        m.commit_step()
    assert m.groups[0].allocator.free_count == 0
    m.release("promised")
    m.begin_step([("free-rider", 1)])
    m.commit_step()
    m.check_consistency()
    pool = PoolAllocator(4)
    assert pool.promise(3)
    taken = pool.allocate(2, promised=True)
    with pytest.raises(ValueError):
        pool.unpromise(3)                    # two pages are still held under it
    pool.free(taken, promised=True)
    pool.unpromise(3)


def resident(needs=(FULL, WINDOW), **options):
    """A manager on the CPU that believes its tables live elsewhere, so that it reports changed rows."""
    defaults = dict(page_size=4, num_pages=16, max_requests=3, max_tokens_per_request=64, dtype=torch.float32,
                    device="cpu", max_step_tokens=16)
    defaults.update(options)
    m = CacheManager(list(needs), **defaults)
    m._shares_host_memory = False
    for group in m.groups:
        group.device_table = group.device_table.clone()
    m.slot_state = m.slot_state.clone()
    return m


def apply_updates(m):
    updates = m.take_resident_updates()
    for table, rows, values in updates:
        table[torch.from_numpy(rows).long()] = torch.from_numpy(values)
    m.resident_updates_sent()
    return updates


def test_only_changed_rows_of_the_resident_tables_are_handed_out():
    from mini_llm_runtime_b200.cache import read_record

    m = resident()
    a = m.create_request("a", temperature=0.5, seed=(7 << 32) | 9)
    m.create_request("b")
    m.begin_step([("a", 6), ("b", 2)])
    updates = apply_updates(m)
    assert [int(table.shape[1]) for table, _, _ in updates] == [16, 16, 8]    # two block tables, the slot records
    assert [rows.tolist() for _, rows, _ in updates] == [[0, 1], [0, 1], [0, 1]]
    record = read_record(m.slot_state[a.slot].numpy())
    assert record == {"length": 0, "last_token": 0, "counter": 0, "temperature": 0.5, "seed": (7 << 32) | 9}
    m.commit_step()
    for _ in range(2):                       # a fills its second page: no row changes, nothing to send
        m.begin_step([("a", 1)])
        assert m.take_resident_updates() == []
        m.resident_updates_sent()
        m.commit_step()
    m.begin_step([("a", 1)])                 # a crosses into a third page: its row alone, in both groups
    updates = apply_updates(m)
    assert [rows.tolist() for _, rows, _ in updates] == [[a.slot], [a.slot]]
    m.commit_step()
    for group in m.groups:
        assert torch.equal(group.device_table, torch.from_numpy(group.table))
    m.release("b")
    assert [rows.tolist() for _, rows, _ in apply_updates(m)] == [[1], [1]]


def test_rows_handed_out_but_never_sent_are_handed_out_again():
    m = resident(needs=(FULL,))
    m.create_request("a")
    m.begin_step([("a", 5)])
    first = m.take_resident_updates()        # the step fails before it can send them
    m.abort_step()
    m.begin_step([("a", 5)])
    again = m.take_resident_updates()
    assert [rows.tolist() for _, rows, _ in again] == [rows.tolist() for _, rows, _ in first] == [[0], [0]]
    m.resident_updates_sent()
    m.commit_step()
    assert m.take_resident_updates() == []


def test_an_aborted_step_restores_fixed_size_state():
    m = CacheManager([FULL, StateNeed((3,))], page_size=4, num_pages=8, max_requests=3,
                     max_tokens_per_request=32, dtype=torch.float32, device="cpu")
    a, b = m.create_request("a"), m.create_request("b")
    m.state[1][a.slot] = torch.tensor([1.0, 2.0, 3.0])
    m.begin_step([("a", 2)])
    m.state[1][a.slot] += 10                 # a mixer writes its state in place during the step
    m.state[1][b.slot] += 1                  # b is not part of the step: not the manager's to restore
    m.abort_step()
    assert m.state[1][a.slot].tolist() == [1.0, 2.0, 3.0] and m.state[1][b.slot].tolist() == [1.0, 1.0, 1.0]
    m.begin_step([("a", 2)])
    m.state[1][a.slot] += 10
    m.commit_step()
    assert m.state[1][a.slot].tolist() == [11.0, 12.0, 13.0]
