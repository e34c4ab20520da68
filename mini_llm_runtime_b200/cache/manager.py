"""The cache manager: keys and values in pages, one block table per request and group, and slots
of fixed-size state per request.

What the model's mixers need is declared per cache entry (one entry per run step that writes):
``KVCacheNeed`` (all earlier keys, or a window of them) or ``StateNeed`` (a fixed-size tensor per
request).  Entries with the same key/value geometry and window form a *group*; each group has
its own page pool, its own allocator and, per request, its own block table, because a windowed
group gives pages back while the request still runs and a full group does not.

Pool layout per group: ``key`` and ``value`` are ``[entry, page, kv_head, offset_in_page,
head_dim]``, the reference's ``[layer, physical_block, kv_head, block_offset, head_dim]``
(src/mini_llm_runtime/paged_kv_cache.py:290,305-318).  Address of token t of a request:
``page = table[t // page_size]``, ``offset = t % page_size`` (:245-262).

Appending is a transaction over all requests of a step, like the reference's
begin/commit/abort (src/mini_llm_runtime/paged_kv_cache.py:202-243, paged_batch.py:89-114):
``begin_step`` takes every page the step needs or none at all, tokens become visible at
``commit_step``, ``abort_step`` returns only the pages this step took.  Pages are given back when
a request is released, when a step is aborted, and - for windowed groups - at commit, once every
position that could still look at a page has moved past it.

What the device keeps.  Each group's block table ``[max_requests, max_pages_per_request]`` and
the slot records (cache/slots.py) stay on the device; the host holds a mirror and remembers which
rows changed (a page taken, a page given back, a request admitted or released).
``take_resident_updates`` hands those rows out as snapshots, and the step function sends them
along with its own metadata; a step that changes no row sends none.  Kernels reach a request's
row through its slot.

Two admission modes.  With a *promise* (``create_request(..., lifetime_tokens=n)``) the pages of
the request's whole life are counted against the pool at creation, as the reference reserves them
(src/mini_llm_runtime/block_admission.py:35-67), so the pool cannot run dry mid-request; pages are
still taken only when tokens arrive.  Without a promise, pages are taken on demand and
``begin_step`` raises ``OutOfPages`` (leaving everything unchanged) when the pool is empty.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from ..parts.base import KVCacheNeed, StateNeed
from .allocator import OutOfPages, PoolAllocator
from .slots import SLOT_WORDS, slot_record


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


@dataclass
class CacheGroup:
    """Cache entries that share a geometry and a window, with their own pages."""

    index: int
    need: KVCacheNeed
    entries: list[int]
    page_size: int
    num_pages: int
    allocator: PoolAllocator
    key: torch.Tensor | None = None    # [entries, pages, kv_heads, page_size, head_dim]
    value: torch.Tensor | None = None
    table: np.ndarray | None = None    # host mirror: int32 [max_requests, max_pages_per_request], -1 = no page
    device_table: torch.Tensor | None = None   # the same table where the kernels read it
    dirty: set = field(default_factory=set)    # slots whose row differs from the device's copy

    @property
    def window(self) -> int | None:
        return self.need.window

    def bytes_per_page(self, itemsize: int) -> int:
        return 2 * len(self.entries) * self.need.num_kv_heads * self.page_size * self.need.head_dim * itemsize


@dataclass
class RequestCache:
    request_id: str
    slot: int
    committed: int = 0
    pending: tuple[int, int] | None = None
    pages: list[list[int]] = field(default_factory=list)      # per group: logical page -> id or -1
    first_live: list[int] = field(default_factory=list)       # per group: lowest logical page held
    promised: list[int] = field(default_factory=list)         # per group pages promised (0: none)
    step_new_pages: list[list[int]] = field(default_factory=list)

    def held(self, group: int) -> int:
        return sum(1 for p in self.pages[group] if p >= 0)


@dataclass(frozen=True)
class CacheStats:
    """Counterpart of the reference's PagedCacheStats (src/mini_llm_runtime/paged_kv_manager.py:34-50)."""

    total_pages: tuple[int, ...]
    free_pages: tuple[int, ...]
    held_pages: tuple[int, ...]
    promised_pages: tuple[int, ...]
    live_requests: int
    committed_tokens: int
    pending_tokens: int
    free_slots: int


class CacheManager:
    def __init__(self, needs: Sequence[KVCacheNeed | StateNeed | None], *, page_size: int,
                 num_pages: int | Sequence[int], max_requests: int, max_tokens_per_request: int,
                 dtype: torch.dtype, device: torch.device | str, max_step_tokens: int | None = None,
                 allocate_device_memory: bool = True) -> None:
        if page_size <= 0 or max_requests <= 0 or max_tokens_per_request <= 0:
            raise ValueError("page_size, max_requests and max_tokens_per_request must be > 0")
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.max_tokens_per_request = int(max_tokens_per_request)
        self.max_pages_per_request = _ceil_div(self.max_tokens_per_request, self.page_size)
        self.max_step_tokens = int(max_step_tokens or max_tokens_per_request)
        self.dtype = dtype
        self.device = torch.device(device)
        self.needs = list(needs)

        # ---- groups of key/value entries
        self.groups: list[CacheGroup] = []
        self.entry_group: dict[int, tuple[int, int]] = {}   # entry -> (group, index within group)
        by_need: dict[KVCacheNeed, int] = {}
        for entry, need in enumerate(self.needs):
            if not isinstance(need, KVCacheNeed):
                continue
            if need not in by_need:
                by_need[need] = len(self.groups)
                self.groups.append(CacheGroup(len(self.groups), need, [], self.page_size, 0, None))
            group = self.groups[by_need[need]]
            self.entry_group[entry] = (group.index, len(group.entries))
            group.entries.append(entry)
        counts = [int(num_pages)] * len(self.groups) if isinstance(num_pages, int) else [int(n) for n in num_pages]
        if len(counts) != len(self.groups):
            raise ValueError(f"num_pages names {len(counts)} groups, the model has {len(self.groups)}")
        for group, count in zip(self.groups, counts):
            if count <= 0:
                raise ValueError("every group needs at least one page")
            group.num_pages = count
            group.allocator = PoolAllocator(count, "page")
            group.table = np.full((self.max_requests, self.max_pages_per_request), -1, dtype=np.int32)
            if allocate_device_memory:
                shape = (len(group.entries), count, group.need.num_kv_heads, self.page_size, group.need.head_dim)
                group.key = torch.zeros(shape, dtype=dtype, device=self.device)
                group.value = torch.zeros(shape, dtype=dtype, device=self.device)
                if self.device.type == "cuda":
                    group.device_table = torch.full((self.max_requests, self.max_pages_per_request), -1,
                                                    dtype=torch.int32, device=self.device)
                else:
                    # a stand-in backend on the host reads the mirror itself: nothing to send
                    group.device_table = torch.from_numpy(group.table)

        # ---- fixed-size state per request
        self.slots = PoolAllocator(self.max_requests, "slot")
        self.state: dict[int, torch.Tensor] = {}
        for entry, need in enumerate(self.needs):
            if isinstance(need, StateNeed) and allocate_device_memory:
                self.state[entry] = torch.zeros((self.max_requests, *need.shape), dtype=need.dtype,
                                                device=self.device)

        # ---- slot records (length, last token, counter, temperature, seed): device + host mirror
        self.slot_mirror = np.zeros((self.max_requests, SLOT_WORDS), dtype=np.int32)
        self.slot_state: torch.Tensor | None = None
        self._new_records: set[int] = set()
        self._unconfirmed: tuple[list[set], set] | None = None    # rows handed out but not yet reported sent
        self._shares_host_memory = self.device.type != "cuda"
        if allocate_device_memory:
            if self._shares_host_memory:
                self.slot_state = torch.from_numpy(self.slot_mirror)
            else:
                self.slot_state = torch.zeros((self.max_requests, SLOT_WORDS), dtype=torch.int32, device=self.device)

        self.requests: dict[str, RequestCache] = {}
        self._step: list[tuple[RequestCache, int]] | None = None
        self._state_backup: tuple[torch.Tensor, dict[int, torch.Tensor]] | None = None

    # ------------------------------------------------------------------ sizing
    def pages_for_lifetime(self, group: CacheGroup, lifetime_tokens: int) -> int:
        """Most pages of ``group`` a request of ``lifetime_tokens`` cached tokens holds at once."""
        full = _ceil_div(lifetime_tokens, self.page_size)
        if group.window is None:
            return full
        live = _ceil_div(group.window - 1 + self.max_step_tokens, self.page_size) + 1
        return min(full, live)

    def lifetime_pages(self, lifetime_tokens: int) -> tuple[int, ...]:
        return tuple(self.pages_for_lifetime(g, lifetime_tokens) for g in self.groups)

    def can_ever_hold(self, lifetime_tokens: int) -> bool:
        if lifetime_tokens > self.max_tokens_per_request:
            return False
        return all(n <= g.num_pages for g, n in zip(self.groups, self.lifetime_pages(lifetime_tokens)))

    # ------------------------------------------------------------------ requests
    def create_request(self, request_id: str, *, lifetime_tokens: int | None = None,
                       temperature: float = 0.0, seed: int = 0) -> RequestCache | None:
        """Register a request and give it a slot.  With ``lifetime_tokens`` its pages are promised
        now; returns None (nothing changed) if the promise cannot be kept or no slot is free.
        ``temperature`` and ``seed`` go into the slot's record for the sampling kernel."""
        if request_id in self.requests:
            raise ValueError(f"request {request_id!r} already has a cache")
        if self.slots.free_count == 0:
            if lifetime_tokens is None:
                raise OutOfPages(f"no free request slot (max_requests={self.max_requests})")
            return None
        promised = [0] * len(self.groups)
        if lifetime_tokens is not None:
            if lifetime_tokens <= 0:
                raise ValueError("lifetime_tokens must be > 0")
            if not self.can_ever_hold(lifetime_tokens):
                raise ValueError(f"request {request_id!r} can never be admitted: it needs "
                                 f"{self.lifetime_pages(lifetime_tokens)} pages per group and "
                                 f"{lifetime_tokens} tokens; the pools hold "
                                 f"{tuple(g.num_pages for g in self.groups)} pages and requests "
                                 f"are limited to {self.max_tokens_per_request} tokens")
            wanted = self.lifetime_pages(lifetime_tokens)
            done = []
            for group, count in zip(self.groups, wanted):
                if not group.allocator.promise(count):
                    for g, c in done:
                        g.allocator.unpromise(c)
                    return None
                done.append((group, count))
            promised = list(wanted)
        slot = self.slots.allocate(1)[0]
        request = RequestCache(request_id, slot,
                               pages=[[] for _ in self.groups],
                               first_live=[0] * len(self.groups),
                               promised=promised,
                               step_new_pages=[[] for _ in self.groups])
        self.requests[request_id] = request
        for tensor in self.state.values():
            tensor[slot].zero_()
        self.slot_mirror[slot] = slot_record(temperature=temperature, seed=seed)
        self._new_records.add(slot)
        return request

    def get(self, request_id: str) -> RequestCache:
        try:
            return self.requests[request_id]
        except KeyError:
            raise KeyError(f"request {request_id!r} has no cache") from None

    def release(self, request_id: str) -> dict[int, list[int]]:
        """Give back everything the request holds; returns the freed page ids per group."""
        request = self.get(request_id)
        if self._step is not None and any(r is request for r, _ in self._step):
            raise RuntimeError(f"request {request_id!r} is part of the step in flight")
        freed: dict[int, list[int]] = {}
        for group in self.groups:
            ids = [p for p in request.pages[group.index] if p >= 0]
            group.allocator.free(ids, promised=bool(request.promised[group.index]))
            group.allocator.unpromise(request.promised[group.index])
            group.table[request.slot, :] = -1
            group.dirty.add(request.slot)
            freed[group.index] = ids
        self.slots.free([request.slot])
        del self.requests[request_id]
        return freed

    # ------------------------------------------------------------------ the step transaction
    def begin_step(self, entries: Sequence[tuple[str, int]]) -> list[RequestCache]:
        """Make room for ``n`` more tokens of each named request: all pages or none."""
        if self._step is not None:
            raise RuntimeError("the previous step was neither committed nor aborted")
        seen = set()
        plan: list[tuple[RequestCache, int]] = []
        for request_id, count in entries:
            if request_id in seen:
                raise ValueError(f"request {request_id!r} appears twice in one step")
            seen.add(request_id)
            if count <= 0:
                raise ValueError(f"request {request_id!r}: a step must bring at least one token")
            request = self.get(request_id)
            if request.committed + count > self.max_tokens_per_request:
                raise ValueError(f"request {request_id!r} would hold {request.committed + count} tokens, "
                                 f"more than max_tokens_per_request={self.max_tokens_per_request}")
            plan.append((request, count))
        taken: list[tuple[RequestCache, CacheGroup, int, list[int]]] = []   # (request, group, first logical page, ids)
        try:
            for request, count in plan:
                end = request.committed + count
                for group in self.groups:
                    pages = request.pages[group.index]
                    need_pages = _ceil_div(end, self.page_size)
                    missing = need_pages - len(pages)
                    if missing <= 0:
                        continue
                    limit = request.promised[group.index]
                    if limit and request.held(group.index) + missing > limit:
                        raise OutOfPages(f"request {request.request_id!r} would exceed the {limit} pages "
                                         f"promised to it in group {group.index}")
                    new_ids = list(group.allocator.allocate(missing, promised=bool(limit)))
                    taken.append((request, group, len(pages), new_ids))
                    pages.extend(new_ids)
        except OutOfPages:
            for request, group, first, new_ids in reversed(taken):
                pages = request.pages[group.index]
                assert pages[first:] == new_ids
                del pages[first:]
                group.allocator.free(new_ids, promised=bool(request.promised[group.index]))
            raise
        for request, group, first, new_ids in taken:
            group.table[request.slot, first:first + len(new_ids)] = new_ids       # a prompt portion brings a hundred pages
            group.dirty.add(request.slot)
            request.step_new_pages[group.index].extend(new_ids)
        for request, count in plan:
            request.pending = (request.committed, request.committed + count)
        self._step = plan
        if self.state:
            # fixed-size state is overwritten in place by the step: keep what an abort must restore
            index = torch.tensor([request.slot for request, _ in plan], dtype=torch.long, device=self.device)
            self._state_backup = (index, {entry: tensor.index_select(0, index)
                                          for entry, tensor in self.state.items()})
        return [request for request, _ in plan]

    def commit_step(self) -> dict[str, dict[int, list[int]]]:
        """Make the step's tokens visible; windowed groups give back the pages no later position
        can see.  Returns the pages given back, per request and group."""
        if self._step is None:
            raise RuntimeError("no step in flight")
        released: dict[str, dict[int, list[int]]] = {}
        for request, _ in self._step:
            request.committed = request.pending[1]
            request.pending = None
            for group in self.groups:
                request.step_new_pages[group.index] = []
                if group.window is None:
                    continue
                # The next query sits at position `committed` and sees keys > committed - window.
                lowest_needed = request.committed - group.window + 1
                first_needed_page = max(0, lowest_needed) // self.page_size
                pages = request.pages[group.index]
                gone = []
                for logical in range(request.first_live[group.index], min(first_needed_page, len(pages))):
                    if pages[logical] >= 0:
                        gone.append(pages[logical])
                        pages[logical] = -1
                        group.table[request.slot, logical] = -1
                        group.dirty.add(request.slot)
                request.first_live[group.index] = max(request.first_live[group.index],
                                                      min(first_needed_page, len(pages)))
                if gone:
                    group.allocator.free(gone, promised=bool(request.promised[group.index]))
                    released.setdefault(request.request_id, {})[group.index] = gone
            self.slot_mirror[request.slot, 0] = request.committed
        self._step = None
        self._state_backup = None
        return released

    def adopt(self, request_id: str, tokens: int) -> None:
        """Declare that the cache already holds ``tokens`` more tokens of the request: the pages are
        taken and the length is committed as after a step, but no kernel runs; what those positions
        hold is whatever the pools hold.  For caches filled by other means (benchmarks that do not
        want to time a prefill first, a cache restored from elsewhere)."""
        request = self.begin_step([(request_id, tokens)])[0]
        self.commit_step()
        self._new_records.add(request.slot)      # the device learns the new length with the next step

    def abort_step(self) -> None:
        """Forget the step: its tokens never become visible, its new pages go back."""
        if self._step is None:
            raise RuntimeError("no step in flight")
        for request, _ in self._step:
            for group in self.groups:
                new_ids = request.step_new_pages[group.index]
                if new_ids:
                    pages = request.pages[group.index]
                    for page_id in reversed(new_ids):
                        popped = pages.pop()
                        assert popped == page_id
                        group.table[request.slot, len(pages)] = -1
                    group.dirty.add(request.slot)
                    group.allocator.free(new_ids, promised=bool(request.promised[group.index]))
                request.step_new_pages[group.index] = []
            request.pending = None
        if self._state_backup is not None:
            index, saved = self._state_backup
            for entry, rows in saved.items():
                self.state[entry].index_copy_(0, index, rows)
            self._state_backup = None
        self._step = None

    @property
    def step_in_flight(self) -> bool:
        return self._step is not None

    # ------------------------------------------------------------------ what the device must learn
    def take_resident_updates(self) -> list[tuple[torch.Tensor, np.ndarray, np.ndarray]]:
        """Rows of the resident tables that changed since the last call, as snapshots:
        ``(device table, row indices int32 [n], rows int32 [n, width])`` for each block table with
        changed rows and for the slot records of newly admitted requests.  The caller sends them
        and scatters them before the step's first kernel.  Empty when nothing changed, and always
        empty when the device tables share the host's memory.  The caller reports with
        ``resident_updates_sent`` once the rows are on their way; rows handed out but never reported
        (the step failed before it could send them) are handed out again."""
        if self._unconfirmed is not None:
            lost_rows, lost_records = self._unconfirmed
            for group, rows in zip(self.groups, lost_rows):
                group.dirty |= rows
            self._new_records |= lost_records
        self._unconfirmed = ([set(group.dirty) for group in self.groups], set(self._new_records))
        updates = []
        for group in self.groups:
            if group.dirty and group.device_table is not None and not self._shares_host_memory:
                rows = np.fromiter(sorted(group.dirty), dtype=np.int32, count=len(group.dirty))
                updates.append((group.device_table, rows, group.table[rows]))
            group.dirty.clear()
        if self._new_records and self.slot_state is not None and not self._shares_host_memory:
            rows = np.fromiter(sorted(self._new_records), dtype=np.int32, count=len(self._new_records))
            updates.append((self.slot_state, rows, self.slot_mirror[rows].copy()))
        self._new_records.clear()
        return updates

    def resident_updates_sent(self) -> None:
        self._unconfirmed = None

    # ------------------------------------------------------------------ views and numbers
    def entry_pools(self, entry: int) -> tuple[torch.Tensor, torch.Tensor, CacheGroup]:
        group_index, local = self.entry_group[entry]
        group = self.groups[group_index]
        return group.key[local], group.value[local], group

    def slot_mapping(self, group: CacheGroup, request: RequestCache, start: int, count: int) -> np.ndarray:
        """Flat slot (page * page_size + offset) of tokens start..start+count-1."""
        positions = np.arange(start, start + count, dtype=np.int64)
        pages = group.table[request.slot, positions // self.page_size].astype(np.int64)
        if (pages < 0).any():
            raise RuntimeError(f"request {request.request_id!r} has no page for a token it is writing")
        return pages * self.page_size + positions % self.page_size

    def stats(self) -> CacheStats:
        return CacheStats(
            total_pages=tuple(g.num_pages for g in self.groups),
            free_pages=tuple(g.allocator.free_count for g in self.groups),
            held_pages=tuple(g.allocator.held_count for g in self.groups),
            promised_pages=tuple(g.allocator.promised for g in self.groups),
            live_requests=len(self.requests),
            committed_tokens=sum(r.committed for r in self.requests.values()),
            pending_tokens=sum((r.pending[1] - r.pending[0]) if r.pending else 0 for r in self.requests.values()),
            free_slots=self.slots.free_count,
        )

    def check_consistency(self) -> None:
        """Every held page belongs to exactly one request; tables mirror the lists (tests)."""
        for group in self.groups:
            owners: dict[int, str] = {}
            for request in self.requests.values():
                pages = request.pages[group.index]
                for logical, page_id in enumerate(pages):
                    if page_id < 0:
                        continue
                    if page_id in owners:
                        raise AssertionError(f"page {page_id} of group {group.index} is held by "
                                             f"{owners[page_id]!r} and {request.request_id!r}")
                    owners[page_id] = request.request_id
                row = group.table[request.slot]
                if list(row[:len(pages)]) != pages or (row[len(pages):] != -1).any():
                    raise AssertionError(f"block table row of {request.request_id!r} differs from its page list")
            if set(owners) != set(group.allocator.held):
                raise AssertionError(f"group {group.index}: allocator holds {sorted(group.allocator.held)}, "
                                     f"requests hold {sorted(owners)}")
            if group.allocator.free_count + group.allocator.held_count != group.num_pages:
                raise AssertionError("free + held != total")
