"""The step function: one ragged batch of (request, its next tokens) through the model.

A step brings, for every request in it, the tokens that follow what the cache already holds for
that request: a portion of a prompt of any length, or one decoded token.  All of them run as one
batch, reading earlier tokens from the cache only, and the logits at the wanted places come back.

The reference needs two model calls for this, a packed prefill that only works on empty caches
and a batched one-token decode (src/mini_llm_runtime/engine.py:186-248,
qwen_model_runner.py:296-376,447-508); row order here follows the order of the entries, as the
reference's result rows follow scheduler item order (engine.py:256-261).  The step is atomic like
the reference's: pages are taken for all requests or none, and a failure anywhere leaves every
request's visible length unchanged (paged_batch.py:89-114, engine.py:249-254).

What the step function knows: segments (which rows belong to which request), positions, slots and
wanted rows.  It knows nothing of attention: work lists that a mixer's kernels need are made by
the mixer (``Mixer.step_plan``) and travel opaquely in the step's one metadata buffer.

What crosses to the device per step.  Block tables and slot records live on the device (the cache
manager owns them); only rows that changed are sent.  A mixed step sends one packed buffer (token
ids, positions, the segment table, the places of new keys and values, work lists, changed rows).
A step of decoded tokens only is described by the slots of its requests: a first small kernel
derives positions, input tokens (the ones the sampling kernel stored) and cache places from the
slot records, so a captured decode step is replayed without sending anything unless the set of
requests changed, the host supplies the tokens, or a request crossed into a new page.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager, RequestCache
from ..models.decoder import DecoderModel


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places whose logits are wanted."""

    request_id: str
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class Segment:
    request_id: str
    slot: int
    row_start: int
    length: int
    position_start: int


@dataclass
class HostBatch:
    """The step's shape as the host knows it before anything is sent: one entry per request."""

    lengths: np.ndarray          # int32: rows each request brings
    row_start: np.ndarray        # int32: its first row in the packed batch
    position_start: np.ndarray   # int32: position of its first row
    num_rows: int

    @property
    def num_segments(self) -> int:
        return int(self.lengths.shape[0])


@dataclass
class CacheView:
    """What a mixer sees of its cache entry during one step."""

    entry: int
    k_pool: torch.Tensor | None = None       # [pages, kv_heads, page_size, head_dim]
    v_pool: torch.Tensor | None = None
    slots: torch.Tensor | None = None        # int64 [rows]: where each row's k and v go
    block_table: torch.Tensor | None = None  # int32 [request slots, pages per request]; row = the request's slot
    page_size: int = 0
    window: int | None = None
    state: torch.Tensor | None = None        # [request slots, ...] for a fixed-size-state entry
    group: int = -1                          # entries of one group share pages, table and ``shared``
    shared: dict = field(default_factory=dict)   # per step and group: mixers may keep derived objects here


@dataclass
class StepContext:
    """Everything the parts may read about the running step."""

    ops: object
    num_rows: int
    num_wanted: int
    segments: list[Segment]
    token_ids: torch.Tensor          # int32 [rows]
    positions: torch.Tensor          # int32 [rows]
    wanted_rows: torch.Tensor        # int32 [wanted]
    seg_q_start: torch.Tensor        # int32 [segments]: first row of each request
    seg_q_len: torch.Tensor          # int32 [segments]: its rows
    seg_pos0: torch.Tensor           # int32 [segments]: position of its first row
    seg_slot: torch.Tensor           # int32 [segments]: its slot (row of resident tables and state)
    max_q_len: int = 0
    max_kv_len: int = 0
    views: dict[int, CacheView] = field(default_factory=dict)
    plans: dict = field(default_factory=dict)       # plan key -> (device arrays by name, counts by name)
    wanted_all_rows: bool = False    # wanted_rows is 0, 1, .., rows-1 (a decode step): no gather needed
    wanted_slot: torch.Tensor | None = None     # int32 [wanted]: slot of each wanted row's request (sampling)

    @property
    def num_segments(self) -> int:
        return len(self.segments)

    @property
    def segment_slots(self) -> torch.Tensor:
        return self.seg_slot

    def cache_view(self, entry: int) -> CacheView:
        return self.views[entry]


class _PinnedRing:
    """A few pinned staging buffers used in turn; a buffer is reused only after the copy that
    read it has finished."""

    def __init__(self, device: torch.device, depth: int = 4) -> None:
        self.device = device
        self.depth = depth
        self.buffers: list[torch.Tensor | None] = [None] * depth
        self.events: list[torch.cuda.Event | None] = [None] * depth
        self.cursor = 0
        self.pinned = device.type == "cuda"

    def stage(self, nbytes: int) -> tuple[torch.Tensor, int]:
        index = self.cursor
        self.cursor = (self.cursor + 1) % self.depth
        if self.events[index] is not None:
            self.events[index].synchronize()
        buffer = self.buffers[index]
        if buffer is None or buffer.numel() < nbytes:
            size = max(1 << 16, 1 << (nbytes - 1).bit_length())
            buffer = torch.empty(size, dtype=torch.uint8, pin_memory=self.pinned)
            self.buffers[index] = buffer
        return buffer, index

    def sent(self, index: int) -> None:
        if self.pinned:
            event = self.events[index] or torch.cuda.Event()
            event.record()
            self.events[index] = event


class _Packer:
    """Lays numpy arrays out in one byte buffer at 16-byte aligned offsets."""

    def __init__(self) -> None:
        self.items: list[tuple[str, np.ndarray, int]] = []
        self.size = 0

    def add(self, name: str, array: np.ndarray) -> None:
        array = np.ascontiguousarray(array)
        self.items.append((name, array, self.size))
        self.size += (array.nbytes + 15) // 16 * 16


@dataclass
class _CapturedStep:
    """A decode step of one batch size as a CUDA graph.  Its metadata buffer has a fixed layout;
    the first bytes hold what the host may have to refresh: the requests' slots, then the input
    tokens (only when the host supplies them)."""

    metadata: torch.Tensor
    graph: "torch.cuda.CUDAGraph | None" = None
    logits: torch.Tensor | None = None
    tokens: torch.Tensor | None = None
    launches: int = 0                      # kernels in the graph
    slots_now: tuple[int, ...] = ()        # the slots the device copy currently holds
    stagings: list = field(default_factory=list)     # pinned [2 * batch] int32 buffers with their events
    cursor: int = 0


_TORCH_OF = {np.dtype(np.int32): torch.int32, np.dtype(np.int64): torch.int64,
             np.dtype(np.float32): torch.float32}


class ModelRunner:
    """Owns the model and its cache; ``step`` is the only way tokens reach the model."""

    def __init__(self, model: DecoderModel, cache: CacheManager) -> None:
        if model.device is None:
            raise ValueError("load the model's weights before building a runner")
        self.model = model
        self.cache = cache
        self.device = model.device
        self.vocab_size = model.spec.vocab_size
        self.max_positions = model.spec.max_positions
        self._ring = _PinnedRing(self.device)
        self._device_meta: torch.Tensor | None = None
        self._typed_views: dict[int, tuple] = {}       # by a metadata buffer's address: (the buffer, its typed views)
        self.steps_run = 0
        self.bytes_sent = 0        # host-to-device bytes of all steps so far (metadata and changed rows)
        # Decode-only steps (one token per request, its logits wanted) are captured into CUDA
        # graphs, one per batch size, and replayed: a decode step is some two hundred small
        # kernels, and launching them one by one from the host costs more than running them.
        self.use_graphs = (self.device.type == "cuda"
                           and all(getattr(part, "graph_safe", False) for part in model.parts()))
        self.graph_max_batch = 256
        # A batch size is captured once it has come up this many times: capturing costs tens of
        # milliseconds, which a size that passes by once (requests finishing one after another)
        # never earns back.
        self.graph_capture_after = 3
        self._graphs: dict[tuple[int, bool, bool, int], _CapturedStep] = {}       # (batch, sample, feed, context limit)
        self._graph_seen: dict[tuple[int, bool, bool, int], int] = {}
        self.graph_replays = 0

    # ------------------------------------------------------------------ metadata
    def _upload(self, packer: _Packer, device_buffer: torch.Tensor | None = None) -> dict[str, torch.Tensor]:
        """Copy the packed arrays to the device in one transfer and return views of them.  With
        ``device_buffer`` (a captured graph's own metadata buffer) the views have fixed addresses."""
        nbytes = max(packer.size, 16)
        staging, index = self._ring.stage(nbytes)
        host = staging.numpy()
        for _, array, offset in packer.items:
            host[offset:offset + array.nbytes] = array.view(np.uint8).reshape(-1)
        if device_buffer is None:
            if self._device_meta is None or self._device_meta.numel() < nbytes:
                size = max(1 << 16, 1 << (nbytes - 1).bit_length())
                self._device_meta = torch.empty(size, dtype=torch.uint8, device=self.device)
            device_buffer = self._device_meta
        elif device_buffer.numel() < nbytes:
            raise RuntimeError("a captured step's metadata outgrew its buffer")
        device_buffer[:nbytes].copy_(staging[:nbytes], non_blocking=True)
        self._ring.sent(index)
        self.bytes_sent += nbytes
        # views of the whole buffer by element type, made once per buffer: one slice per array then
        typed = self._typed_views.get(device_buffer.data_ptr())
        if typed is None or typed[0] is not device_buffer:
            typed = (device_buffer, {dtype: device_buffer[:device_buffer.numel() // 8 * 8].view(dtype)
                                     for dtype in set(_TORCH_OF.values())})
            if len(self._typed_views) > 64:
                self._typed_views.clear()
            self._typed_views[device_buffer.data_ptr()] = typed
        out = {}
        for name, array, offset in packer.items:
            size = array.itemsize
            flat = typed[1][_TORCH_OF[array.dtype]][offset // size:(offset + array.nbytes) // size]
            out[name] = flat if array.ndim == 1 else flat.view(array.shape)
        return out

    def _pack_resident_updates(self, packer: _Packer) -> list[tuple[torch.Tensor, str, str]]:
        """Changed rows of the resident tables join the step's buffer; returns what to scatter."""
        pending = []
        for number, (table, rows, values) in enumerate(self.cache.take_resident_updates()):
            packer.add(f"update{number}.rows", rows)
            packer.add(f"update{number}.values", values)
            pending.append((table, f"update{number}.rows", f"update{number}.values"))
        return pending

    def _scatter_resident_updates(self, pending, dev) -> None:
        kernels = ops.current()
        for table, rows, values in pending:
            kernels.scatter_rows(table, dev[rows], dev[values])
        self.cache.resident_updates_sent()

    def _send_resident_updates(self) -> None:
        """The same for a step whose own metadata is not sent (a replayed decode step)."""
        packer = _Packer()
        pending = self._pack_resident_updates(packer)
        if pending:
            self._scatter_resident_updates(pending, self._upload(packer))

    def _host_batch(self, entries: Sequence[StepEntry], requests: list[RequestCache]) -> HostBatch:
        lengths = np.array([len(e.tokens) for e in entries], dtype=np.int32)
        row_start = np.zeros(len(entries), dtype=np.int32)
        np.cumsum(lengths[:-1], out=row_start[1:])
        position_start = np.array([r.pending[0] for r in requests], dtype=np.int32)
        return HostBatch(lengths, row_start, position_start, int(lengths.sum()))

    def _step_plans(self, host: HostBatch) -> dict:
        """Work lists from the mixers, one per plan key (mixers with equal keys share one)."""
        plans = {}
        for block in self.model.blocks:
            key = getattr(block.mixer, "plan_key", None)
            if key is not None and key not in plans:
                plans[key] = block.mixer.step_plan(host)
        return plans

    def _pack(self, entries: Sequence[StepEntry], requests: list[RequestCache], *, want_slots: bool, fixed: bool,
              token_arrays: list | None = None):
        """Lay the step's metadata out on the host.  ``fixed``: the layout of a captured decode step
        (the requests' slots first, then the token ids: what a replay may have to refresh)."""
        cache = self.cache
        host = self._host_batch(entries, requests)
        lengths, row_start, position_start, total = host.lengths, host.row_start, host.position_start, host.num_rows
        if token_arrays is None:
            token_arrays = [None] * len(entries)
        pieces = [np.asarray(e.tokens, dtype=np.int32) if array is None else array
                  for e, array in zip(entries, token_arrays)]
        token_ids = pieces[0] if len(pieces) == 1 else np.concatenate(pieces)
        if len(entries) == 1:
            segment_of_row = np.zeros(total, dtype=np.int32)
            positions = np.arange(position_start[0], position_start[0] + total, dtype=np.int32)
        else:
            segment_of_row = np.repeat(np.arange(len(entries), dtype=np.int32), lengths)
            positions = (np.arange(total, dtype=np.int32) - row_start[segment_of_row]
                         + position_start[segment_of_row]).astype(np.int32)
        wanted = [row_start[i] + np.asarray(e.want, dtype=np.int32) for i, e in enumerate(entries) if len(e.want)]
        wanted_rows = np.concatenate(wanted).astype(np.int32) if wanted else np.zeros(0, dtype=np.int32)
        slots = np.array([r.slot for r in requests], dtype=np.int32)

        packer = _Packer()
        packer.add("seg_slot", slots)
        packer.add("token_ids", token_ids)
        packer.add("positions", positions)
        packer.add("wanted_rows", wanted_rows)
        packer.add("seg_q_start", row_start)
        packer.add("seg_q_len", lengths)
        packer.add("seg_pos0", position_start)
        if want_slots and not fixed:      # in a decode step the wanted rows' slots are the segments' slots
            packer.add("wanted_slot", slots[segment_of_row[wanted_rows]] if len(wanted_rows) else wanted_rows)
        for group in cache.groups:
            places = np.concatenate([
                cache.slot_mapping(group, request, int(position_start[i]), int(lengths[i]))
                for i, request in enumerate(requests)])
            packer.add(f"places{group.index}", places.astype(np.int64))
        plans = self._step_plans(host)
        for key, (arrays, _) in plans.items():
            for name, array in arrays.items():
                packer.add(f"plan.{key}.{name}", array)
        pending = self._pack_resident_updates(packer)
        return packer, host, slots, wanted_rows, plans, pending

    def _build_context(self, entries: Sequence[StepEntry], requests: list[RequestCache], *,
                       want_slots: bool = False, fixed: bool = False, packed=None,
                       device_buffer: torch.Tensor | None = None, token_arrays: list | None = None,
                       kv_limit: int | None = None) -> StepContext:
        """Host-side description of the step, sent to the device.  ``fixed``: a captured decode step
        (contexts as long as the cache allows, so that every kernel plans against the cache's
        capacity); ``device_buffer`` is that graph's own metadata buffer.  ``want_slots`` adds the
        slot of every wanted row (for sampling by slot)."""
        cache = self.cache
        packer, host, slots, wanted_rows, plans, pending = packed or self._pack(
            entries, requests, want_slots=want_slots, fixed=fixed, token_arrays=token_arrays)
        lengths, row_start, position_start, total = host.lengths, host.row_start, host.position_start, host.num_rows
        dev = self._upload(packer, device_buffer)
        self._scatter_resident_updates(pending, dev)

        segments = [Segment(e.request_id, int(slots[i]), int(row_start[i]), int(lengths[i]),
                            int(position_start[i])) for i, e in enumerate(entries)]
        ctx = StepContext(
            ops=ops.current(), num_rows=total, num_wanted=int(wanted_rows.shape[0]), segments=segments,
            token_ids=dev["token_ids"], positions=dev["positions"], wanted_rows=dev["wanted_rows"],
            seg_q_start=dev["seg_q_start"], seg_q_len=dev["seg_q_len"], seg_pos0=dev["seg_pos0"],
            seg_slot=dev["seg_slot"], max_q_len=int(lengths.max()),
            max_kv_len=((kv_limit or cache.max_pages_per_request * cache.page_size) if fixed
                        else int((position_start + lengths).max())),
            wanted_all_rows=(wanted_rows.shape[0] == total
                             and bool((wanted_rows == np.arange(total, dtype=np.int32)).all())))
        if want_slots:
            ctx.wanted_slot = dev["seg_slot"] if fixed else dev["wanted_slot"]
        for key, (arrays, counts) in plans.items():
            ctx.plans[key] = ({name: dev[f"plan.{key}.{name}"] for name in arrays}, counts)
        shared_by_group: dict[int, dict] = {group.index: {} for group in cache.groups}
        for entry, need in enumerate(cache.needs):
            if entry in cache.entry_group:
                k_pool, v_pool, group = cache.entry_pools(entry)
                ctx.views[entry] = CacheView(entry, k_pool, v_pool, dev[f"places{group.index}"],
                                             group.device_table, cache.page_size, group.window,
                                             group=group.index, shared=shared_by_group[group.index])
            else:
                ctx.views[entry] = CacheView(entry, state=cache.state.get(entry))
        return ctx

    # ------------------------------------------------------------------ the step
    def _validate(self, entries: Sequence[StepEntry]) -> list:
        """Check the entries; returns each entry's tokens as an int32 array (converted once: a
        prompt portion is thousands of Python integers), or None for the common decode entry."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        arrays = []
        for entry in entries:
            count = len(entry.tokens)
            if count == 0:
                raise ValueError(f"request {entry.request_id!r}: a step must bring at least one token")
            if count == 1 and type(entry.tokens[0]) is int and 0 <= entry.tokens[0] < self.vocab_size \
                    and len(entry.want) <= 1 and (not entry.want or entry.want[0] == 0):
                if self.cache.get(entry.request_id).committed + 1 > self.max_positions:
                    raise ValueError(f"request {entry.request_id!r} would exceed the model's "
                                     f"{self.max_positions} positions")
                arrays.append(None)           # the common decode entry: nothing more to check
                continue
            tokens = np.asarray(entry.tokens)
            if tokens.dtype.kind not in "iu" or tokens.min() < 0 or tokens.max() >= self.vocab_size:
                raise ValueError(f"request {entry.request_id!r}: token ids must be integers in "
                                 f"[0, {self.vocab_size})")
            arrays.append(tokens.astype(np.int32, copy=False))
            for place in entry.want:
                if not 0 <= int(place) < count:
                    raise ValueError(f"request {entry.request_id!r}: wanted place {place} is outside "
                                     f"its {count} tokens")
            held = self.cache.get(entry.request_id).committed
            if held + count > self.max_positions:
                raise ValueError(f"request {entry.request_id!r} would reach {held + count} positions, "
                                 f"the model allows {self.max_positions}")
        return arrays

    def _forward(self, ctx: StepContext, sample: bool, *, lengths_by_device: bool):
        """The model, then the choice of tokens, then the slots' new lengths.  ``lengths_by_device``:
        every request brought one token and the device's own lengths are advanced by one (inside the
        sampling kernel when it runs); otherwise they are set from the host's figures."""
        kernels = ctx.ops
        state = self.cache.slot_state
        logits = self.model.forward(ctx)
        tokens = None
        if sample:
            tokens = kernels.sample_slots(logits, ctx.wanted_slot, state, advance=lengths_by_device)
        if lengths_by_device:
            if not sample:
                kernels.advance_slots(ctx.seg_slot, state)
        else:
            kernels.advance_slots(ctx.seg_slot, state, ctx.seg_q_len, ctx.seg_pos0)
        return logits, tokens

    # A captured step plans its kernels against a context limit, not against the contexts of the
    # step it was captured in.  The limits: the first of these that no request exceeds (kernels may
    # then choose plans that only pay for such contexts: the decode attention sizes the thread-block
    # clusters that merge its chunks by it), else the cache's capacity per request.
    CONTEXT_LIMITS = (1024, 1536, 2048, 4096)

    def _context_limit(self, requests: list[RequestCache]) -> int:
        capacity = self.cache.max_pages_per_request * self.cache.page_size
        longest = max(r.pending[1] for r in requests)
        for limit in self.CONTEXT_LIMITS:
            if limit >= capacity:
                break
            if longest <= limit:
                return limit
        return capacity

    def _graph_eligible(self, entries: Sequence[StepEntry], requests: list[RequestCache], sample: bool, feed: bool) -> bool:
        if not (self.use_graphs and len(entries) <= self.graph_max_batch
                and isinstance(ops.current(), ops.CudaOps)
                and all(len(e.tokens) == 1 and len(e.want) == 1 for e in entries)):
            return False
        key = (len(entries), sample, feed, self._context_limit(requests))
        if key in self._graphs:
            return True
        seen = self._graph_seen.get(key, 0) + 1
        self._graph_seen[key] = seen
        return seen >= self.graph_capture_after

    def _prepare_decode(self, ctx: StepContext, feed: bool) -> None:
        """Positions, cache places and (with ``feed``) input tokens of a decode step, derived on the
        device from the slot records; one launch per cache group."""
        kernels = ctx.ops
        state = self.cache.slot_state
        first = True
        for group in self.cache.groups:
            places = next(view.slots for view in ctx.views.values() if view.group == group.index)
            kernels.decode_prepare(ctx.seg_slot, state,
                                   token_ids=ctx.token_ids if (feed and first) else None,
                                   positions=ctx.positions if first else None,
                                   seg_pos0=ctx.seg_pos0 if first else None,
                                   table=group.device_table, page_size=self.cache.page_size, kv_slots=places)
            first = False
        if first:      # a model without paged groups still needs positions and tokens
            kernels.decode_prepare(ctx.seg_slot, state, token_ids=ctx.token_ids if feed else None,
                                   positions=ctx.positions, seg_pos0=ctx.seg_pos0)

    def _graph_step(self, entries, requests, sample: bool, feed: bool):
        """A decode-only step through the captured graph of its batch size.  The first step of a
        size runs eagerly on the graph's fixed buffers and is then captured; later steps refresh at
        most the slots and the host's tokens, send changed table rows, and replay."""
        count = len(entries)
        key = (count, sample, feed, self._context_limit(requests))
        captured = self._graphs.get(key)
        slots = tuple(r.slot for r in requests)
        if captured is not None and captured.graph is not None:
            self._send_resident_updates()
            refresh_slots = slots != captured.slots_now
            if refresh_slots or not feed:
                staging = captured.stagings[captured.cursor]
                captured.cursor = (captured.cursor + 1) % len(captured.stagings)
                buffer, event = staging
                if event is not None:
                    event.synchronize()
                view = buffer.numpy().view(np.int32)
                aligned = (count * 4 + 15) // 16 * 4       # token ids start at the next 16-byte boundary
                view[:count] = slots
                nbytes = count * 4
                if not feed:
                    view[aligned:aligned + count] = np.fromiter((e.tokens[0] for e in entries), np.int32, count)
                    nbytes = (aligned + count) * 4
                captured.metadata[:nbytes].copy_(buffer[:nbytes], non_blocking=True)
                self.bytes_sent += nbytes
                if event is None:
                    staging[1] = event = torch.cuda.Event()
                event.record()
                captured.slots_now = slots
            captured.graph.replay()
            self.graph_replays += 1
            return captured.logits, captured.tokens

        # first time at this size: give the graph its own buffer for the step's layout, run the
        # step eagerly on it, then capture
        packed = self._pack(entries, requests, want_slots=sample, fixed=True)
        captured = _CapturedStep(torch.empty(packed[0].size + 64, dtype=torch.uint8, device=self.device))
        captured.stagings = [[torch.empty((2 * count + 8) * 4, dtype=torch.uint8, pin_memory=True), None]
                             for _ in range(3)]
        ctx = self._build_context(entries, requests, want_slots=sample, fixed=True, packed=packed,
                                  device_buffer=captured.metadata, kv_limit=key[3])
        self._graphs[key] = captured
        captured.slots_now = slots
        self._prepare_decode(ctx, feed)
        logits, tokens = self._forward(ctx, sample, lengths_by_device=True)     # this step's real result
        torch.cuda.synchronize(self.device)
        # Capturing runs nothing: the records keep the lengths this step gave them.
        graph = torch.cuda.CUDAGraph()
        from ..ops import cuda_ops
        before = cuda_ops.launches
        with torch.cuda.graph(graph):
            self._prepare_decode(ctx, feed)
            captured.logits, captured.tokens = self._forward(ctx, sample, lengths_by_device=True)
        captured.launches = cuda_ops.launches - before
        captured.graph = graph
        return logits, tokens

    def launches_per_replay(self, batch: int, sampling: bool, feed: bool | None = None) -> int:
        """Kernels one replay of the captured step of this batch size launches (0 if not captured)."""
        for (count, sample, fed, _), captured in self._graphs.items():
            if count == batch and sample == sampling and (feed is None or fed == feed) and captured.graph is not None:
                return captured.launches
        return 0

    def check_device(self) -> None:
        """Raise if a kernel reported, through its error word, that a bounded wait ran out since the
        last check.  To be called where the host has just synchronised with the device."""
        check = getattr(ops.current(), "raise_if_device_error", None)
        if check is not None:
            check()

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry], *, sample: bool = False, borrow: bool = False,
             feed: bool = False):
        """Run the entries as one batch.  Returns float32 logits [wanted places, vocab] on the
        device, in the order of the entries and of each entry's ``want``.  With ``sample`` it
        returns ``(logits, tokens)``: one int32 token per wanted place (at most one per request),
        chosen on the device with the temperature, seed and counter of the request's slot record,
        which also receives the token.  ``borrow=True`` may return buffers that the next step
        overwrites (no copy is made).  ``feed=True``: every entry holds one placeholder token and the
        real input is the token the request sampled last, taken from its slot record on the device
        without the host having seen it."""
        token_arrays = self._validate(entries)
        if feed and any(len(e.tokens) != 1 for e in entries):
            raise ValueError("feed needs entries of exactly one token each")
        if sample and any(len(e.want) > 1 for e in entries):
            raise ValueError("sampling takes at most one wanted place per request")
        requests = self.cache.begin_step([(e.request_id, len(e.tokens)) for e in entries])
        try:
            if self._graph_eligible(entries, requests, sample, feed):
                logits, tokens = self._graph_step(entries, requests, sample, feed)
                if not borrow:
                    logits = logits.clone()
                    tokens = tokens.clone() if tokens is not None else None
            else:
                ctx = self._build_context(entries, requests, want_slots=sample, token_arrays=token_arrays)
                if feed:
                    ctx.ops.decode_prepare(ctx.seg_slot, self.cache.slot_state, token_ids=ctx.token_ids)
                logits, tokens = self._forward(ctx, sample, lengths_by_device=False)
        except BaseException:
            self.cache.abort_step()
            raise
        self.cache.commit_step()
        self.steps_run += 1
        return (logits, tokens) if sample else logits
