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

Host-side work per step is one packed metadata buffer (token ids, positions, segment table,
attention tiles, per-group slot mapping and block tables) written into pinned memory and sent
with a single host-to-device copy.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheGroup, CacheManager, RequestCache
from ..models.decoder import DecoderModel
from ..ops.cuda_ops import AttentionBatch

ROWS_PER_TILE = 16    # rows one CTA of the generic attention kernel handles
WIDE_TILE_ROWS = 64   # rows one CTA of the tensor-core prefill kernel handles
BIG_TILE_ROWS = 128   # rows of one work item of the tcgen05 prefill kernel


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places whose logits are wanted."""

    request_id: str
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class SamplingRows:
    """Per wanted row: temperature (0 = greedy), the request's seed, and the index of the token
    being produced (the counter of the request's random stream)."""

    temperatures: Sequence[float]
    seeds: Sequence[int]
    token_indices: Sequence[int]


@dataclass
class Segment:
    request_id: str
    slot: int
    row_start: int
    length: int
    position_start: int


@dataclass
class CacheView:
    """What a mixer sees of its cache entry during one step."""

    entry: int
    k_pool: torch.Tensor | None = None     # [pages, kv_heads, page_size, head_dim]
    v_pool: torch.Tensor | None = None
    slots: torch.Tensor | None = None      # int64 [rows]: where each row's k and v go
    batch: AttentionBatch | None = None
    page_size: int = 0
    window: int | None = None
    state: torch.Tensor | None = None      # [max_requests, ...] for a fixed-size-state entry


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
    segment_slots: torch.Tensor      # int32 [segments]: each request's state slot
    views: dict[int, CacheView] = field(default_factory=dict)
    sampling: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None
    wanted_all_rows: bool = False    # wanted_rows is 0, 1, .., rows-1 (a decode step): no gather needed

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
    """A decode step of one batch size as a CUDA graph with its fixed metadata buffer."""

    metadata: torch.Tensor
    graph: "torch.cuda.CUDAGraph | None" = None
    logits: torch.Tensor | None = None
    tokens: torch.Tensor | None = None
    launches: int = 0      # kernels in the graph
    nbytes: int = 0
    token_ids: torch.Tensor | None = None    # the input ids inside ``metadata`` (fixed address)
    # pinned staging buffers with numpy views of every array at its fixed offset, used in turn
    stagings: list = field(default_factory=list)
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
        self._last_layout_bytes = 0
        self._last_layout: list = []
        self.steps_run = 0
        # Decode-only steps (one token per request, its logits wanted) are captured into CUDA
        # graphs, one per batch size, and replayed: a decode step is some two hundred small
        # kernels, and launching them one by one from the host costs more than running them.
        self.use_graphs = (self.device.type == "cuda"
                           and all(getattr(part, "graph_safe", False) for part in model.parts()))
        self.graph_max_batch = 256
        self._graphs: dict[tuple[int, bool], _CapturedStep] = {}
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
        out = {}
        for name, array, offset in packer.items:
            flat = device_buffer[offset:offset + array.nbytes].view(_TORCH_OF[array.dtype])
            out[name] = flat.view(array.shape)
        return out

    def _build_context(self, entries: Sequence[StepEntry], requests: list[RequestCache],
                       sampling: SamplingRows | None = None, *, fixed_width: int | None = None,
                       device_buffer: torch.Tensor | None = None) -> StepContext:
        """Host-side description of the step, sent to the device.  ``fixed_width`` pins the block
        tables' width (and with it the whole buffer layout for a given batch shape), which a
        captured graph needs; ``device_buffer`` is that graph's own metadata buffer."""
        cache = self.cache
        lengths = np.array([len(e.tokens) for e in entries], dtype=np.int32)
        row_start = np.zeros(len(entries), dtype=np.int32)
        np.cumsum(lengths[:-1], out=row_start[1:])
        position_start = np.array([r.pending[0] for r in requests], dtype=np.int32)
        total = int(lengths.sum())

        token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        segment_of_row = np.repeat(np.arange(len(entries), dtype=np.int32), lengths)
        positions = (np.arange(total, dtype=np.int32) - row_start[segment_of_row]
                     + position_start[segment_of_row]).astype(np.int32)
        wanted = [row_start[i] + np.asarray(e.want, dtype=np.int32) for i, e in enumerate(entries) if len(e.want)]
        wanted_rows = np.concatenate(wanted).astype(np.int32) if wanted else np.zeros(0, dtype=np.int32)

        # Attention tiles of at most 16 rows: segments longer than one row first, then the
        # single-row (decode) segments, which a split-KV kernel may take instead.
        decode_seg = np.flatnonzero(lengths == 1).astype(np.int32)
        order = np.concatenate([np.flatnonzero(lengths != 1), decode_seg]).astype(np.int32)
        tiles_per_segment = ((lengths + ROWS_PER_TILE - 1) // ROWS_PER_TILE)[order]
        tile_seg = np.repeat(order, tiles_per_segment)
        tile_first = np.zeros(len(entries), dtype=np.int32)
        np.cumsum(tiles_per_segment[:-1], out=tile_first[1:])
        tile_row0 = ((np.arange(len(tile_seg), dtype=np.int32) - np.repeat(tile_first, tiles_per_segment))
                     * ROWS_PER_TILE).astype(np.int32)

        # tiles of at most 64 rows over the longer segments, for the tensor-core prefill kernel
        longer = np.flatnonzero(lengths != 1).astype(np.int32)
        wide_per_segment = (lengths[longer] + WIDE_TILE_ROWS - 1) // WIDE_TILE_ROWS
        wide_tile_seg = np.repeat(longer, wide_per_segment)
        wide_first = np.zeros(len(longer), dtype=np.int32)
        np.cumsum(wide_per_segment[:-1], out=wide_first[1:])
        wide_tile_row0 = ((np.arange(len(wide_tile_seg), dtype=np.int32) - np.repeat(wide_first, wide_per_segment))
                          * WIDE_TILE_ROWS).astype(np.int32)
        # heaviest first (most keys to walk): the kernel that draws tiles from a queue ends evenly
        if len(wide_tile_seg) > 1:
            keys = position_start[wide_tile_seg] + np.minimum(wide_tile_row0 + WIDE_TILE_ROWS, lengths[wide_tile_seg])
            heavy_first = np.argsort(-keys, kind="stable")
            wide_tile_seg = np.ascontiguousarray(wide_tile_seg[heavy_first])
            wide_tile_row0 = np.ascontiguousarray(wide_tile_row0[heavy_first])

        # and tiles of at most 128 rows, heaviest first, for the tcgen05 prefill kernel
        big_per_segment = (lengths[longer] + BIG_TILE_ROWS - 1) // BIG_TILE_ROWS
        big_tile_seg = np.repeat(longer, big_per_segment)
        big_first = np.zeros(len(longer), dtype=np.int32)
        np.cumsum(big_per_segment[:-1], out=big_first[1:])
        big_tile_row0 = ((np.arange(len(big_tile_seg), dtype=np.int32) - np.repeat(big_first, big_per_segment))
                         * BIG_TILE_ROWS).astype(np.int32)
        if len(big_tile_seg) > 1:
            keys = position_start[big_tile_seg] + np.minimum(big_tile_row0 + BIG_TILE_ROWS, lengths[big_tile_seg])
            heavy_first = np.argsort(-keys, kind="stable")
            big_tile_seg = np.ascontiguousarray(big_tile_seg[heavy_first])
            big_tile_row0 = np.ascontiguousarray(big_tile_row0[heavy_first])

        slots = np.array([r.slot for r in requests], dtype=np.int32)
        kv_end = position_start + lengths
        table_width = fixed_width or max(1, int(-(-int(kv_end.max()) // cache.page_size)))

        packer = _Packer()
        packer.add("token_ids", token_ids)
        packer.add("positions", positions)
        packer.add("wanted_rows", wanted_rows)
        packer.add("seg_q_start", row_start)
        packer.add("seg_q_len", lengths)
        packer.add("seg_pos0", position_start)
        packer.add("seg_slots", slots)
        packer.add("tile_seg", tile_seg)
        packer.add("tile_row0", tile_row0)
        packer.add("decode_seg", decode_seg)
        packer.add("wide_tile_seg", wide_tile_seg)
        packer.add("wide_tile_row0", wide_tile_row0)
        packer.add("big_tile_seg", big_tile_seg)
        packer.add("big_tile_row0", big_tile_row0)
        for group in cache.groups:
            rows_slots = np.concatenate([
                cache.slot_mapping(group, request, int(position_start[i]), int(lengths[i]))
                for i, request in enumerate(requests)])
            packer.add(f"slots{group.index}", rows_slots.astype(np.int64))
            packer.add(f"table{group.index}", group.table[slots, :table_width])
        if sampling is not None:
            if not (len(sampling.temperatures) == len(sampling.seeds) == len(sampling.token_indices)
                    == wanted_rows.shape[0]):
                raise ValueError("sampling needs one temperature, seed and token index per wanted row")
            packer.add("temperatures", np.asarray(sampling.temperatures, dtype=np.float32))
            packer.add("seeds", np.asarray(sampling.seeds, dtype=np.int64))
            packer.add("token_indices", np.asarray(sampling.token_indices, dtype=np.int64))
        dev = self._upload(packer, device_buffer)
        self._last_layout_bytes = packer.size
        self._last_layout = [(name, array.dtype, array.shape, offset, array) for name, array, offset in packer.items]

        segments = [Segment(e.request_id, int(slots[i]), int(row_start[i]), int(lengths[i]),
                            int(position_start[i])) for i, e in enumerate(entries)]
        ctx = StepContext(ops=ops.current(), num_rows=total, num_wanted=int(wanted_rows.shape[0]),
                          segments=segments, token_ids=dev["token_ids"], positions=dev["positions"],
                          wanted_rows=dev["wanted_rows"], segment_slots=dev["seg_slots"],
                          wanted_all_rows=(wanted_rows.shape[0] == total
                                           and bool((wanted_rows == np.arange(total, dtype=np.int32)).all())))
        if sampling is not None:
            ctx.sampling = (dev["temperatures"], dev["seeds"], dev["token_indices"])
        batches = {}
        for group in cache.groups:
            batches[group.index] = AttentionBatch(
                seg_q_start=dev["seg_q_start"], seg_q_len=dev["seg_q_len"], seg_pos0=dev["seg_pos0"],
                block_table=dev[f"table{group.index}"], tile_seg=dev["tile_seg"], tile_row0=dev["tile_row0"],
                num_segments=len(entries), num_tiles=int(tile_seg.shape[0]),
                max_q_len=int(lengths.max()),
                max_kv_len=int(kv_end.max()) if fixed_width is None else fixed_width * cache.page_size,
                decode_seg=dev["decode_seg"], num_decode=int(decode_seg.shape[0]),
                wide_tile_seg=dev["wide_tile_seg"], wide_tile_row0=dev["wide_tile_row0"],
                num_wide_tiles=int(wide_tile_seg.shape[0]),
                big_tile_seg=dev["big_tile_seg"], big_tile_row0=dev["big_tile_row0"],
                num_big_tiles=int(big_tile_seg.shape[0]))
        for entry, need in enumerate(cache.needs):
            if entry in cache.entry_group:
                k_pool, v_pool, group = cache.entry_pools(entry)
                ctx.views[entry] = CacheView(entry, k_pool, v_pool, dev[f"slots{group.index}"],
                                             batches[group.index], cache.page_size, group.window)
            else:
                ctx.views[entry] = CacheView(entry, state=cache.state.get(entry))
        return ctx

    # ------------------------------------------------------------------ the step
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise ValueError("a step needs at least one entry")
        for entry in entries:
            count = len(entry.tokens)
            if count == 0:
                raise ValueError(f"request {entry.request_id!r}: a step must bring at least one token")
            if count == 1 and type(entry.tokens[0]) is int and 0 <= entry.tokens[0] < self.vocab_size \
                    and len(entry.want) <= 1 and (not entry.want or entry.want[0] == 0):
                if self.cache.get(entry.request_id).committed + 1 > self.max_positions:
                    raise ValueError(f"request {entry.request_id!r} would exceed the model's "
                                     f"{self.max_positions} positions")
                continue                      # the common decode entry: nothing more to check
            tokens = np.asarray(entry.tokens)
            if tokens.dtype.kind not in "iu" or tokens.min() < 0 or tokens.max() >= self.vocab_size:
                raise ValueError(f"request {entry.request_id!r}: token ids must be integers in "
                                 f"[0, {self.vocab_size})")
            for place in entry.want:
                if not 0 <= int(place) < count:
                    raise ValueError(f"request {entry.request_id!r}: wanted place {place} is outside "
                                     f"its {count} tokens")
            held = self.cache.get(entry.request_id).committed
            if held + count > self.max_positions:
                raise ValueError(f"request {entry.request_id!r} would reach {held + count} positions, "
                                 f"the model allows {self.max_positions}")

    def _forward(self, ctx: StepContext, sampling: SamplingRows | None):
        logits = self.model.forward(ctx)
        tokens = ctx.ops.sample(logits, *ctx.sampling) if sampling is not None else None
        return logits, tokens

    def _graph_eligible(self, entries: Sequence[StepEntry]) -> bool:
        return (self.use_graphs and len(entries) <= self.graph_max_batch
                and isinstance(ops.current(), ops.CudaOps)
                and all(len(e.tokens) == 1 and len(e.want) == 1 for e in entries))

    def _graph_step(self, entries, requests, sampling, feed=None):
        """A decode-only step through the captured graph of its batch size.  The first step of a
        size runs eagerly on the graph's fixed buffers and is then captured; later steps only
        refresh the metadata buffer and replay.  ``feed``: see ``step``."""
        key = (len(entries), sampling is not None)
        kernels = ops.current()
        captured = self._graphs.get(key)
        # The context is built at the block table's full width, so every kernel plans its grid
        # against the cache's capacity, not against this step's contexts.
        width = self.cache.max_pages_per_request
        if captured is None:
            # learn the layout's size with a throw-away packing, then give the graph its own buffer
            probe = self._build_context(entries, requests, sampling, fixed_width=width)
            del probe
            captured = _CapturedStep(torch.empty(self._last_layout_bytes + 64, dtype=torch.uint8, device=self.device))
            self._graphs[key] = captured
        if captured.graph is not None:
            self._refresh_captured(captured, entries, requests, sampling)
            if feed is not None:
                captured.token_ids.copy_(feed)       # after the metadata copy, before the replay reads it
            captured.graph.replay()
            self.graph_replays += 1
            return captured.logits, captured.tokens
        ctx = self._build_context(entries, requests, sampling, fixed_width=width,
                                  device_buffer=captured.metadata)
        captured.token_ids = ctx.token_ids
        if feed is not None:
            ctx.token_ids.copy_(feed)
        self._prepare_stagings(captured)
        logits, tokens = self._forward(ctx, sampling)          # this step's real result, eagerly
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        from ..ops import cuda_ops
        before = cuda_ops.launches
        with torch.cuda.graph(graph):
            captured.logits, captured.tokens = self._forward(ctx, sampling)
        captured.launches = cuda_ops.launches - before
        captured.graph = graph
        return logits, tokens

    def _prepare_stagings(self, captured: "_CapturedStep") -> None:
        """Pinned copies of the step's metadata layout, each with numpy views of its arrays.  What
        depends only on the batch size (segment table, tiles, wanted rows) is written once."""
        captured.nbytes = max(self._last_layout_bytes, 16)
        captured.stagings = []
        for _ in range(3):
            buffer = torch.empty(captured.nbytes, dtype=torch.uint8, pin_memory=True)
            host = buffer.numpy()
            views = {}
            for name, dtype, shape, offset, array in self._last_layout:
                view = host[offset:offset + array.nbytes].view(dtype).reshape(shape)
                view[...] = array
                views[name] = view
            captured.stagings.append([buffer, views, None])

    def _refresh_captured(self, captured: "_CapturedStep", entries, requests, sampling) -> None:
        """Write what changes from one decode step to the next (tokens, positions, slots, block
        tables, sampling rows) into the next pinned copy and send it in one transfer."""
        staging = captured.stagings[captured.cursor]
        captured.cursor = (captured.cursor + 1) % len(captured.stagings)
        buffer, views, event = staging
        if event is not None:
            event.synchronize()
        count = len(entries)
        cache = self.cache
        views["token_ids"][:] = np.fromiter((e.tokens[0] for e in entries), np.int32, count)
        positions = np.fromiter((r.pending[0] for r in requests), np.int32, count)
        slots = np.fromiter((r.slot for r in requests), np.int32, count)
        views["positions"][:] = positions
        views["seg_pos0"][:] = positions
        views["seg_slots"][:] = slots
        logical = positions // cache.page_size
        offsets = positions - logical * cache.page_size
        for group in cache.groups:
            pages = group.table[slots, logical].astype(np.int64)
            if (pages < 0).any():
                raise RuntimeError("a request has no page for the token it is writing")
            views[f"slots{group.index}"][:] = pages * cache.page_size + offsets
            np.take(group.table, slots, axis=0, out=views[f"table{group.index}"])
        if sampling is not None:
            views["temperatures"][:] = sampling.temperatures
            views["seeds"][:] = sampling.seeds
            views["token_indices"][:] = sampling.token_indices
        captured.metadata[:captured.nbytes].copy_(buffer, non_blocking=True)
        if staging[2] is None:
            staging[2] = torch.cuda.Event()
        staging[2].record()

    def launches_per_replay(self, batch: int, sampling: bool) -> int:
        """Kernels one replay of the captured step of this batch size launches (0 if not captured)."""
        captured = self._graphs.get((batch, sampling))
        return captured.launches if captured is not None and captured.graph is not None else 0

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry], sampling: SamplingRows | None = None, *,
             borrow: bool = False, feed: torch.Tensor | None = None):
        """Run the entries as one batch.  Returns float32 logits [wanted places, vocab] on the
        device, in the order of the entries and of each entry's ``want``.  With ``sampling`` it
        returns ``(logits, tokens)``: one int32 token per wanted place, chosen on the device.
        ``borrow=True`` may return buffers that the next step overwrites (no copy is made).
        ``feed``: int32 device tensor with the input token of every entry (each entry then holds
        exactly one placeholder token): the ids are taken from the device, e.g. from the tokens the
        previous step chose, without the host having seen them."""
        self._validate(entries)
        if feed is not None:
            if any(len(e.tokens) != 1 for e in entries) or feed.shape != (len(entries),) or feed.dtype != torch.int32:
                raise ValueError("feed needs one int32 token per entry and entries of one token each")
        requests = self.cache.begin_step([(e.request_id, len(e.tokens)) for e in entries])
        try:
            if self._graph_eligible(entries):
                logits, tokens = self._graph_step(entries, requests, sampling, feed)
                if not borrow:
                    logits = logits.clone()
                    tokens = tokens.clone() if tokens is not None else None
            else:
                ctx = self._build_context(entries, requests, sampling)
                if feed is not None:
                    ctx.token_ids.copy_(feed)
                logits, tokens = self._forward(ctx, sampling)
        except BaseException:
            self.cache.abort_step()
            raise
        self.cache.commit_step()
        self.steps_run += 1
        return logits if sampling is None else (logits, tokens)
