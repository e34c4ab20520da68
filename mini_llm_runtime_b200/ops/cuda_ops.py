"""Python face of the hand-written sm_100a kernels.

Each method checks its arguments (device, dtype, contiguity, shapes), allocates the output with
torch, and calls one ``extern "C"`` entry point on torch's current CUDA stream.  There is no CPU
path and no other backend: tensors that are not on a CUDA device, a library that cannot be
built, or a size a kernel refuses raise an exception.

The reference reaches its one kernel through a similar checked wrapper
(src/mini_llm_runtime/paged_attention_cuda.py:10-73); everything else there is a torch call.
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import numpy as np
import torch

from . import build

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_STATUS_TEXT = {
    -1: "unsupported dtype",
    -2: "a size is zero, negative or inconsistent",
    -3: "a pointer or stride is not aligned as the kernel needs",
    -4: "a size exceeds what this kernel supports",
    -5: "the kernel reported an error through its device flag",
}


class KernelError(RuntimeError):
    pass


launches = 0  # kernels launched through this module since import (bench.py reports the count)


def _check(status: int, what: str) -> None:
    global launches
    if status == 0:
        launches += 1
        return
    if status < 0:
        raise KernelError(f"{what}: refused ({_STATUS_TEXT.get(status, status)})")
    raise KernelError(f"{what}: the launch failed with cudaError_t {status}")


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}") from None


def _need(tensor: torch.Tensor, name: str, dtype: torch.dtype | None = None, dims: int | None = None) -> None:
    if not isinstance(tensor, torch.Tensor) or not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor; this engine has no CPU path")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if dims is not None and tensor.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, got shape {tuple(tensor.shape)}")


def _ptr(tensor: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())


def _stream() -> ctypes.c_void_p:
    """The current stream of the current device (the raw handle: the wrapper object of
    ``torch.cuda.current_stream`` costs microseconds, and a step asks hundreds of times)."""
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


@dataclass
class AttentionBatch:
    """Device-side description of one step's ragged batch for one cache group.

    ``seg_*`` have one entry per request in the step.  ``block_table`` is the group's resident
    table, int32 [request slots, table_width] with -1 where a request holds no page; segment i
    reads row ``seg_slot[i]`` of it.  ``plan`` holds the work lists of the attention kernels
    (``plan_attention`` below builds them on the host, the step function sends them with the rest of
    its metadata) and ``counts`` their lengths.
    """

    seg_q_start: torch.Tensor
    seg_q_len: torch.Tensor
    seg_pos0: torch.Tensor
    seg_slot: torch.Tensor
    block_table: torch.Tensor
    num_segments: int
    max_q_len: int
    max_kv_len: int
    plan: dict
    counts: dict

    @property
    def num_decode(self) -> int:
        return self.counts.get("decode", 0)


# Rows of one work item of the three prompt-attention kernels.
GENERIC_TILE_ROWS = 16    # attention_generic.cu: one CTA
MMA_TILE_ROWS = 64        # attention_mma.cu: one CTA of the mma.sync kernel
TCGEN05_TILE_ROWS = 128   # attention_tcgen05.cu: one work item


def _tiles(lengths: np.ndarray, segments: np.ndarray, rows: int, position_start: np.ndarray | None):
    """Cut the given segments into tiles of at most ``rows`` rows: (segment of each tile, its first
    row).  With ``position_start`` the tiles are ordered heaviest first (most keys to walk), so that
    kernels drawing tiles from a queue end evenly."""
    per_segment = (lengths[segments] + rows - 1) // rows
    tile_seg = np.repeat(segments, per_segment)
    first = np.zeros(len(segments), dtype=np.int32)
    np.cumsum(per_segment[:-1], out=first[1:])
    row0 = ((np.arange(len(tile_seg), dtype=np.int32) - np.repeat(first, per_segment)) * rows).astype(np.int32)
    if position_start is not None and len(tile_seg) > 1:
        keys = position_start[tile_seg] + np.minimum(row0 + rows, lengths[tile_seg])
        heavy_first = np.argsort(-keys, kind="stable")
        tile_seg = np.ascontiguousarray(tile_seg[heavy_first])
        row0 = np.ascontiguousarray(row0[heavy_first])
    return tile_seg.astype(np.int32), row0


def plan_attention(lengths: np.ndarray, position_start: np.ndarray) -> tuple[dict, dict]:
    """Work lists of the attention kernels for a step whose request i brings ``lengths[i]`` rows
    starting at position ``position_start[i]``: int32 arrays by name, and counts by name.

    ``tile_*``: tiles of at most 16 rows, those of segments longer than one row first, so that a
    split-KV kernel may take the one-row segments (``decode_seg``, ``counts["decode"]`` of them)
    instead of the last tiles.  ``wide_*`` / ``big_*``: tiles of 64 / 128 rows over the longer
    segments only, heaviest first."""
    lengths = np.asarray(lengths, dtype=np.int32)
    position_start = np.asarray(position_start, dtype=np.int32)
    if lengths.shape[0] == 1 and lengths[0] > 1:
        # one prompt portion (the common prefill step): its tiles in order, heaviest (= last) first
        # where the general path sorts; a dozen array operations instead of forty
        rows = int(lengths[0])
        arrays, counts = {"decode_seg": np.zeros(0, dtype=np.int32)}, {"decode": 0}
        for prefix, count_name, tile_rows, heavy_first in (("tile", "tiles", GENERIC_TILE_ROWS, False),
                                                           ("wide_tile", "wide", MMA_TILE_ROWS, True),
                                                           ("big_tile", "big", TCGEN05_TILE_ROWS, True)):
            count = -(-rows // tile_rows)
            row0 = np.arange(count, dtype=np.int32) * np.int32(tile_rows)
            arrays[prefix + "_seg"] = np.zeros(count, dtype=np.int32)
            arrays[prefix + "_row0"] = row0[::-1].copy() if heavy_first else row0
            counts[count_name] = count
        return arrays, counts
    decode_seg = np.flatnonzero(lengths == 1).astype(np.int32)
    longer = np.flatnonzero(lengths != 1).astype(np.int32)
    tile_seg, tile_row0 = _tiles(lengths, np.concatenate([longer, decode_seg]).astype(np.int32),
                                 GENERIC_TILE_ROWS, None)
    wide_seg, wide_row0 = _tiles(lengths, longer, MMA_TILE_ROWS, position_start)
    big_seg, big_row0 = _tiles(lengths, longer, TCGEN05_TILE_ROWS, position_start)
    arrays = {"tile_seg": tile_seg, "tile_row0": tile_row0, "decode_seg": decode_seg,
              "wide_tile_seg": wide_seg, "wide_tile_row0": wide_row0,
              "big_tile_seg": big_seg, "big_tile_row0": big_row0}
    counts = {"tiles": int(tile_seg.shape[0]), "decode": int(decode_seg.shape[0]),
              "wide": int(wide_seg.shape[0]), "big": int(big_seg.shape[0])}
    return arrays, counts


class CudaOps:
    """The kernels, as methods.  One instance per process is enough.

    Kernels that need scratch memory (split-K partial tiles, split-KV partial softmax states) share
    per-device buffers owned by this object; calls are ordered by the CUDA stream they run on, so
    one stream at a time may use an instance.
    """

    name = "cuda"
    GEMM_SCRATCH_BYTES = 32 << 20
    GEMM_COUNTERS = 1 << 15
    ATTENTION_COUNTERS = 1 << 16
    # Partial states of the split-KV decode attention.  The buffer is never replaced: captured
    # launches keep its address, so a call that would need more lowers its split count instead.
    ATTENTION_SCRATCH_BYTES = 64 << 20

    def __init__(self) -> None:
        self._workspaces: dict[int, dict[str, torch.Tensor]] = {}
        # Switches for tests and measurements: each takes one kernel family out, and the next one
        # in line (see the dispatch in linear / paged_attention) serves instead.
        self.use_tensor_cores = True
        self.use_decode_kernel = True
        self.use_mma_attention = True
        self.use_fused_swiglu = True
        self.use_skinny = True
        self.use_fused_norm = True
        self.use_tma_attention = True
        self.use_fused_rope = True
        self.use_cluster_merge = True       # chunks of a decode row merge through a cluster's shared memory
        self.split_prefill_items = True     # the tcgen05 prompt attention may cut long items into parts
        # MLR_TCGEN05_ATTENTION=0 in the environment keeps prompt attention on the mma.sync kernels
        self.use_tcgen05_attention = os.environ.get("MLR_TCGEN05_ATTENTION", "1") != "0"
        self.decode_stages = None      # tiles in flight per CTA of the bulk-copy decode kernel (None: its default)
        self.decode_chunk: int | None = None      # None: chosen per call from the batch's shape
        self.decode_max_splits: int | None = None  # None: just enough for the longest context

    def _workspace(self, device: torch.device) -> dict[str, torch.Tensor]:
        index = device.index if device.type == "cuda" and device.index is not None else torch.cuda.current_device()
        if index not in self._workspaces:
            device = torch.device("cuda", index)
            self._workspaces[index] = {
                "gemm_scratch": torch.empty(self.GEMM_SCRATCH_BYTES, dtype=torch.uint8, device=device),
                "gemm_counters": torch.zeros(self.GEMM_COUNTERS, dtype=torch.int32, device=device),
                "attention_counters": torch.zeros(self.ATTENTION_COUNTERS, dtype=torch.int32, device=device),
                "attention_scratch": torch.empty(self.ATTENTION_SCRATCH_BYTES, dtype=torch.uint8, device=device),
                "sm_count": torch.cuda.get_device_properties(device).multi_processor_count,
                # written by a kernel whose bounded wait ran out; read by the host without a copy
                "error_word": torch.zeros(1, dtype=torch.int32).pin_memory(),
                "prefill_queue": torch.zeros(2, dtype=torch.int32, device=device),
                # states of prompt-attention items that are cut into parts, and one counter per item
                "prefill_scratch": torch.empty(64 << 20, dtype=torch.uint8, device=device),
                "prefill_counters": torch.zeros(1 << 16, dtype=torch.int32, device=device),
            }
        return self._workspaces[index]

    def raise_if_device_error(self) -> None:
        """Call after a synchronisation point: raises if a kernel gave up on a bounded wait.  Such
        a kernel may have left its work queue and its split counters half-used, which every later
        launch would trip over, so they are cleared before the exception leaves."""
        for space in self._workspaces.values():
            code = int(space["error_word"][0])
            if code != 0:
                space["error_word"][0] = 0
                for name in ("gemm_counters", "attention_counters", "prefill_queue", "prefill_counters"):
                    space[name].zero_()
                raise KernelError(f"a kernel's bounded wait ran out (code {code}); the results of the "
                                  "steps since the last check are invalid")

    def sm_count(self, device: torch.device) -> int:
        return self._workspace(device)["sm_count"]

    # ------------------------------------------------------------------ elementwise
    def embedding(self, ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        _need(ids, "ids", torch.int32, 1)
        _need(table, "table", dims=2)
        out = torch.empty((ids.shape[0], table.shape[1]), dtype=table.dtype, device=table.device)
        lib = build.load_library("elementwise")
        _check(lib.mlr_embedding(_ptr(ids), _ptr(table), _ptr(out), ids.shape[0], table.shape[1],
                                 table.shape[0], _code(table.dtype), _stream()), "embedding")
        return out

    def gather_rows(self, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        _need(x, "x", dims=2)
        _need(rows, "rows", torch.int32, 1)
        out = torch.empty((rows.shape[0], x.shape[1]), dtype=x.dtype, device=x.device)
        lib = build.load_library("elementwise")
        _check(lib.mlr_gather_rows(_ptr(x), _ptr(rows), _ptr(out), rows.shape[0], x.shape[1],
                                   _code(x.dtype), _stream()), "gather_rows")
        return out

    def rms_norm(self, x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
        """weight * x * rsqrt(mean(x^2) + eps), row by row; without a weight, the normalised row."""
        return self._rms_norm(x, None, weight, eps)

    def add_inplace(self, target: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        """target += delta (float32 add, rounded once)."""
        _need(target, "target")
        _need(delta, "delta", target.dtype)
        if target.shape != delta.shape:
            raise KernelError("add_inplace needs equal shapes")
        lib = build.load_library("elementwise")
        _check(lib.mlr_add_inplace(_ptr(target), _ptr(delta), ctypes.c_longlong(target.numel()),
                                   _code(target.dtype), _stream()), "add_inplace")
        return target

    def fuses_norm(self, rows: int) -> bool:
        """True if products of ``rows`` rows can take an RMS norm (``rms_eps``) and a residual add
        in their own kernel: the few-rows kernel computes the row scale from the fragments it
        holds anyway.  Callers then skip the norm kernel; otherwise they run it first."""
        return self.use_skinny and self.use_fused_norm and 0 < rows <= self.SKINNY_ROWS

    def add_rms_norm(self, residual: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor | None,
                     eps: float) -> torch.Tensor:
        """residual += delta (in place), then the norm of the new residual."""
        _need(delta, "delta", residual.dtype, 2)
        if delta.shape != residual.shape:
            raise KernelError(f"delta {tuple(delta.shape)} and residual {tuple(residual.shape)} differ")
        return self._rms_norm(residual, delta, weight, eps)

    def _rms_norm(self, x, delta, weight, eps):
        _need(x, "x", dims=2)
        if weight is not None:
            _need(weight, "weight", None, 1)
            if weight.dtype != x.dtype and weight.dtype != torch.float32:
                raise KernelError(f"norm weight must be {x.dtype} or float32, got {weight.dtype}")
            if weight.shape[0] != x.shape[1]:
                raise KernelError(f"norm weight has {weight.shape[0]} entries, rows have {x.shape[1]}")
        out = torch.empty_like(x)
        lib = build.load_library("elementwise")
        _check(lib.mlr_rms_norm(_ptr(x), _ptr(delta), _ptr(weight), _ptr(out), x.shape[0], x.shape[1],
                                ctypes.c_float(eps), _code(x.dtype),
                                _code(x.dtype if weight is None else weight.dtype), _stream()), "rms_norm")
        return out

    def swiglu(self, gate_up: torch.Tensor, block: int | None = None) -> torch.Tensor:
        """silu(gate) * up.  Rows hold blocks of ``block`` gate values followed by the ``block`` up
        values of the same outputs; by default one block: [all gates | all ups]."""
        _need(gate_up, "gate_up", dims=2)
        if gate_up.shape[1] % 2 != 0:
            raise KernelError("gate_up rows must hold gate and up halves of equal width")
        inner = gate_up.shape[1] // 2
        block = inner if block is None else int(block)
        if block <= 0 or inner % block:
            raise KernelError(f"the block size {block} does not divide the inner width {inner}")
        out = torch.empty((gate_up.shape[0], inner), dtype=gate_up.dtype, device=gate_up.device)
        lib = build.load_library("elementwise")
        _check(lib.mlr_swiglu(_ptr(gate_up), _ptr(out), ctypes.c_longlong(gate_up.shape[0]), inner, block,
                              _code(gate_up.dtype), _stream()), "swiglu")
        return out

    SWIGLU_BLOCK = 64   # rows of gate, then rows of up, per 128-row weight tile of the fused kernel

    def linear_swiglu(self, x: torch.Tensor, weight: torch.Tensor, block: int,
                      rms_eps: float | None = None) -> torch.Tensor:
        """silu(x Wg^T) * (x Wu^T) where ``weight`` [2*inner, K] interleaves ``block`` gate rows
        with the ``block`` up rows of the same outputs.  One tensor-core kernel when the shapes
        allow (block 64), else the product followed by the activation kernel.  ``rms_eps`` as in
        ``linear``."""
        _need(x, "x", dims=2)
        _need(weight, "weight", x.dtype, 2)
        if x.shape[1] != weight.shape[1] or weight.shape[0] % (2 * block):
            raise KernelError("linear_swiglu: shapes do not fit the interleaved gate/up layout")
        if (self.use_tensor_cores and self.use_fused_swiglu and block == self.SWIGLU_BLOCK
                and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.shape[0] > 0
                and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0):
            if self._skinny_fits(x, weight, swiglu=True):
                return self._linear_skinny(x, weight, None, torch.bfloat16, swiglu=True, rms_eps=rms_eps)
            if rms_eps is not None:
                x = self.rms_norm(x, None, rms_eps)
                rms_eps = None
            out = self._linear_tcgen05(x, weight, None, torch.bfloat16, swiglu=True)
            if out is not None:
                return out
        return self.swiglu(self.linear(x, weight, rms_eps=rms_eps), block)

    def rope_kv_write(self, qkv: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
                      slots: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, num_heads: int,
                      num_kv_heads: int, head_dim: int, write_kv: bool = True) -> torch.Tensor:
        """Rotate q and k by position (rotate-half pairs, angle = position * inv_freq), return
        q [tokens, heads*head_dim] and store rotated k and raw v at ``slots`` of the page pools
        [pages, kv_heads, page_size, head_dim]."""
        _need(qkv, "qkv", dims=2)
        _need(positions, "positions", torch.int32, 1)
        _need(inv_freq, "inv_freq", torch.float32, 1)
        _need(slots, "slots", torch.int64, 1)
        _need(k_pool, "k_pool", qkv.dtype, 4)
        _need(v_pool, "v_pool", qkv.dtype, 4)
        tokens = qkv.shape[0]
        if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
            raise KernelError(f"qkv rows have {qkv.shape[1]} entries, expected "
                              f"{(num_heads + 2 * num_kv_heads) * head_dim}")
        if inv_freq.shape[0] != head_dim // 2 or head_dim % 2:
            raise KernelError("inv_freq must hold head_dim/2 entries and head_dim must be even")
        if positions.shape[0] != tokens or slots.shape[0] != tokens:
            raise KernelError("positions and slots need one entry per token")
        if k_pool.shape != v_pool.shape or k_pool.shape[1] != num_kv_heads or k_pool.shape[3] != head_dim:
            raise KernelError(f"page pools have shape {tuple(k_pool.shape)}, expected "
                              f"[pages, {num_kv_heads}, page_size, {head_dim}]")
        q = torch.empty((tokens, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
        lib = build.load_library("elementwise")
        _check(lib.mlr_rope_kv_write(_ptr(qkv), _ptr(positions), _ptr(inv_freq), _ptr(slots), _ptr(q),
                                     _ptr(k_pool), _ptr(v_pool), tokens, num_heads, num_kv_heads,
                                     head_dim, k_pool.shape[2], int(bool(write_kv)), _code(qkv.dtype),
                                     _stream()), "rope_kv_write")
        return q

    # ------------------------------------------------------------------ resident tables and slot records
    def plan_attention(self, lengths, position_start):
        """Host-side work lists for this object's attention kernels (see ``plan_attention``)."""
        return plan_attention(lengths, position_start)

    def scatter_rows(self, table: torch.Tensor, row_index: torch.Tensor, rows: torch.Tensor) -> None:
        """table[row_index[i]] = rows[i] for int32 tables that stay on the device."""
        _need(table, "table", torch.int32, 2)
        _need(row_index, "row_index", torch.int32, 1)
        _need(rows, "rows", torch.int32, 2)
        if rows.shape != (row_index.shape[0], table.shape[1]):
            raise KernelError("scatter_rows needs one row of the table's width per index")
        _check(build.load_library("elementwise").mlr_scatter_rows(
            _ptr(table), _ptr(row_index), _ptr(rows), row_index.shape[0], table.shape[1], _stream()), "scatter_rows")

    def decode_prepare(self, seg_slot: torch.Tensor, slot_state: torch.Tensor, *, token_ids=None, positions=None,
                       seg_pos0=None, table=None, page_size: int = 0, kv_slots=None) -> None:
        """Fill a decode step's metadata from the slot records of its requests: positions (the slot's
        length), input tokens (the slot's last sampled token) and where the new key and value go."""
        _need(seg_slot, "seg_slot", torch.int32, 1)
        _need(slot_state, "slot_state", torch.int32, 2)
        count = seg_slot.shape[0]
        for name, tensor, dtype in (("token_ids", token_ids, torch.int32), ("positions", positions, torch.int32),
                                    ("seg_pos0", seg_pos0, torch.int32), ("kv_slots", kv_slots, torch.int64)):
            if tensor is not None:
                _need(tensor, name, dtype, 1)
                if tensor.shape[0] != count:
                    raise KernelError(f"{name} needs one entry per segment")
        if kv_slots is not None:
            _need(table, "table", torch.int32, 2)
        _check(build.load_library("elementwise").mlr_decode_prepare(
            _ptr(seg_slot), _ptr(slot_state), count, _ptr(token_ids), _ptr(positions), _ptr(seg_pos0), _ptr(table),
            0 if table is None else table.shape[1], int(page_size), _ptr(kv_slots), _stream()), "decode_prepare")

    def advance_slots(self, seg_slot: torch.Tensor, slot_state: torch.Tensor, seg_q_len=None, seg_pos0=None) -> None:
        """The slots' lengths after a step: pos0 + len where the host's figures are given, else the
        slot's own length plus len (plus one without ``seg_q_len``)."""
        _need(seg_slot, "seg_slot", torch.int32, 1)
        _need(slot_state, "slot_state", torch.int32, 2)
        _check(build.load_library("elementwise").mlr_advance_slots(
            _ptr(seg_slot), _ptr(seg_q_len), _ptr(seg_pos0), seg_slot.shape[0], _ptr(slot_state), _stream()),
            "advance_slots")

    def sample_slots(self, logits: torch.Tensor, row_slot: torch.Tensor, slot_state: torch.Tensor,
                     advance: bool = False) -> torch.Tensor:
        """``sample`` with temperature, seed and counter read from the slot record of each row's
        request; the record receives the token and its counter grows by one (with ``advance`` its
        length too).  A request may own at most one row."""
        _need(logits, "logits", torch.float32, 2)
        _need(row_slot, "row_slot", torch.int32, 1)
        _need(slot_state, "slot_state", torch.int32, 2)
        if row_slot.shape[0] != logits.shape[0]:
            raise KernelError("row_slot needs one entry per logits row")
        tokens = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
        _check(build.load_library("sampling").mlr_sample_slots(
            _ptr(logits), _ptr(row_slot), _ptr(slot_state), _ptr(tokens), logits.shape[0], logits.shape[1],
            int(bool(advance)), _stream()), "sample_slots")
        return tokens

    # ------------------------------------------------------------------ matrix product
    def linear(self, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
               out_dtype: torch.dtype | None = None, rms_eps: float | None = None,
               residual: torch.Tensor | None = None) -> torch.Tensor:
        """x [M,K] times weight [N,K] transposed, plus bias [N].

        ``rms_eps``: the product is taken of the RMS-normalised rows x * rsqrt(mean(x^2) + eps)
        (a norm whose weight has been folded into ``weight``).  ``residual`` [M,N]: the result is
        added into it in place and it is returned.  The few-rows kernel does both itself; for
        other shapes a normalising kernel runs first and an add kernel last."""
        _need(x, "x", dims=2)
        _need(weight, "weight", x.dtype, 2)
        if bias is not None:
            _need(bias, "bias", x.dtype, 1)
            if bias.shape[0] != weight.shape[0]:
                raise KernelError("bias length differs from the weight's output rows")
        if x.shape[1] != weight.shape[1]:
            raise KernelError(f"x has {x.shape[1]} columns, weight expects {weight.shape[1]}")
        out_dtype = out_dtype or x.dtype
        if residual is not None:
            _need(residual, "residual", out_dtype, 2)
            if residual.shape != (x.shape[0], weight.shape[0]):
                raise KernelError("residual must have the shape of the result")
        tensor_cores = (self.use_tensor_cores and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
                        and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and x.shape[0] > 0)
        if tensor_cores and self._skinny_fits(x, weight) and (residual is None or out_dtype == torch.bfloat16):
            return self._linear_skinny(x, weight, bias, out_dtype, swiglu=False, rms_eps=rms_eps, residual=residual)
        if rms_eps is not None:
            x = self.rms_norm(x, None, rms_eps)
        out = self._linear_tcgen05(x, weight, bias, out_dtype) if tensor_cores else None
        if out is None:
            out = self._linear_simt(x, weight, bias, out_dtype)
        return self.add_inplace(residual, out) if residual is not None else out

    # Rows up to which the few-rows kernel is chosen.  It accepts up to 64, but measured on the
    # 0.5B layer sizes it loses to the tcgen05 kernel at 64 rows (3.72 against 3.23 ms per step).
    SKINNY_ROWS = 16
    SKINNY_ROWS_SMALL_WEIGHT = 32     # rows up to which matrices of at most SKINNY_SMALL_WEIGHT elements stay with it
    SKINNY_SMALL_WEIGHT = 2 << 20
    SKINNY_LARGE_WEIGHT = 32 << 20    # elements from which more than SKINNY_LARGE_WEIGHT_ROWS rows go to the tcgen05 kernel
    SKINNY_LARGE_WEIGHT_ONE_ROW = 64 << 20   # the same for a single row (14B sizes, one request: 6.26 -> 6.14 ms per step)
    SKINNY_LARGE_WEIGHT_ROWS = 0
    skinny_one_round = True
    SKINNY_ROUNDS_WEIGHT = 4 << 20    # elements from which a grid of more than one round goes to the tcgen05 kernel
    # Chunks of one decode row and kv head that may form one thread-block cluster, and the longest
    # chunk worth it.  A cluster lies within one GPC, one CTA per SM; with 18 SMs per GPC, 8 GPCs and
    # three CTAs per SM only so many clusters run together, and a launch with more comes in rounds
    # (measured: 32 clusters of 13 CTAs lose to no clusters at all, 32 clusters of 8 win).
    # The smallest of these sizes that leaves a CTA at most CLUSTER_CHUNK keys is taken, else the
    # largest that fits (a step of 8 requests at 0.5B sizes: contexts of 1,024 keys 582 us with
    # clusters of 6, 598 with 8, 624 with 16; contexts of 3,072 keys 661, 653 and 646 us).
    CLUSTER_SIZES = (2, 3, 4, 6, 8, 16)     # 2 and 3: the few chunks of many requests (64 requests, contexts of 1,000: 1.453 -> 1.427 ms)
    CLUSTER_CHUNK = 256
    CLUSTER_MAX_CHUNK = 768

    def clusters_together(self, size: int) -> int:
        """Clusters of ``size`` CTAs that certainly run at once (a tenth below the arithmetic: launches
        right at it measured slower than without clusters)."""
        return 8 * (18 // size) * self.TMA_CTAS_PER_SM * 9 // 10

    TMA_MIN_CHUNK = 256               # keys per CTA of the bulk-copy decode attention, at least
    TMA_CTAS_PER_SM = 3               # its CTAs that are resident at once on one SM

    def _skinny_fits(self, x, weight, swiglu=False) -> bool:
        """Few rows and a weight too small for one 128-row tile per SM: the latency-lean kernel.
        Small matrices (the attention projections of small models) stay with it up to 32 rows:
        measured at 1152 x 896 and 32 rows, 3.0 against 7.1 us; a batch-32 decode step 1.50 -> 1.44 ms.
        (At 64 rows it wins alone, 6.3 against 8.4 us, but loses inside a step: 1.96 -> 2.20 ms.)"""
        rows = x.shape[0]
        # a weight with a 128-row tile for every SM keeps the tcgen05 kernel's tensor-memory tiles busy
        if (not self.use_skinny or weight.shape[0] >= 128 * self.sm_count(x.device)
                or (swiglu and x.shape[1] > 2048)):
            return False
        # Matrices of tens of megabytes go to the tcgen05 kernel at every row count, even with the
        # separate norm and add kernels that path needs: its operands wait in shared memory, not
        # in registers, so its CTAs start beside the kernels before them, while this kernel's
        # 512-thread CTAs for long rows fill a register file each and come in two rounds (7B sizes,
        # 8 rows, down projection inside a step: 51 us against 28; the whole step 4.42 -> 3.77 ms).
        elements = weight.shape[0] * weight.shape[1]
        if rows > self.SKINNY_LARGE_WEIGHT_ROWS and elements >= (self.SKINNY_LARGE_WEIGHT if rows > 1
                                                                 else self.SKINNY_LARGE_WEIGHT_ONE_ROW):
            return False
        if rows <= self.SKINNY_ROWS:
            # Its CTAs keep their operands in registers, so a grid that the device does not hold at once
            # runs in rounds, the last of them nearly empty and as long as the first; with more than
            # one token row such products do better in the tcgen05 kernel once the matrix is more
            # than a few megabytes.  Decode steps, one-round rule off and on: 14B sizes 2 rows 6.43 ->
            # 6.31 ms, 4 rows 6.72 -> 6.55, 8 rows 7.19 -> 6.83, 16 rows 8.50 -> 7.80; 7B sizes 16 rows
            # 3.77 -> 3.64; but 14B sizes 1 row 6.22 -> 6.37 (a single row's x costs no traffic), and the
            # fused gate/up product of the 0.5B sizes at 9 to 16 rows 0.89 -> 0.92 ms.
            if (self.skinny_one_round and rows > 1 and not swiglu and elements >= self.SKINNY_ROUNDS_WEIGHT
                    and self._skinny_rounds(rows, weight.shape[0], weight.shape[1], swiglu) > 1):
                return False
            return True
        return (not swiglu and rows <= self.SKINNY_ROWS_SMALL_WEIGHT
                and weight.shape[0] * weight.shape[1] <= self.SKINNY_SMALL_WEIGHT)

    def _skinny_rounds(self, rows: int, n: int, k: int, swiglu: bool) -> int:
        """Rounds in which the few-rows kernel's CTAs for this product would run on this device."""
        key = (min(rows, 64) if rows > 16 else (8 if rows <= 8 else 16), n, k, bool(swiglu))
        cache = self.__dict__.setdefault("_rounds_cache", {})
        if key not in cache:
            lib = build.load_library("gemm_skinny")
            cache[key] = int(lib.mlr_gemm_skinny_rounds(int(rows), int(n), int(k), int(bool(swiglu))))
        return cache[key]

    def _linear_skinny(self, x, weight, bias, out_dtype, swiglu, rms_eps=None, residual=None):
        M, K = x.shape
        N = weight.shape[0]
        if residual is not None:
            out = residual      # the kernel adds the product into it
        else:
            out = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
        lib = build.load_library("gemm_skinny")
        _check(lib.mlr_gemm_skinny(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), _ptr(residual), M, N, K,
                                   int(out_dtype == torch.float32), int(swiglu),
                                   ctypes.c_float(-1.0 if rms_eps is None else rms_eps), _stream()),
               "linear (few rows)")
        return out

    def _linear_tcgen05(self, x, weight, bias, out_dtype, swiglu=False):
        M, K = x.shape
        N = weight.shape[0]
        lib = build.load_library("gemm_tcgen05")
        lib.mlr_gemm_tcgen05_plan.restype = ctypes.c_longlong
        splits, tiles = ctypes.c_int(0), ctypes.c_int(0)
        need = lib.mlr_gemm_tcgen05_plan(M, N, K, int(swiglu), ctypes.byref(splits), ctypes.byref(tiles))
        space = self._workspace(x.device)
        if need > space["gemm_scratch"].numel() or (splits.value > 1 and tiles.value > space["gemm_counters"].numel()):
            return None
        out = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
        _check(lib.mlr_gemm_tcgen05(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), M, N, K,
                                    int(out_dtype == torch.float32), int(swiglu), _ptr(space["gemm_scratch"]),
                                    _ptr(space["gemm_counters"]), _ptr(space["error_word"]), _stream()),
               "linear (tcgen05)")
        return out

    def _linear_simt(self, x, weight, bias, out_dtype):
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
        lib = build.load_library("linear_simt")
        _check(lib.mlr_linear_simt(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), x.shape[0],
                                   weight.shape[0], x.shape[1], _code(x.dtype), _code(out_dtype),
                                   _stream()), "linear")
        return out

    # ------------------------------------------------------------------ attention
    def rope_paged_attention(self, qkv: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
                             slots: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                             batch: "AttentionBatch", num_heads: int, num_kv_heads: int, head_dim: int,
                             scale: float, window: int | None = None, write_kv: bool = True) -> torch.Tensor:
        """``rope_kv_write`` followed by ``paged_attention``.  A step of decoded tokens only, in
        bfloat16 with a head size and page size the bulk-copy decode kernel takes, runs as that one
        kernel: it rotates q while loading it and stores the new key and value itself."""
        page_size = k_pool.shape[2] if k_pool.dim() == 4 else 0
        group = num_heads // max(1, num_kv_heads)
        fused = (self.use_fused_rope and self.use_mma_attention and self.use_tma_attention
                 and self.decode_chunk is None
                 and qkv.dtype == torch.bfloat16 and head_dim in (64, 128) and group <= 16
                 and "decode_seg" in batch.plan and 0 < batch.num_decode == batch.num_segments
                 and page_size >= 8 and page_size & (page_size - 1) == 0
                 and batch.num_decode * num_kv_heads <= self.ATTENTION_COUNTERS)
        if not fused:
            q = self.rope_kv_write(qkv, positions, inv_freq, slots, k_pool, v_pool, num_heads, num_kv_heads,
                                   head_dim, write_kv)
            return self.paged_attention(q, k_pool, v_pool, batch, num_heads, num_kv_heads, head_dim, scale, window)
        _need(qkv, "qkv", dims=2)
        _need(inv_freq, "inv_freq", torch.float32, 1)
        _need(slots, "slots", torch.int64, 1)
        _need(k_pool, "k_pool", qkv.dtype, 4)
        _need(v_pool, "v_pool", qkv.dtype, 4)
        tokens = qkv.shape[0]
        if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
            raise KernelError("qkv width does not match the head counts")
        if slots.shape[0] != tokens or inv_freq.shape[0] != head_dim // 2 or batch.num_decode != tokens:
            raise KernelError("one slot per token, head_dim/2 frequencies, one decoded token per segment")
        if k_pool.shape[1] != num_kv_heads or k_pool.shape[3] != head_dim or v_pool.shape != k_pool.shape:
            raise KernelError("page pools do not match the head sizes")
        out = torch.empty((tokens, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
        self._decode_attention(None, k_pool, v_pool, out, batch, num_heads, num_kv_heads, head_dim, scale, window,
                               mma=True, rope=(qkv, inv_freq, slots, write_kv))
        return out

    def paged_attention(self, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                        batch: AttentionBatch, num_heads: int, num_kv_heads: int, head_dim: int,
                        scale: float, window: int | None) -> torch.Tensor:
        """Causal attention of every row of the step over its request's cached keys."""
        _need(q, "q", dims=2)
        _need(k_pool, "k_pool", q.dtype, 4)
        _need(v_pool, "v_pool", q.dtype, 4)
        if q.shape[1] != num_heads * head_dim:
            raise KernelError(f"q rows have {q.shape[1]} entries, expected {num_heads * head_dim}")
        if k_pool.shape[1] != num_kv_heads or k_pool.shape[3] != head_dim or k_pool.shape != v_pool.shape:
            raise KernelError(f"page pools have shape {tuple(k_pool.shape)}, expected "
                              f"[pages, {num_kv_heads}, page_size, {head_dim}]")
        if "tile_seg" not in batch.plan:
            raise KernelError("the batch carries no attention work lists (plan_attention)")
        out = torch.empty_like(q)
        plan, counts = batch.plan, batch.counts
        generic_tiles = counts["tiles"]
        group = num_heads // num_kv_heads
        page_size = k_pool.shape[2]
        paged_by_tma = page_size >= 8 and page_size & (page_size - 1) == 0
        common = (_ptr(batch.seg_q_start), _ptr(batch.seg_q_len), _ptr(batch.seg_pos0), _ptr(batch.block_table),
                  _ptr(batch.seg_slot), batch.block_table.shape[1])
        if (self.use_mma_attention and q.dtype == torch.bfloat16 and head_dim in (64, 128) and group <= 16
                and batch.num_decode * num_kv_heads <= self.ATTENTION_COUNTERS):
            if batch.num_decode > 0:
                self._decode_attention(q, k_pool, v_pool, out, batch, num_heads, num_kv_heads, head_dim, scale,
                                       window, mma=True)
            if counts["big"] > 0 and self.use_tcgen05_attention and paged_by_tma:
                # S = Q K^T and P V on tcgen05 with tensor-memory accumulators
                space = self._workspace(q.device)
                _check(build.load_library("attention_tcgen05").mlr_attention_prefill_tcgen05(
                    _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(plan["big_tile_seg"]),
                    _ptr(plan["big_tile_row0"]), *common, counts["big"], q.shape[0], num_heads,
                    num_kv_heads, head_dim, page_size, k_pool.shape[0], int(window or 0), ctypes.c_float(scale),
                    int(batch.max_kv_len), _ptr(space["prefill_queue"]), _ptr(space["error_word"]),
                    _ptr(space["prefill_scratch"] if self.split_prefill_items else None),
                    ctypes.c_longlong(space["prefill_scratch"].numel()),
                    _ptr(space["prefill_counters"]), space["prefill_counters"].numel(), _stream()),
                    "prefill attention (tcgen05)")
            elif counts["wide"] > 0 and self.use_tma_attention and paged_by_tma:
                space = self._workspace(q.device)
                _check(build.load_library("attention_mma").mlr_attention_prefill_tma(
                    _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(plan["wide_tile_seg"]),
                    _ptr(plan["wide_tile_row0"]), *common, counts["wide"], num_heads,
                    num_kv_heads, head_dim, page_size, k_pool.shape[0], int(window or 0), ctypes.c_float(scale),
                    _ptr(space["prefill_queue"]), _ptr(space["error_word"]), _stream()),
                    "prefill attention (TMA)")
            elif counts["wide"] > 0:
                _check(build.load_library("attention_mma").mlr_attention_prefill_mma(
                    _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(plan["wide_tile_seg"]),
                    _ptr(plan["wide_tile_row0"]), *common, counts["wide"], num_heads,
                    num_kv_heads, head_dim, page_size, int(window or 0), ctypes.c_float(scale), _stream()),
                    "prefill attention")
            return out
        if (self.use_decode_kernel and batch.num_decode > 0
                and q.dtype == torch.bfloat16 and head_dim in (64, 128) and group <= 8
                and batch.num_decode * num_kv_heads <= self.ATTENTION_COUNTERS):
            self._decode_attention(q, k_pool, v_pool, out, batch, num_heads, num_kv_heads, head_dim, scale, window)
            generic_tiles -= batch.num_decode
        if generic_tiles > 0:
            _check(build.load_library("attention_generic").mlr_attention_generic(
                _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(plan["tile_seg"]), _ptr(plan["tile_row0"]),
                *common, generic_tiles, num_heads, num_kv_heads, head_dim,
                page_size, int(window or 0), ctypes.c_float(scale), _code(q.dtype), _stream()),
                "paged_attention")
        return out

    def plan_decode(self, num_decode: int, num_kv_heads: int, longest: int, sms: int) -> tuple[int, int]:
        """(chunk, splits): keys per CTA so that the grid has about two CTAs per SM."""
        chunk = 512
        while chunk > 128 and num_decode * num_kv_heads * -(-longest // chunk) < 2 * sms:
            chunk //= 2
        while -(-longest // chunk) > 64:      # the final merge handles at most 64 chunks per request
            chunk *= 2
        return chunk, max(1, -(-longest // chunk))

    def _decode_attention(self, q, k_pool, v_pool, out, batch, num_heads, num_kv_heads, head_dim, scale, window,
                          mma=False, rope=None):
        page_size = k_pool.shape[2]
        space = self._workspace(out.device)
        sms = space["sm_count"]
        tma = mma and self.use_tma_attention and page_size >= 8 and page_size & (page_size - 1) == 0
        even_split = tma and self.decode_chunk is None
        cluster = 0
        # float32 partial states of one split of every (row, head); the scratch buffer is fixed
        per_split = batch.num_decode * num_heads * (head_dim + 2) * 4
        most_splits = space["attention_scratch"].numel() // max(1, per_split)
        if most_splits < 1:
            raise KernelError(f"{batch.num_decode} decode rows of {num_heads} heads do not fit the "
                              f"{space['attention_scratch'].numel() >> 20} MiB of split-KV scratch")
        if even_split:
            # the kernel divides each request's context over `splits` chunks of at least `chunk` keys
            chunk = self.TMA_MIN_CHUNK
            pairs = max(1, batch.num_decode * num_kv_heads)
            resident = self.TMA_CTAS_PER_SM * sms
            # More (request, kv head) pairs than resident CTAs: whole contexts per CTA would leave a
            # second, nearly empty wave; four chunks each even it out (14B sizes, 64 requests:
            # 320 -> 305 us per layer; below that number of pairs, cutting further only costs).
            wanted = resident // pairs if pairs <= resident else 4
            splits = max(1, min(64, most_splits, wanted, -(-batch.max_kv_len // chunk)))
            # Up to 16 chunks can merge through their thread-block cluster's shared memory, which
            # saves several microseconds of global round trips; worth fewer chunks of up to 768 keys.
            for size in self.CLUSTER_SIZES:
                if (self.use_cluster_merge and size <= splits and pairs <= self.clusters_together(size)
                        and (size == splits or batch.max_kv_len <= size * self.CLUSTER_MAX_CHUNK)):
                    cluster = size
                    if batch.max_kv_len <= size * self.CLUSTER_CHUNK:
                        break
            if cluster:
                splits = cluster
        else:
            chunk, splits = self.plan_decode(batch.num_decode, num_kv_heads, batch.max_kv_len, sms)
            if self.decode_chunk is not None:
                chunk = self.decode_chunk
                splits = max(1, -(-batch.max_kv_len // chunk))
            if self.decode_max_splits is not None:
                splits = max(splits, self.decode_max_splits)
            while splits > most_splits:        # longer chunks until the states fit the fixed buffer
                chunk *= 2
                splits = max(1, -(-batch.max_kv_len // chunk))
        if even_split and self.decode_max_splits is not None:
            splits = min(most_splits, max(splits, self.decode_max_splits))
            cluster = 0
        if rope is not None and not tma:
            raise KernelError("the fused position encoding needs the bulk-copy decode kernel")
        qkv, inv_freq, slots, write_kv = rope if rope is not None else (None, None, None, False)
        decode_seg = batch.plan["decode_seg"]
        if tma:
            # pages arrive by the tensor memory accelerator, one bulk copy per page and kv head
            entry = build.load_library("attention_mma").mlr_attention_decode_tma

            # every segment one decoded row: segment and row are the index itself, the kernel skips the list
            listed = None if batch.num_decode == batch.num_segments else decode_seg

            def launch(clustered: bool) -> int:
                return entry(
                    _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(listed), _ptr(batch.seg_q_start),
                    _ptr(batch.seg_pos0), _ptr(batch.block_table), _ptr(batch.seg_slot), batch.block_table.shape[1],
                    batch.num_decode, num_heads, num_kv_heads, head_dim, page_size, k_pool.shape[0], int(window or 0),
                    ctypes.c_float(scale), chunk, int(even_split), splits, stages,
                    _ptr(space["attention_scratch"]), _ptr(space["attention_counters"]), _ptr(space["error_word"]),
                    _ptr(qkv), _ptr(inv_freq), _ptr(slots), int(bool(write_kv)), int(clustered), _stream())

            clustered = cluster == splits and cluster >= 2
            # head_dim 64: a warp that walks more than two 64-key tiles does better with 32-key tiles
            # and two of them in flight (same shared memory; measured 2 to 3 % of a decode step
            # from 24 requests on, slower below, and slower at contexts of 32k)
            stages = int(self.decode_stages or 0)
            if (self.decode_stages is None and head_dim == 64 and batch.max_kv_len <= 8192
                    and -(-batch.max_kv_len // splits) > 2 * self.TMA_MIN_CHUNK):
                stages = 12
            status = launch(clustered)
            if status > 0 and clustered:
                # the device refused clusters of this size (a partitioned GPU, say): the merge through
                # scratch memory serves from now on
                self.use_cluster_merge = False
                status = launch(False)
            _check(status, "decode attention (TMA)")
            return
        entry = (build.load_library("attention_mma").mlr_attention_decode_mma if mma
                 else build.load_library("attention_decode").mlr_attention_decode)
        _check(entry(
            _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(decode_seg), _ptr(batch.seg_q_start),
            _ptr(batch.seg_pos0), _ptr(batch.block_table), _ptr(batch.seg_slot), batch.block_table.shape[1],
            batch.num_decode, num_heads, num_kv_heads, head_dim, k_pool.shape[2], int(window or 0),
            ctypes.c_float(scale), chunk, splits, _ptr(space["attention_scratch"]), _ptr(space["attention_counters"]),
            _stream()),
            "decode attention")

    # ------------------------------------------------------------------ sampling
    def sample(self, logits: torch.Tensor, temperatures: torch.Tensor, seeds: torch.Tensor,
               counters: torch.Tensor) -> torch.Tensor:
        """One token per row of float32 logits: argmax where temperature <= 0, else a draw from
        softmax(logits / temperature) with the uniform number of (seed, counter)."""
        _need(logits, "logits", torch.float32, 2)
        _need(temperatures, "temperatures", torch.float32, 1)
        _need(seeds, "seeds", torch.int64, 1)
        _need(counters, "counters", torch.int64, 1)
        rows = logits.shape[0]
        if not (temperatures.shape[0] == seeds.shape[0] == counters.shape[0] == rows):
            raise KernelError("temperatures, seeds and counters need one entry per logits row")
        tokens = torch.empty((rows,), dtype=torch.int32, device=logits.device)
        lib = build.load_library("sampling")
        _check(lib.mlr_sample(_ptr(logits), _ptr(temperatures), _ptr(seeds), _ptr(counters), _ptr(tokens),
                              rows, logits.shape[1], _stream()), "sample")
        return tokens
