"""Interfaces and registries of the parts a decoder is put together from.

A part is built from a ``PartSpec`` (its sizes and constants), names the checkpoint tensors it
needs, receives them, and computes on the rows of one step.  Five kinds exist:

* ``mixer``            mixes information between positions (attention here); may own cache
* ``feed_forward``     works on each row alone (dense here; experts elsewhere)
* ``norm``             normalises rows; also offers the fused "add to the residual, then norm"
* ``position``         position encoding, used by a mixer as a component
* ``embedding`` / ``head``  token ids to rows, rows to logits

plus ``block``, the arrangement of a layer's parts.  A part never learns which model it is in;
an architecture is only a function from its configuration to a ``ModelSpec``.  New kinds are
added with ``register_part`` from anywhere, without touching this package.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping

import torch

from ..config.spec import PartSpec

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "embedding", "head", "block")


@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part needs.

    ``init`` tells the random-weights mode how to fill it: ``matrix`` ~ N(0, 0.02),
    ``norm`` ~ 1 + N(0, 0.02), ``bias`` ~ N(0, 0.02), ``table`` = integers below ``high``.
    ``storage`` is what the checkpoint stores: ``float`` (bfloat16 unless the checkpoint holds
    32-bit, which is kept) or ``int`` (kept as int32).
    """

    shape: tuple[int, ...]
    init: str = "matrix"
    storage: str = "float"
    high: int = 0
    optional: bool = False


@dataclass(frozen=True)
class KVCacheNeed:
    """The mixer wants keys and values of its past positions: all of them, or a window."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """The mixer wants a fixed-size tensor per live request (shape without the slot axis)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Base of all parts.  ``compute_dtype`` is float32 or bfloat16 for the whole model."""

    category = ""
    # True if forward() only launches kernels whose arguments are device buffers of the step
    # context (no host-side dependence on the batch's contents): such a part can be captured
    # into a CUDA graph and replayed for other batches of the same shape.
    graph_safe = False

    def __init__(self, spec: PartSpec, compute_dtype: torch.dtype) -> None:
        self.spec = spec
        self.args = dict(spec.args)
        self.prefix = spec.prefix
        self.compute_dtype = compute_dtype

    # -- weights
    def tensors(self) -> dict[str, TensorSpec]:
        """Checkpoint name -> what is expected there."""
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        """Take the tensors named by ``tensors()`` (as stored, on the CPU) and keep what the
        kernels need on ``device``."""

    # -- helpers for subclasses
    def _to_compute(self, tensor: torch.Tensor, device: torch.device) -> torch.Tensor:
        return tensor.to(device=device, dtype=self.compute_dtype).contiguous()

    def _keep_precision(self, tensor: torch.Tensor, device: torch.device) -> torch.Tensor:
        """32-bit stays 32-bit; anything narrower goes to the compute dtype."""
        if tensor.dtype == torch.float32:
            return tensor.to(device=device).contiguous()
        return self._to_compute(tensor, device)


class Norm(Part):
    category = "norm"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def fold(self) -> tuple[torch.Tensor, float] | None:
        """If this norm is "scale each row by rsqrt(mean(x^2) + eps), then multiply by a weight":
        hand out (weight, eps) and from now on apply the row scale only - the caller multiplies
        the weight into the matrix that follows.  None if the norm cannot be expressed so."""
        return None

    def add_forward(self, residual: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        """residual += delta in place; returns norm(residual)."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Used by a mixer as a component: it turns q and k by their positions and stores k and v."""

    category = "position"

    def rotate_and_store(self, qkv: torch.Tensor, ctx, view, num_heads: int, num_kv_heads: int,
                         head_dim: int, write_kv: bool) -> torch.Tensor:
        """Apply the encoding to the q and k heads packed in ``qkv`` at the rows' positions,
        store k and v into the cache view's pages, return q [rows, heads*head_dim]."""
        raise NotImplementedError

    def rotary_frequencies(self) -> torch.Tensor | None:
        """If the encoding is "turn pair (i, i + head_dim/2) by position * f[i]": the float32
        frequencies f [head_dim/2] on the device, which lets a mixer use kernels that rotate, store
        and attend in one launch.  None (the default) for any other encoding; the mixer then calls
        ``rotate_and_store`` and its attention kernel one after the other."""
        return None


class Mixer(Part):
    category = "mixer"
    # A part that sets this implements ``absorb_input_norm`` and accepts ``raw_input=`` and
    # ``residual=`` in forward: the block may hand it the un-normalised stream (the part applies the
    # row scale inside its first product) and let it add its output into the stream in place.
    supports_norm_fusion = False
    # Mixers whose kernels need host-made work lists name them here; mixers with equal keys share
    # one list per step.  The step function calls ``step_plan`` once per key and step, sends the
    # arrays with its own metadata and hands the device copies back in ``ctx.plans[plan_key]``.
    plan_key: str | None = None

    def cache_need(self) -> KVCacheNeed | StateNeed | None:
        return None

    def step_plan(self, host) -> tuple[dict, dict]:
        """``host`` (``HostBatch``): rows, first row and first position of every request of the
        step.  Returns (int32/int64/float32 numpy arrays by name, plain counts by name)."""
        return {}, {}

    def forward(self, x: torch.Tensor, ctx, view, writes_cache: bool) -> torch.Tensor:
        """x: [rows, hidden] of this step; ``view`` is this run step's cache entry."""
        raise NotImplementedError

    def absorb_input_norm(self, weight: torch.Tensor, eps: float) -> None:
        """Multiply the preceding norm's weight into the input projection."""
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"
    supports_norm_fusion = False

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError

    def absorb_input_norm(self, weight: torch.Tensor, eps: float) -> None:
        raise NotImplementedError


class Embedding(Part):
    category = "embedding"

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    category = "head"

    def forward(self, x: torch.Tensor, embedding: Embedding) -> torch.Tensor:
        """Rows [m, hidden] -> float32 logits [m, vocab]."""
        raise NotImplementedError


class Block:
    """Arrangement of one layer's parts; owns no tensors of its own."""

    category = "block"

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, feed_forward_norm: Norm,
                 extras: Mapping[str, Part] | None = None):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        self.extras = dict(extras or {})      # further parts the layer's spec names (``LayerSpec.extra_parts``)

    def parts(self) -> tuple[Part, ...]:
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward, *self.extras.values())

    def finish_load(self, compute_dtype: torch.dtype) -> None:
        """Called once all four parts hold their tensors; an arrangement may fuse across them."""

    def forward(self, residual: torch.Tensor, pending: torch.Tensor | None, ctx, view,
                writes_cache: bool) -> tuple[torch.Tensor, torch.Tensor | None]:
        """Takes and returns (residual stream, output not yet added to it)."""
        raise NotImplementedError


_REGISTRY: dict[str, dict[str, Callable[..., Any]]] = {category: {} for category in CATEGORIES}


def register_part(category: str, kind: str, factory: Callable[..., Any], *, replace: bool = False) -> None:
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category {category!r}; categories: {', '.join(CATEGORIES)}")
    if kind in _REGISTRY[category] and not replace:
        raise ValueError(f"{category} {kind!r} is already registered")
    _REGISTRY[category][kind] = factory


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY[category].pop(kind, None)


def part_factory(category: str, kind: str) -> Callable[..., Any]:
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(category, {}))) or "none"
        raise KeyError(f"no {category} named {kind!r} is registered (known: {known})") from None


def build_part(category: str, spec: PartSpec, compute_dtype: torch.dtype) -> Part:
    return part_factory(category, spec.kind)(spec, compute_dtype)


def known_parts(category: str) -> tuple[str, ...]:
    return tuple(sorted(_REGISTRY[category]))
