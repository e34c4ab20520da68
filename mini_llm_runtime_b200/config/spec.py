"""Architecture-neutral description of a decoder: which parts, with which sizes, in which order.

An architecture's typed configuration (for instance ``Qwen2Config``) is turned into a
``ModelSpec`` by the function registered for it.  Everything below the registry (weights,
parts, cache manager, step function) reads only the ``ModelSpec``; no part learns the name
of the model it is in.  Sizes and constants appear here as data, never in code.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part chosen by its registered ``kind`` with the parameters it is built from."""

    kind: str
    args: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""  # tensor-name prefix in the checkpoint, e.g. "model.layers.3.self_attn."


@dataclass(frozen=True)
class LayerSpec:
    """One block: how the parts are arranged (``block``) and which parts they are.  Every block has
    a mixer, a feed-forward and a norm before each; an arrangement that needs more (norms after the
    mixer and the feed-forward, a gate, a second feed-forward) names them in ``extra_parts`` as
    (name, category, spec) and finds them built in ``Block.extras[name]``."""

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    extra_parts: tuple[tuple[str, str, PartSpec], ...] = ()


@dataclass(frozen=True)
class RunStep:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named twice).  ``cache`` names the
    cache entry the mixer uses; two run steps with the same ``cache`` share it, and a step
    with ``writes_cache=False`` only reads what an earlier step wrote there.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    run_order: tuple[RunStep, ...]
    final_norm: PartSpec
    head: PartSpec

    def __post_init__(self) -> None:
        if not self.layers or not self.run_order:
            raise ValueError("a model needs at least one layer and one run step")
        writers: dict[int, int] = {}
        for position, step in enumerate(self.run_order):
            if not 0 <= step.layer < len(self.layers):
                raise ValueError(f"run step {position} names layer {step.layer}, "
                                 f"but the model has {len(self.layers)} layers")
            if step.cache < 0:
                raise ValueError(f"run step {position} has a negative cache entry")
            if step.writes_cache:
                if step.cache in writers:
                    raise ValueError(f"cache entry {step.cache} is written by run steps "
                                     f"{writers[step.cache]} and {position}")
                writers[step.cache] = position
            elif step.cache not in writers:
                raise ValueError(f"run step {position} reads cache entry {step.cache} "
                                 "before any step writes it")
        entries = sorted({step.cache for step in self.run_order})
        if entries != list(range(len(entries))):
            raise ValueError(f"cache entries must be numbered 0..n-1 without gaps, got {entries}")

    @property
    def cache_entries(self) -> int:
        return len({step.cache for step in self.run_order})
