"""A decoder put together from a ``ModelSpec``: embedding, blocks in their run order, final norm,
head.  This class is the same for every architecture; what differs is the spec.

It corresponds to the reference's ``QwenPrefillRunner`` (src/mini_llm_runtime/qwen_model_runner.py:
227-508) with its four entry points (prefill, prefill_batch, decode_one, decode_batch) replaced by
one ``forward`` over a ragged step batch.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.spec import ModelSpec
from ..parts.base import Block, KVCacheNeed, StateNeed, TensorSpec, build_part, part_factory
from ..weights.loader import check_tensors


class DecoderModel:
    def __init__(self, spec: ModelSpec, compute_dtype: torch.dtype) -> None:
        if compute_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("the model computes in float32 or bfloat16")
        self.spec = spec
        self.compute_dtype = compute_dtype
        self.embedding = build_part("embedding", spec.embedding, compute_dtype)
        self.blocks: list[Block] = []
        for layer in spec.layers:
            block_cls = part_factory("block", layer.block)
            extras = {name: build_part(category, part_spec, compute_dtype)
                      for name, category, part_spec in layer.extra_parts}
            self.blocks.append(block_cls(
                build_part("mixer", layer.mixer, compute_dtype),
                build_part("feed_forward", layer.feed_forward, compute_dtype),
                build_part("norm", layer.mixer_norm, compute_dtype),
                build_part("norm", layer.feed_forward_norm, compute_dtype),
                **({"extras": extras} if extras else {}),
            ))
        self.final_norm = build_part("norm", spec.final_norm, compute_dtype)
        self.head = build_part("head", spec.head, compute_dtype)
        self.device: torch.device | None = None

    # ------------------------------------------------------------------ weights
    def parts(self):
        yield self.embedding
        for block in self.blocks:
            yield from block.parts()
        yield self.final_norm
        yield self.head

    def expected_tensors(self) -> dict[str, TensorSpec]:
        expected: dict[str, TensorSpec] = {}
        for part in self.parts():
            for name, tensor_spec in part.tensors().items():
                if name in expected and expected[name] != tensor_spec:
                    raise ValueError(f"two parts claim tensor {name!r} with different expectations")
                expected[name] = tensor_spec
        return expected

    def load(self, tensors: Mapping[str, torch.Tensor], device: torch.device | str) -> "DecoderModel":
        """Check ``tensors`` (as stored, on the CPU) against the parts and hand them over."""
        expected = self.expected_tensors()
        check_tensors(expected, tensors)
        self.device = torch.device(device)
        for part in self.parts():
            part.load(tensors, self.device)
        for block in self.blocks:
            block.finish_load(self.compute_dtype)
        return self

    # ------------------------------------------------------------------ cache
    def cache_needs(self) -> list[KVCacheNeed | StateNeed | None]:
        """What each cache entry must hold, taken from the mixer of the run step that writes it."""
        needs: list[KVCacheNeed | StateNeed | None] = [None] * self.spec.cache_entries
        for step in self.spec.run_order:
            need = self.blocks[step.layer].mixer.cache_need()
            if step.writes_cache:
                needs[step.cache] = need
            elif needs[step.cache] != need:
                raise ValueError(f"layer {step.layer} reads cache entry {step.cache}, whose layout "
                                 f"{needs[step.cache]} differs from what it needs ({need})")
        return needs

    # ------------------------------------------------------------------ forward
    def forward(self, ctx) -> torch.Tensor:
        """Run the step's rows through the model; float32 logits [wanted rows, vocab]."""
        residual = self.embedding.forward(ctx.token_ids)
        pending = None
        for step in self.spec.run_order:
            view = ctx.cache_view(step.cache)
            residual, pending = self.blocks[step.layer].forward(residual, pending, ctx, view, step.writes_cache)
        if ctx.num_wanted == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=residual.device)
        k = ctx.ops
        everything = getattr(ctx, "wanted_all_rows", False)      # every row in order (a decode step)
        rows = residual if everything else k.gather_rows(residual, ctx.wanted_rows)
        if pending is None:
            normed = self.final_norm.forward(rows)
        else:
            delta = pending if everything else k.gather_rows(pending, ctx.wanted_rows)
            # the stream itself must stay as it is only if it is read again; it is not after the last layer
            normed = self.final_norm.add_forward(rows, delta)
        return self.head.forward(normed, self.embedding)
