"""Pre-norm residual arrangement: h = x + mixer(norm(x)); out = h + feed_forward(norm(h))
(reference: the ``_decoder_layer`` function, src/mini_llm_runtime/qwen_model_runner.py:199-218).

The residual stream and the newest output not yet added to it travel together, so that each
add is fused into the norm that follows it: one kernel reads and writes the stream once.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Block, register_part


class PreNormResidual(Block):
    """In bfloat16, when both norms are of the "row scale times weight" kind and mixer and
    feed-forward can take it, each norm's weight is folded into the matrix that follows it at load
    time.  Steps of few rows (decode) then run without norm kernels: the products apply the row
    scale themselves and the products that end the mixer and the feed-forward add their result
    into the stream in place.  Steps of many rows keep the arrangement below, with norm kernels
    that only scale.  The float32 path keeps the reference's order of operations."""

    folded = False

    def finish_load(self, compute_dtype):
        if (compute_dtype == torch.bfloat16 and self.mixer.supports_norm_fusion
                and self.feed_forward.supports_norm_fusion):
            first, second = self.mixer_norm.fold(), self.feed_forward_norm.fold()
            if first is None or second is None:
                raise ValueError("a norm that cannot be folded must say so before it is asked to")
            self.mixer.absorb_input_norm(*first)
            self.feed_forward.absorb_input_norm(*second)
            self.folded = True

    def forward(self, residual, pending, ctx, view, writes_cache):
        kernels = ops.current()
        if self.folded and kernels.fuses_norm(residual.shape[0]):
            if pending is not None:
                residual = kernels.add_inplace(residual, pending)
            self.mixer.forward(residual, ctx, view, writes_cache, raw_input=True, residual=residual)
            self.feed_forward.forward(residual, ctx, raw_input=True, residual=residual)
            return residual, None
        if pending is None:
            normed = self.mixer_norm.forward(residual)
        else:
            normed = self.mixer_norm.add_forward(residual, pending)
        mixed = self.mixer.forward(normed, ctx, view, writes_cache)
        normed = self.feed_forward_norm.add_forward(residual, mixed)
        return residual, self.feed_forward.forward(normed, ctx)


register_part("block", "pre_norm_residual", PreNormResidual)
