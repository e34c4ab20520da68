"""Pre-norm residual arrangement: h = x + mixer(norm(x)); out = h + feed_forward(norm(h))
(reference: the ``_decoder_layer`` function, src/mini_llm_runtime/qwen_model_runner.py:199-218).

The residual stream and the newest output not yet added to it travel together, so that each
add is fused into the norm that follows it: one kernel reads and writes the stream once.
"""

from __future__ import annotations

from .base import Block, register_part


class PreNormResidual(Block):
    def forward(self, residual, pending, ctx, view, writes_cache):
        if pending is None:
            normed = self.mixer_norm.forward(residual)
        else:
            normed = self.mixer_norm.add_forward(residual, pending)
        mixed = self.mixer.forward(normed, ctx, view, writes_cache)
        normed = self.feed_forward_norm.add_forward(residual, mixed)
        return residual, self.feed_forward.forward(normed, ctx)


register_part("block", "pre_norm_residual", PreNormResidual)
