"""Rotate-half rotary position encoding (reference: src/mini_llm_runtime/qwen_model_runner.py:34-61).

inv_freq[i] = 1 / theta^(2i/D) for i < D/2 in float32; angle = position * inv_freq[i]; element i is
paired with element i + D/2; q and k are rotated, v is not.  The frequency table is computed once
here, with the reference's expression, and handed to the kernel, which evaluates sine and cosine
in float32 and fuses the rotation with the write of k and v into the cache pages.  No table over
positions is kept, so ``max_position_embeddings`` only bounds lengths, as in the reference.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import PositionEncoding, register_part


class RotateHalfRope(PositionEncoding):
    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.head_dim = int(self.args["head_dim"])
        self.theta = float(self.args["theta"])
        if self.head_dim % 2:
            raise ValueError("rotate-half position encoding needs an even head_dim")
        exponents = torch.arange(0, self.head_dim, 2, dtype=torch.float32) / self.head_dim
        self._inv_freq_cpu = 1.0 / (self.theta ** exponents)
        self.inv_freq: torch.Tensor | None = None

    def load(self, tensors, device):
        self.inv_freq = self._inv_freq_cpu.to(device)

    def rotate_and_store(self, qkv, ctx, view, num_heads, num_kv_heads, head_dim, write_kv):
        if head_dim != self.head_dim:
            raise ValueError(f"position encoding was built for head_dim {self.head_dim}, mixer has {head_dim}")
        return ops.current().rope_kv_write(qkv, ctx.positions, self.inv_freq, view.slots, view.k_pool,
                                           view.v_pool, num_heads, num_kv_heads, head_dim, write_kv)

    def rotary_frequencies(self):
        return self.inv_freq


register_part("position", "rope_half", RotateHalfRope)
