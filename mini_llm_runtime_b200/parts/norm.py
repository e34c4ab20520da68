"""RMSNorm: y = w * x * rsqrt(mean(x^2) + eps), all in float32, eps inside the root, no centering
and no bias (reference: src/mini_llm_runtime/qwen_model_runner.py:22-26).  The reference casts the
normalised row back to the model dtype before multiplying by w; here the product is taken in
float32 and rounded once."""

from __future__ import annotations

import torch

from .. import ops
from .base import Norm, TensorSpec, register_part


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.size = int(self.args["size"])
        self.eps = float(self.args["eps"])
        self.weight: torch.Tensor | None = None
        self.folded = False       # True once the weight lives in the matrix that follows

    def tensors(self):
        return {self.prefix + "weight": TensorSpec((self.size,), init="norm")}

    def load(self, tensors, device):
        self.weight = self._keep_precision(tensors[self.prefix + "weight"], device)

    def fold(self):
        self.folded = True
        return self.weight, self.eps

    def forward(self, x):
        return ops.current().rms_norm(x, None if self.folded else self.weight, self.eps)

    def add_forward(self, residual, delta):
        return ops.current().add_rms_norm(residual, delta, None if self.folded else self.weight, self.eps)


register_part("norm", "rms_norm", RMSNorm)
