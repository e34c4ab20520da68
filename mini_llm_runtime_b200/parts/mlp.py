"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases
(reference: src/mini_llm_runtime/qwen_model_runner.py:215-217).  gate and up are stacked into one
[2*intermediate, hidden] matrix at load time so that one product feeds the activation kernel."""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec, register_part


class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.hidden_size = int(self.args["hidden_size"])
        self.intermediate_size = int(self.args["intermediate_size"])
        self.w_gate_up = self.w_down = None

    def tensors(self):
        p = self.prefix
        return {
            p + "gate_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            p + "up_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            p + "down_proj.weight": TensorSpec((self.hidden_size, self.intermediate_size)),
        }

    def load(self, tensors, device):
        p = self.prefix
        self.w_gate_up = self._to_compute(
            torch.cat([tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]], dim=0), device)
        self.w_down = self._to_compute(tensors[p + "down_proj.weight"], device)

    def forward(self, x, ctx):
        k = ops.current()
        return k.linear(k.swiglu(k.linear(x, self.w_gate_up)), self.w_down)


register_part("feed_forward", "swiglu", SwiGLU)
