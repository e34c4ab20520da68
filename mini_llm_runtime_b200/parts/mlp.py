"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases
(reference: src/mini_llm_runtime/qwen_model_runner.py:215-217).  gate and up are stacked into one
[2*intermediate, hidden] matrix at load time so that one product feeds the activation.  When the
intermediate width is a multiple of 64 the rows are interleaved in blocks (64 gate rows, then the
64 up rows of the same outputs), which lets the tensor-core kernel apply the activation in its
epilogue; otherwise all gate rows come first."""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec, register_part


class SwiGLU(FeedForward):
    graph_safe = True
    supports_norm_fusion = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.hidden_size = int(self.args["hidden_size"])
        self.intermediate_size = int(self.args["intermediate_size"])
        self.w_gate_up = self.w_down = None
        self.block = self.intermediate_size   # gate/up interleaving of w_gate_up
        self.input_norm_eps: float | None = None

    def tensors(self):
        p = self.prefix
        return {
            p + "gate_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            p + "up_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            p + "down_proj.weight": TensorSpec((self.hidden_size, self.intermediate_size)),
        }

    def load(self, tensors, device):
        p = self.prefix
        gate, up = tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]
        if self.intermediate_size % 64 == 0:
            self.block = 64
            stacked = torch.cat([gate.view(-1, 64, self.hidden_size), up.view(-1, 64, self.hidden_size)], dim=1)
            stacked = stacked.reshape(2 * self.intermediate_size, self.hidden_size)
        else:
            stacked = torch.cat([gate, up], dim=0)
        self.w_gate_up = self._to_compute(stacked, device)
        self.w_down = self._to_compute(tensors[p + "down_proj.weight"], device)

    def absorb_input_norm(self, weight, eps):
        folded = self.w_gate_up.float() * weight.to(self.w_gate_up.device).float()[None, :]
        self.w_gate_up = folded.to(self.compute_dtype).contiguous()
        self.input_norm_eps = float(eps)

    def forward(self, x, ctx, raw_input=False, residual=None):
        k = ops.current()
        hidden = k.linear_swiglu(x, self.w_gate_up, self.block,
                                 rms_eps=self.input_norm_eps if raw_input else None)
        return k.linear(hidden, self.w_down, residual=residual)


register_part("feed_forward", "swiglu", SwiGLU)
