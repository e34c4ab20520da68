"""Token embedding and the two heads.

Embedding is a row gather without scaling (reference: qwen_model_runner.py:263).  The tied head
multiplies by the embedding matrix as the reference always does (:289-290); the separate
``lm_head.weight`` has no counterpart there (the reference rejects untied checkpoints).  Logits
leave the head as float32.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Embedding, Head, TensorSpec, register_part


class TokenEmbedding(Embedding):
    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.vocab_size = int(self.args["vocab_size"])
        self.hidden_size = int(self.args["hidden_size"])
        self.weight: torch.Tensor | None = None

    def tensors(self):
        return {self.prefix + "weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors, device):
        self.weight = self._to_compute(tensors[self.prefix + "weight"], device)

    def forward(self, token_ids):
        return ops.current().embedding(token_ids, self.weight)


class TiedHead(Head):
    """logits = x E^T.  A checkpoint may still carry the head's own matrix; it must then equal the
    embedding's tensor, whose checkpoint name the spec gives as ``tied_to`` (reference rule:
    src/mini_llm_runtime/qwen_weights.py:113-119).  Without ``tied_to`` nothing is compared."""

    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.vocab_size = int(self.args["vocab_size"])
        self.hidden_size = int(self.args["hidden_size"])
        self.tied_to = self.args.get("tied_to")

    def tensors(self):
        return {self.prefix + "weight": TensorSpec((self.vocab_size, self.hidden_size), optional=True)}

    def load(self, tensors, device):
        copy = tensors.get(self.prefix + "weight")
        original = tensors.get(self.tied_to) if self.tied_to else None
        if copy is not None and original is not None and not torch.equal(copy, original):
            raise ValueError(f"{self.prefix}weight is present but differs from {self.tied_to} "
                             "although tie_word_embeddings is true")

    def extra_inputs(self):
        return (self.tied_to,) if self.tied_to else ()

    def forward(self, x, embedding):
        return ops.current().linear(x, embedding.weight, None, out_dtype=torch.float32)


class LinearHead(Head):
    graph_safe = True

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.vocab_size = int(self.args["vocab_size"])
        self.hidden_size = int(self.args["hidden_size"])
        self.weight: torch.Tensor | None = None

    def tensors(self):
        return {self.prefix + "weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors, device):
        self.weight = self._to_compute(tensors[self.prefix + "weight"], device)

    def forward(self, x, embedding):
        return ops.current().linear(x, self.weight, None, out_dtype=torch.float32)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "tied_head", TiedHead)
register_part("head", "linear_head", LinearHead)
