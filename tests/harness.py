"""Shared helpers of the tests: build a tiny engine with random weights, run the plain
implementation on the same tensors, compare with tolerances fixed per dtype.

Tolerances.  float32: kernels and the plain code differ only in the order of float32 additions,
so logits must agree to 2e-5 of their scale.  bfloat16: every kernel rounds its output to 8
mantissa bits (relative 2^-9 per rounding); through a few layers that gives about one percent,
so rows must agree to 2e-2 in relative L2 norm and 4e-2 of the scale in the worst element.
"""

from __future__ import annotations

import torch

import plain_qwen2 as plain
from mini_llm_runtime_b200.cache import CacheManager
from mini_llm_runtime_b200.engine import ModelRunner, StepEntry
from mini_llm_runtime_b200.models import build_model
from mini_llm_runtime_b200.weights import random_tensors


def tolerance(dtype: torch.dtype) -> dict:
    if dtype == torch.float32:
        return {"rel_l2": 1e-5, "max_abs": 2e-5}
    return {"rel_l2": 2e-2, "max_abs": 4e-2}


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: torch.dtype, what: str = "") -> None:
    got = got.detach().float().cpu()
    want = want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values in the result"
    tol = tolerance(dtype)
    scale = max(float(want.abs().max()), 1e-6)
    worst = float((got - want).abs().max())
    rows_got = got.reshape(-1, got.shape[-1])
    rows_want = want.reshape(-1, want.shape[-1])
    rel = (rows_got - rows_want).norm(dim=-1) / rows_want.norm(dim=-1).clamp_min(1e-6 * scale)
    worst_row = int(rel.argmax()) if rel.numel() else 0
    assert worst <= tol["max_abs"] * scale, (
        f"{what}: worst element differs by {worst:.3e} (scale {scale:.3e}, allowed "
        f"{tol['max_abs'] * scale:.3e}); worst row {worst_row}")
    assert float(rel.max()) <= tol["rel_l2"], (
        f"{what}: row {worst_row} differs by {float(rel.max()):.3e} in relative L2 "
        f"(allowed {tol['rel_l2']:.1e})")


def random_prompt(vocab: int, length: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=generator).tolist()


class TinyEngine:
    """A model with seeded random weights, its cache and runner, plus the plain oracle."""

    def __init__(self, config, page_size: int, dtype: torch.dtype, device: str, *, num_pages: int = 64,
                 max_requests: int = 4, max_tokens: int = 512, seed: int = 0, max_step_tokens: int = 512,
                 tensors=None):
        self.config = config
        self.config_dict = config.to_dict()
        self.dtype = dtype
        self.model = build_model(config, dtype)
        self.tensors = tensors if tensors is not None else random_tensors(
            self.model.expected_tensors(), seed, torch.bfloat16)
        self.model.load(self.tensors, device)
        self.cache = CacheManager(self.model.cache_needs(), page_size=page_size, num_pages=num_pages,
                                  max_requests=max_requests, max_tokens_per_request=max_tokens,
                                  dtype=dtype, device=device, max_step_tokens=max_step_tokens)
        self.runner = ModelRunner(self.model, self.cache)
        self.runner.graph_capture_after = 1          # tests want the captured step from the first recurrence on

    def plain_logits(self, tokens) -> torch.Tensor:
        return plain.forward_logits(self.tensors, self.config_dict, tokens)

    def run_whole(self, request_id: str, tokens) -> torch.Tensor:
        self.cache.create_request(request_id)
        return self.runner.step([StepEntry(request_id, list(tokens), list(range(len(tokens))))])

    def run_cuts(self, request_id: str, tokens, cuts) -> torch.Tensor:
        """Feed ``tokens`` in portions ending at the positions in ``cuts``; all logits."""
        self.cache.create_request(request_id)
        outputs = []
        start = 0
        for end in list(cuts) + [len(tokens)]:
            if end <= start:
                continue
            outputs.append(self.runner.step(
                [StepEntry(request_id, list(tokens[start:end]), list(range(end - start)))]))
            start = end
        return torch.cat(outputs)
