"""Turns the step's logits into one token per request on the device.

Greedy (temperature 0) is the reference's only mode (``argmax`` at src/mini_llm_runtime/engine.py:
222,246).  Temperature sampling draws from softmax(logits / T) with a counter-based generator
keyed by the request's seed and the index of the token being produced, so a request's tokens do
not depend on what else is in the batch or on how its prompt was cut.
"""

from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from .. import ops


class Sampler:
    def __init__(self, device: torch.device | str) -> None:
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], seeds: Sequence[int],
               token_indices: Sequence[int]) -> torch.Tensor:
        """int32 tokens [rows] on the device; row r uses temperatures[r] (0 = greedy), seeds[r]
        and token_indices[r] (how many tokens the request has produced so far)."""
        rows = logits.shape[0]
        if not (len(temperatures) == len(seeds) == len(token_indices) == rows):
            raise ValueError("one temperature, seed and token index per logits row")
        pinned = self.device.type == "cuda"
        t = torch.from_numpy(np.asarray(temperatures, dtype=np.float32))
        s = torch.from_numpy(np.asarray(seeds, dtype=np.int64))
        c = torch.from_numpy(np.asarray(token_indices, dtype=np.int64))
        if pinned:
            t, s, c = t.pin_memory(), s.pin_memory(), c.pin_memory()
        return ops.current().sample(logits, t.to(self.device, non_blocking=True),
                                    s.to(self.device, non_blocking=True),
                                    c.to(self.device, non_blocking=True))
