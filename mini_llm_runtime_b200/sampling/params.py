"""How a request chooses its tokens.

The reference chooses greedily only (``argmax`` at src/mini_llm_runtime/engine.py:222,246;
docs/continuous_batch_engine.md:67 names sampling as missing).  Here a request carries a
temperature (0 selects greedy) and a seed.  Both are written into the request's slot record on the
device when it is admitted (cache/slots.py); the sampling kernel (csrc/sampling.cu) reads them by
slot, draws from softmax(logits / temperature) with a counter-based generator keyed by the seed
and the index of the token being produced, and keeps that index in the record.  A request's tokens
therefore depend neither on what else is in its batch nor on how its prompt was cut.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self) -> None:
        if isinstance(self.temperature, bool) or not isinstance(self.temperature, (int, float)) \
                or self.temperature < 0:
            raise ValueError("temperature must be a number >= 0 (0 selects greedy)")
        if isinstance(self.seed, bool) or not isinstance(self.seed, int) or not 0 <= self.seed < (1 << 63):
            raise ValueError("seed must be an integer in [0, 2^63)")
        object.__setattr__(self, "temperature", float(self.temperature))

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


GREEDY = SamplingParams()
