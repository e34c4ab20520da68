"""The per-request record that stays on the device, one per slot.

A live request owns one slot.  Beside the fixed-size state tensors of mixers that ask for them,
the slot holds one record of eight 32-bit words (``struct SlotState`` in csrc/common.cuh): how many
tokens the cache holds for the request (the position of its next token), the token it sampled last,
the index of the token it samples next (the counter of its random stream), its temperature and its
seed.  Kernels find all of it by slot: a step of decoded tokens is described to the device by the
slots of its requests and nothing else.  The reference keeps the same facts in Python objects
(``RequestState`` in src/mini_llm_runtime/scheduler.py:34-46 and the block tables' ``token_count``
in paged_kv_cache.py:116-284) and sends positions and tokens to the device each step.

The host writes a whole record when a request is admitted (``slot_record``); after that only the
device changes it: the sampling kernel stores the token and bumps the counter, the step's last
kernel advances the length.
"""

from __future__ import annotations

import struct

import numpy as np

SLOT_WORDS = 8
LENGTH, LAST_TOKEN, COUNTER, TEMPERATURE, SEED_LOW, SEED_HIGH = range(6)


def slot_record(*, length: int = 0, last_token: int = 0, counter: int = 0, temperature: float = 0.0,
                seed: int = 0) -> np.ndarray:
    """The eight words of one record, as int32."""
    if not 0 <= seed < (1 << 64):
        raise ValueError("a seed must fit 64 bits")
    words = np.zeros(SLOT_WORDS, dtype=np.uint32)
    words[LENGTH] = length
    words[LAST_TOKEN] = last_token
    words[COUNTER] = counter
    words[TEMPERATURE] = struct.unpack("<I", struct.pack("<f", float(temperature)))[0]
    words[SEED_LOW] = seed & 0xFFFFFFFF
    words[SEED_HIGH] = seed >> 32
    return words.view(np.int32)


def read_record(words: np.ndarray) -> dict:
    """A record back as a dictionary (tests and debugging)."""
    raw = np.asarray(words, dtype=np.int32).view(np.uint32)
    return {
        "length": int(raw[LENGTH]), "last_token": int(raw[LAST_TOKEN]), "counter": int(raw[COUNTER]),
        "temperature": struct.unpack("<f", struct.pack("<I", int(raw[TEMPERATURE])))[0],
        "seed": int(raw[SEED_LOW]) | (int(raw[SEED_HIGH]) << 32),
    }
