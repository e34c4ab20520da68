"""Random-weights mode: fills every tensor a model's parts name from a seed and can write the
result as a model folder (config.json + model.safetensors) that the ordinary loader reads.

The reference has no such mode; its tests draw a tiny state dict from a seeded generator
(tests/test_qwen_weights.py:25-65 there).  Distributions: matrices ~ N(0, 0.02), norm weights
~ 1 + N(0, 0.02), biases ~ N(0, 0.02), integer tables uniform below their bound.  Tensors are
drawn one by one in sorted-name order from one CPU generator, in float32, then rounded to the
storage dtype, so a given (configuration, seed, dtype) always yields the same bytes.  For models
of many gigabytes ``device=`` draws from that device's generator instead (other bytes, the same
distributions, seconds instead of minutes); model folders are always written from the CPU stream.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping

import torch
from safetensors.torch import save_file

from .loader import SINGLE_FILE

STD = 0.02


def random_tensors(expected: Mapping[str, "TensorSpec"], seed: int,
                   dtype: torch.dtype = torch.bfloat16, device: str | torch.device = "cpu") -> dict[str, torch.Tensor]:
    device = torch.device(device)
    generator = torch.Generator(device=device)
    generator.manual_seed(int(seed))
    tensors: dict[str, torch.Tensor] = {}
    for name in sorted(expected):
        spec = expected[name]
        if spec.optional:
            continue
        shape = tuple(spec.shape)
        if spec.storage == "int" or spec.init == "table":
            tensors[name] = torch.randint(0, max(int(spec.high), 1), shape, generator=generator,
                                          dtype=torch.int32, device=device)
            continue
        values = torch.randn(shape, generator=generator, dtype=torch.float32, device=device) * STD
        if spec.init == "norm":
            values = values + 1.0
        elif spec.init not in ("matrix", "bias"):
            raise ValueError(f"tensor {name}: unknown init kind {spec.init!r}")
        tensors[name] = values.to(dtype)
    return tensors


def write_model_dir(path: str | Path, config, expected: Mapping[str, "TensorSpec"], seed: int,
                    dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with seeded random weights."""
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    data = config.to_dict()
    data["torch_dtype"] = str(dtype).replace("torch.", "")
    with (path / "config.json").open("w", encoding="utf-8") as handle:
        json.dump(data, handle, indent=2)
    tensors = random_tensors(expected, seed, dtype)
    save_file({name: tensor.contiguous() for name, tensor in tensors.items()}, str(path / SINGLE_FILE))
    return path
