"""Reads a checkpoint's tensors by name from safetensors and checks them against what the model's
parts expect.

File handling follows the reference's loader (src/mini_llm_runtime/qwen_loader.py:30-99): a single
``model.safetensors``, or ``model.safetensors.index.json`` with its shards; shards without an
index, a missing shard, a tensor in two shards, or an index that disagrees with a shard are
errors.  Tensors come back on the CPU exactly as stored: bfloat16 stays bfloat16, a tensor
stored in 32-bit stays 32-bit, integer tables become int32.  Nothing is renamed here; fusing
(q|k|v, gate|up) is the business of the part that owns the tensors.

Unlike the reference, which stops at the first problem (src/mini_llm_runtime/qwen_weights.py:55-64,
121-124), ``check_tensors`` reports every missing tensor, unexpected tensor and wrong shape in
one error.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping

import torch
from safetensors import safe_open

SINGLE_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"

_INTEGER = (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)


class WeightError(ValueError):
    """The checkpoint does not hold what the model needs; the message lists every difference."""

    def __init__(self, message, *, missing=(), unexpected=(), wrong_shape=(), wrong_kind=()):
        super().__init__(message)
        self.missing = tuple(missing)
        self.unexpected = tuple(unexpected)
        self.wrong_shape = tuple(wrong_shape)
        self.wrong_kind = tuple(wrong_kind)


def _shard_plan(model_dir: Path) -> dict[str, list[str] | None]:
    """file name -> tensor names the index promises there (None: single file, take all)."""
    index = model_dir / INDEX_FILE
    single = model_dir / SINGLE_FILE
    if index.is_file():
        with index.open("r", encoding="utf-8") as handle:
            data = json.load(handle)
        weight_map = data.get("weight_map") if isinstance(data, dict) else None
        if not isinstance(weight_map, dict) or not weight_map:
            raise ValueError(f"{index} has no usable 'weight_map'")
        plan: dict[str, list[str]] = {}
        for tensor_name, file_name in weight_map.items():
            if not isinstance(tensor_name, str) or not isinstance(file_name, str):
                raise ValueError(f"{index}: weight_map must map strings to strings")
            plan.setdefault(file_name, []).append(tensor_name)
        for file_name in plan:
            if not (model_dir / file_name).is_file():
                raise FileNotFoundError(f"{index} names shard {file_name!r}, which is missing")
        return plan
    if single.is_file():
        return {SINGLE_FILE: None}
    shards = sorted(p.name for p in model_dir.glob("model-*.safetensors"))
    if shards:
        raise FileNotFoundError(f"{model_dir} holds shards ({shards[0]}, ...) but no {INDEX_FILE}")
    raise FileNotFoundError(f"{model_dir} holds neither {SINGLE_FILE} nor {INDEX_FILE}")


def read_checkpoint(model_dir: str | Path) -> dict[str, torch.Tensor]:
    model_dir = Path(model_dir)
    tensors: dict[str, torch.Tensor] = {}
    for file_name, promised in _shard_plan(model_dir).items():
        with safe_open(str(model_dir / file_name), framework="pt", device="cpu") as handle:
            present = list(handle.keys())
            if promised is not None and set(present) != set(promised):
                only_index = sorted(set(promised) - set(present))[:5]
                only_shard = sorted(set(present) - set(promised))[:5]
                raise ValueError(f"shard {file_name} disagrees with the index: only in the index "
                                 f"{only_index}, only in the shard {only_shard}")
            for name in present:
                if name in tensors:
                    raise ValueError(f"tensor {name!r} appears in more than one shard")
                tensor = handle.get_tensor(name)
                if tensor.dtype in _INTEGER:
                    tensor = tensor.to(torch.int32)
                tensors[name] = tensor
    return tensors


def check_tensors(expected: Mapping[str, "TensorSpec"], found: Mapping[str, torch.Tensor]) -> None:
    """Raise one ``WeightError`` naming all missing, unexpected, mis-shaped and mis-typed tensors."""
    missing = sorted(name for name, spec in expected.items() if name not in found and not spec.optional)
    unexpected = sorted(name for name in found if name not in expected)
    wrong_shape = []
    wrong_kind = []
    for name, spec in expected.items():
        if name not in found:
            continue
        tensor = found[name]
        if tuple(tensor.shape) != tuple(spec.shape):
            wrong_shape.append((name, tuple(tensor.shape), tuple(spec.shape)))
        is_int = not tensor.dtype.is_floating_point
        if (spec.storage == "int") != is_int:
            wrong_kind.append((name, str(tensor.dtype), spec.storage))
    if not (missing or unexpected or wrong_shape or wrong_kind):
        return
    lines = ["the checkpoint does not match the model:"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong_shape:
        lines.append(f"  wrong shape ({len(wrong_shape)}): " + "; ".join(
            f"{name} is {actual}, expected {wanted}" for name, actual, wanted in wrong_shape))
    if wrong_kind:
        lines.append(f"  wrong kind ({len(wrong_kind)}): " + "; ".join(
            f"{name} is {actual}, expected {wanted}" for name, actual, wanted in wrong_kind))
    raise WeightError("\n".join(lines), missing=missing, unexpected=unexpected,
                      wrong_shape=wrong_shape, wrong_kind=wrong_kind)
