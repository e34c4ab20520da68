"""From a model folder (or a configuration and a seed) to a loaded ``DecoderModel``.

``load_model`` is the counterpart of the reference's ``load_qwen_checkpoint``
(src/mini_llm_runtime/qwen_loader.py:102-110); the model class is picked by config.json through
the architecture registry instead of being fixed.
"""

from __future__ import annotations

import math
from pathlib import Path

import torch

from ..config.registry import architecture_of, load_config
from ..weights.loader import read_checkpoint
from ..weights.random_init import random_tensors, write_model_dir
from .decoder import DecoderModel

_DTYPES = {
    "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
}


def parse_dtype(dtype: str | torch.dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("the engine computes in float32 or bfloat16")
        return dtype
    try:
        return _DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype {dtype!r}; use bfloat16 or float32") from None


def architecture_for(config):
    return architecture_of({"architectures": [config.architecture]})


def build_model(config, dtype: str | torch.dtype) -> DecoderModel:
    """An unloaded model for a typed configuration of any registered architecture."""
    return DecoderModel(architecture_for(config).model_spec(config), parse_dtype(dtype))


def reserve_weight_arena(model: DecoderModel, device: str | torch.device) -> None:
    """Before a model's weights are placed on a CUDA device: take one block of about their total
    size from the driver, write it once and hand it back to torch's caching allocator, which then
    carves the weights out of that one contiguous, already touched range instead of asking the
    driver for a fresh range per tensor.  Measured on a B200 with the 0.5B sizes (``bench.py`` with
    and without ``--no-arena``): 0.81 against 0.85 ms per decode step for the first model of a
    process.  Skipped when the block would take more than half of the free memory."""
    device = torch.device(device)
    if device.type != "cuda":
        return
    itemsize = torch.empty((), dtype=model.compute_dtype).element_size()
    nbytes = sum(math.prod(spec.shape) for spec in model.expected_tensors().values()) * itemsize
    nbytes = int(nbytes * 1.5) + (256 << 20)
    free, _ = torch.cuda.mem_get_info(device)
    if nbytes > free // 2:
        return
    block = torch.empty(nbytes, dtype=torch.uint8, device=device)
    block.zero_()
    del block


def load_model(model_dir: str | Path, dtype: str | torch.dtype = "bfloat16",
               device: str | torch.device = "cuda:0", *, arena: bool = True) -> tuple[object, DecoderModel]:
    """Read config.json and the safetensors of ``model_dir``; returns (config, loaded model)."""
    architecture, config = load_config(model_dir)
    model = DecoderModel(architecture.model_spec(config), parse_dtype(dtype))
    tensors = read_checkpoint(model_dir)
    if arena:
        reserve_weight_arena(model, device)
    model.load(tensors, device)
    return config, model


def random_model(config, seed: int, dtype: str | torch.dtype = "bfloat16",
                 device: str | torch.device = "cuda:0",
                 storage_dtype: torch.dtype = torch.bfloat16, *, draw_on_device: bool = False,
                 arena: bool = True) -> DecoderModel:
    """A model with seeded random weights: the tensors ``write_random_model_dir`` stores, or, with
    ``draw_on_device`` (models of many gigabytes), tensors of the same distributions drawn by the
    device's own generator."""
    model = build_model(config, dtype)
    if arena and not draw_on_device:
        reserve_weight_arena(model, device)
    model.load(random_tensors(model.expected_tensors(), seed, storage_dtype,
                              device=device if draw_on_device else "cpu"), device)
    return model


def write_random_model_dir(path: str | Path, config, seed: int,
                           storage_dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write a model folder (config.json + model.safetensors) with seeded random weights."""
    model = build_model(config, torch.float32)
    return write_model_dir(path, config, model.expected_tensors(), seed, storage_dtype)
