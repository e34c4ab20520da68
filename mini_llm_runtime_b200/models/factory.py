"""From a model folder (or a configuration and a seed) to a loaded ``DecoderModel``.

``load_model`` is the counterpart of the reference's ``load_qwen_checkpoint``
(src/mini_llm_runtime/qwen_loader.py:102-110); the model class is picked by config.json through
the architecture registry instead of being fixed.
"""

from __future__ import annotations

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


def load_model(model_dir: str | Path, dtype: str | torch.dtype = "bfloat16",
               device: str | torch.device = "cuda:0") -> tuple[object, DecoderModel]:
    """Read config.json and the safetensors of ``model_dir``; returns (config, loaded model)."""
    architecture, config = load_config(model_dir)
    model = DecoderModel(architecture.model_spec(config), parse_dtype(dtype))
    model.load(read_checkpoint(model_dir), device)
    return config, model


def random_model(config, seed: int, dtype: str | torch.dtype = "bfloat16",
                 device: str | torch.device = "cuda:0",
                 storage_dtype: torch.dtype = torch.bfloat16) -> DecoderModel:
    """A model with seeded random weights, the same tensors ``write_random_model_dir`` stores."""
    model = build_model(config, dtype)
    model.load(random_tensors(model.expected_tensors(), seed, storage_dtype), device)
    return model


def write_random_model_dir(path: str | Path, config, seed: int,
                           storage_dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write a model folder (config.json + model.safetensors) with seeded random weights."""
    model = build_model(config, torch.float32)
    return write_model_dir(path, config, model.expected_tensors(), seed, storage_dtype)
