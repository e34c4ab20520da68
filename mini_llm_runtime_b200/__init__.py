"""B200-native inference engine for Qwen2 / Qwen2.5 decoders: typed config and registry, weights
by tensor name, a decoder assembled from parts, a paged KV cache manager, one step function for
ragged batches, a scheduler with chunked prefill, sampling, and hand-written sm_100a kernels."""

from .cache import CacheManager, OutOfPages
from .config import Qwen2Config, config_from_dict, load_config, register_architecture
from .engine import (BatchingPolicy, CacheGate, ContinuousBatchEngine, ModelRunner, RequestScheduler, StepEntry,
                     greedy_generate)
from .models import DecoderModel, build_model, load_model, random_model, write_random_model_dir
from .parts import register_part
from .sampling import SamplingParams

__version__ = "0.1.0"

__all__ = [
    "BatchingPolicy", "CacheGate", "CacheManager", "ContinuousBatchEngine", "DecoderModel", "ModelRunner",
    "OutOfPages", "Qwen2Config", "RequestScheduler", "SamplingParams", "StepEntry",
    "build_model", "config_from_dict", "greedy_generate", "load_config", "load_model", "random_model",
    "register_architecture", "register_part", "write_random_model_dir",
]
