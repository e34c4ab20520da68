"""Typed configuration of ``Qwen2ForCausalLM`` read from the keys of its own config.json.

Same eleven required keys, coercions and validation rules as the reference's
``QwenConfig`` (src/mini_llm_runtime/qwen_config.py:9-93), with three differences:
``tie_word_embeddings=false`` is accepted (the reference rejects it at :43-44), ``head_dim``
is read when present (the reference derives it, :46-48), and the sliding-window keys are
read instead of ignored.  Error messages are in English.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .spec import LayerSpec, ModelSpec, PartSpec, RunStep

_REQUIRED = (
    "vocab_size",
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "num_key_value_heads",
    "max_position_embeddings",
    "rms_norm_eps",
    "rope_theta",
    "hidden_act",
    "tie_word_embeddings",
)


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    hidden_act: str
    tie_word_embeddings: bool
    head_dim: int = 0  # 0 -> hidden_size // num_attention_heads
    use_sliding_window: bool = False
    sliding_window: int | None = None
    max_window_layers: int = 0
    eos_token_id: int | None = None

    architecture = "Qwen2ForCausalLM"
    model_type = "qwen2"

    def __post_init__(self) -> None:
        if self.head_dim == 0:
            if self.hidden_size % max(self.num_attention_heads, 1) != 0:
                raise ValueError("hidden_size must be divisible by num_attention_heads "
                                 "when config.json gives no head_dim")
            object.__setattr__(self, "head_dim", self.hidden_size // max(self.num_attention_heads, 1))
        integers = {
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "max_position_embeddings": self.max_position_embeddings,
            "head_dim": self.head_dim,
        }
        bad = [name for name, value in integers.items() if value <= 0]
        if bad:
            raise ValueError(f"Qwen2Config: these sizes must be > 0: {', '.join(bad)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ValueError("num_attention_heads must be divisible by num_key_value_heads")
        if self.head_dim % 2 != 0:
            raise ValueError("head_dim must be even for rotate-half position encoding")
        if self.rms_norm_eps <= 0 or self.rope_theta <= 0:
            raise ValueError("rms_norm_eps and rope_theta must be > 0")
        if self.hidden_act != "silu":
            raise ValueError(f"Qwen2 uses hidden_act='silu', config.json says {self.hidden_act!r}")
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                raise ValueError("use_sliding_window=true needs a positive sliding_window")
            if not 0 <= self.max_window_layers <= self.num_hidden_layers:
                raise ValueError("max_window_layers must lie in 0..num_hidden_layers")

    @property
    def gqa_group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def layer_window(self, layer: int) -> int | None:
        """Layers from ``max_window_layers`` on see only the last ``sliding_window`` keys."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Qwen2Config":
        if data.get("model_type") != cls.model_type:
            raise ValueError(f"Qwen2Config needs model_type='qwen2', got {data.get('model_type')!r}")
        if data.get("rope_scaling") is not None:
            raise ValueError("rope_scaling is not supported (config.json must give null or omit it)")
        missing = [name for name in _REQUIRED if name not in data]
        if missing:
            raise KeyError(f"config.json lacks these keys: {', '.join(missing)}")
        window = data.get("sliding_window")
        eos = data.get("eos_token_id")
        return cls(
            vocab_size=int(data["vocab_size"]),
            hidden_size=int(data["hidden_size"]),
            intermediate_size=int(data["intermediate_size"]),
            num_hidden_layers=int(data["num_hidden_layers"]),
            num_attention_heads=int(data["num_attention_heads"]),
            num_key_value_heads=int(data["num_key_value_heads"]),
            max_position_embeddings=int(data["max_position_embeddings"]),
            rms_norm_eps=float(data["rms_norm_eps"]),
            rope_theta=float(data["rope_theta"]),
            hidden_act=str(data["hidden_act"]),
            tie_word_embeddings=bool(data["tie_word_embeddings"]),
            head_dim=int(data.get("head_dim") or 0),
            use_sliding_window=bool(data.get("use_sliding_window", False)),
            sliding_window=None if window is None else int(window),
            max_window_layers=int(data.get("max_window_layers", 0)),
            eos_token_id=eos if isinstance(eos, int) else None,
        )

    def to_dict(self) -> dict[str, Any]:
        """The config.json that describes this configuration (used by the random-weights mode)."""
        data: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
        }
        for name in _REQUIRED:
            data[name] = getattr(self, name)
        data["head_dim"] = self.head_dim
        data["use_sliding_window"] = self.use_sliding_window
        data["sliding_window"] = self.sliding_window
        data["max_window_layers"] = self.max_window_layers
        data["rope_scaling"] = None
        if self.eos_token_id is not None:
            data["eos_token_id"] = self.eos_token_id
        return data


def qwen2_model_spec(config: Qwen2Config) -> ModelSpec:
    """Qwen2 as parts: pre-norm blocks of (RMSNorm, GQA attention with biased q/k/v and
    rotate-half RoPE, RMSNorm, SwiGLU), final RMSNorm, tied or untied head.  Tensor names are
    the Hugging Face ones the reference reads (src/mini_llm_runtime/qwen_weights.py:69-115)."""
    norm_args = {"size": config.hidden_size, "eps": config.rms_norm_eps}
    layers = []
    for index in range(config.num_hidden_layers):
        prefix = f"model.layers.{index}."
        mixer = PartSpec(
            "gqa_attention",
            {
                "hidden_size": config.hidden_size,
                "num_heads": config.num_attention_heads,
                "num_kv_heads": config.num_key_value_heads,
                "head_dim": config.head_dim,
                "qkv_bias": True,
                "out_bias": False,
                "window": config.layer_window(index),
                "position": PartSpec("rope_half", {"head_dim": config.head_dim,
                                                   "theta": config.rope_theta}),
            },
            prefix + "self_attn.",
        )
        feed_forward = PartSpec(
            "swiglu",
            {"hidden_size": config.hidden_size, "intermediate_size": config.intermediate_size},
            prefix + "mlp.",
        )
        layers.append(
            LayerSpec(
                block="pre_norm_residual",
                mixer=mixer,
                feed_forward=feed_forward,
                mixer_norm=PartSpec("rms_norm", norm_args, prefix + "input_layernorm."),
                feed_forward_norm=PartSpec("rms_norm", norm_args, prefix + "post_attention_layernorm."),
            )
        )
    sizes = {"vocab_size": config.vocab_size, "hidden_size": config.hidden_size}
    embedding_prefix = "model.embed_tokens."
    if config.tie_word_embeddings:
        head = PartSpec("tied_head", {**sizes, "tied_to": embedding_prefix + "weight"}, "lm_head.")
    else:
        head = PartSpec("linear_head", sizes, "lm_head.")
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab_size,
        hidden_size=config.hidden_size,
        max_positions=config.max_position_embeddings,
        embedding=PartSpec("token_embedding", sizes, embedding_prefix),
        layers=tuple(layers),
        run_order=tuple(RunStep(layer=i, cache=i) for i in range(config.num_hidden_layers)),
        final_norm=PartSpec("rms_norm", norm_args, "model.norm."),
        head=head,
    )
