"""Toy parts defined by the tests, registered from outside the package: a mixer with state of its
own, a feed-forward with routing, another position encoding, and a toy architecture that uses
them beside the package's own parts.  They show that the part interfaces carry more than one
architecture; they are written with plain torch operations and are no model of anyone's."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from mini_llm_runtime_b200 import ops
from mini_llm_runtime_b200.config import LayerSpec, ModelSpec, PartSpec, RunStep
from mini_llm_runtime_b200.parts import (FeedForward, Mixer, PositionEncoding, StateNeed, TensorSpec,
                                         register_part)


class RunningMeanMixer(Mixer):
    """out[p] = W * mean(x[0..p]): the running sum and the count live in the request's state slot
    and are carried from step to step."""

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.size = int(self.args["hidden_size"])
        self.weight = None

    def cache_need(self):
        return StateNeed((self.size + 1,), torch.float32)

    def tensors(self):
        return {self.prefix + "mix.weight": TensorSpec((self.size, self.size))}

    def load(self, tensors, device):
        self.weight = self._to_compute(tensors[self.prefix + "mix.weight"], device)

    def forward(self, x, ctx, view, writes_cache):
        out = torch.empty_like(x)
        for segment in ctx.segments:
            rows = slice(segment.row_start, segment.row_start + segment.length)
            state = view.state[segment.slot]
            sums = state[: self.size] + torch.cumsum(x[rows].float(), dim=0)
            counts = state[self.size] + torch.arange(1, segment.length + 1, device=x.device, dtype=torch.float32)
            out[rows] = (sums / counts[:, None]).to(x.dtype)
            if writes_cache:
                state[: self.size] = sums[-1]
                state[self.size] = counts[-1]
        return ctx.ops.linear(out, self.weight)


class TopOneRouted(FeedForward):
    """A router picks one of ``experts`` small SwiGLU-free MLPs per row (router logits in float32)."""

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        self.size = int(self.args["hidden_size"])
        self.inner = int(self.args["intermediate_size"])
        self.experts = int(self.args["experts"])

    def tensors(self):
        out = {self.prefix + "router.weight": TensorSpec((self.experts, self.size))}
        for e in range(self.experts):
            out[self.prefix + f"experts.{e}.up.weight"] = TensorSpec((self.inner, self.size))
            out[self.prefix + f"experts.{e}.down.weight"] = TensorSpec((self.size, self.inner))
        return out

    def load(self, tensors, device):
        self.router = tensors[self.prefix + "router.weight"].to(device=device, dtype=torch.float32)
        self.up = [self._to_compute(tensors[self.prefix + f"experts.{e}.up.weight"], device) for e in range(self.experts)]
        self.down = [self._to_compute(tensors[self.prefix + f"experts.{e}.down.weight"], device) for e in range(self.experts)]

    def forward(self, x, ctx):
        choice = torch.argmax(x.float() @ self.router.T, dim=-1)
        out = torch.zeros_like(x)
        for e in range(self.experts):
            rows = torch.nonzero(choice == e).flatten()
            if rows.numel():
                hidden = torch.relu(ctx.ops.linear(x[rows].contiguous(), self.up[e]))
                out[rows] = ctx.ops.linear(hidden, self.down[e])
        return out


class NoRotation(PositionEncoding):
    """A position encoding that leaves q and k alone (the cache write still happens)."""

    def load(self, tensors, device):
        self.zero_freq = torch.zeros(int(self.args["head_dim"]) // 2, dtype=torch.float32, device=device)

    def rotate_and_store(self, qkv, ctx, view, num_heads, num_kv_heads, head_dim, write_kv):
        return ctx.ops.rope_kv_write(qkv, ctx.positions, self.zero_freq, view.slots, view.k_pool, view.v_pool,
                                     num_heads, num_kv_heads, head_dim, write_kv)


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int = 97
    hidden_size: int = 48
    architecture = "ToyForCausalLM"

    @classmethod
    def from_dict(cls, data):
        return cls(int(data["vocab_size"]), int(data["hidden_size"]))

    def to_dict(self):
        return {"architectures": [self.architecture], "model_type": "toy",
                "vocab_size": self.vocab_size, "hidden_size": self.hidden_size}


def toy_model_spec(config: ToyConfig) -> ModelSpec:
    """Layer 0: attention without rotation + routed feed-forward; layer 1: running-mean mixer +
    SwiGLU; the run order names layer 1 twice (two state entries) and ends with a layer that reads
    layer 0's keys and values without writing."""
    h = config.hidden_size
    norm = {"size": h, "eps": 1e-5}

    def attention(prefix):
        return PartSpec("gqa_attention", {"hidden_size": h, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16,
                                          "qkv_bias": False, "out_bias": True, "window": None,
                                          "position": PartSpec("toy_no_rotation", {"head_dim": 16})}, prefix)

    layers = (
        LayerSpec("pre_norm_residual", attention("l0.attn."),
                  PartSpec("toy_routed", {"hidden_size": h, "intermediate_size": 40, "experts": 3}, "l0.ffn."),
                  PartSpec("rms_norm", norm, "l0.n1."), PartSpec("rms_norm", norm, "l0.n2.")),
        LayerSpec("pre_norm_residual", PartSpec("toy_running_mean", {"hidden_size": h}, "l1.mixer."),
                  PartSpec("swiglu", {"hidden_size": h, "intermediate_size": 56}, "l1.mlp."),
                  PartSpec("rms_norm", norm, "l1.n1."), PartSpec("rms_norm", norm, "l1.n2.")),
        LayerSpec("pre_norm_residual", attention("l2.attn."),
                  PartSpec("swiglu", {"hidden_size": h, "intermediate_size": 24}, "l2.mlp."),
                  PartSpec("rms_norm", norm, "l2.n1."), PartSpec("rms_norm", norm, "l2.n2.")),
    )
    sizes = {"vocab_size": config.vocab_size, "hidden_size": h}
    return ModelSpec(
        architecture=config.architecture, vocab_size=config.vocab_size, hidden_size=h, max_positions=256,
        embedding=PartSpec("token_embedding", sizes, "embed."),
        layers=layers,
        run_order=(RunStep(0, 0), RunStep(1, 1), RunStep(1, 2), RunStep(2, 0, writes_cache=False)),
        final_norm=PartSpec("rms_norm", norm, "final."),
        head=PartSpec("tied_head", sizes, "head."))


def register_toys():
    register_part("mixer", "toy_running_mean", RunningMeanMixer, replace=True)
    register_part("feed_forward", "toy_routed", TopOneRouted, replace=True)
    register_part("position", "toy_no_rotation", NoRotation, replace=True)


# ---------------------------------------------------------------- the toy model, plainly
def plain_toy_logits(tensors, config: ToyConfig, tokens):
    """Whole sequence, no cache, float32: what the toy architecture computes."""
    import plain_qwen2 as plain

    t = {k: v.float() for k, v in tensors.items()}
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = t["embed.weight"][ids]

    def attention(prefix, y):
        q = plain.split_heads(y @ t[prefix + "q_proj.weight"].T, 3, 16)
        k = plain.split_heads(y @ t[prefix + "k_proj.weight"].T, 1, 16)
        v = plain.split_heads(y @ t[prefix + "v_proj.weight"].T, 1, 16)
        mixed = plain.causal_attention(q, k, v).transpose(0, 1).reshape(len(tokens), 48)
        return mixed @ t[prefix + "o_proj.weight"].T + t[prefix + "o_proj.bias"], k, v

    def swiglu(prefix, y):
        return (torch.nn.functional.silu(y @ t[prefix + "gate_proj.weight"].T) * (y @ t[prefix + "up_proj.weight"].T)) \
            @ t[prefix + "down_proj.weight"].T

    def running_mean(y):
        counts = torch.arange(1, len(tokens) + 1, dtype=torch.float32)[:, None]
        return (torch.cumsum(y, dim=0) / counts) @ t["l1.mixer.mix.weight"].T

    # layer 0
    mixed, k0, v0 = attention("l0.attn.", plain.rms_norm(x, t["l0.n1.weight"], 1e-5))
    x = x + mixed
    y = plain.rms_norm(x, t["l0.n2.weight"], 1e-5)
    choice = torch.argmax(y @ t["l0.ffn.router.weight"].T, dim=-1)
    routed = torch.zeros_like(y)
    for e in range(3):
        rows = choice == e
        routed[rows] = torch.relu(y[rows] @ t[f"l0.ffn.experts.{e}.up.weight"].T) @ t[f"l0.ffn.experts.{e}.down.weight"].T
    x = x + routed
    # layer 1, twice
    for _ in range(2):
        x = x + running_mean(plain.rms_norm(x, t["l1.n1.weight"], 1e-5))
        x = x + swiglu("l1.mlp.", plain.rms_norm(x, t["l1.n2.weight"], 1e-5))
    # layer 2 reads layer 0's keys and values
    y = plain.rms_norm(x, t["l2.n1.weight"], 1e-5)
    q = plain.split_heads(y @ t["l2.attn.q_proj.weight"].T, 3, 16)
    mixed = plain.causal_attention(q, k0, v0).transpose(0, 1).reshape(len(tokens), 48)
    x = x + mixed @ t["l2.attn.o_proj.weight"].T + t["l2.attn.o_proj.bias"]
    x = x + swiglu("l2.mlp.", plain.rms_norm(x, t["l2.n2.weight"], 1e-5))
    return plain.rms_norm(x, t["final.weight"], 1e-5) @ t["embed.weight"].T
