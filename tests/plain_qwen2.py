"""Plain, slow Qwen2 decoder used as the oracle of every engine test.

Whole sequences only, no cache, one function per part, float32 on the CPU (or on
whatever device the tensors live on).  It shares no code with the package: it reads
the Hugging Face tensor names straight out of a ``dict`` and the sizes out of the
``config.json`` dictionary.

Every function restates a formula of the reference project
(``src/mini_llm_runtime/qwen_model_runner.py`` unless another file is named) and
cites the lines it was written from.  ``tests/golden/make_reference_golden.py``
compared this file once with the reference's own importable model code on a tiny
random model; the committed outputs live beside that script.

Two things here have no counterpart in the reference and rest on formulas only:
the untied ``lm_head`` (the reference rejects ``tie_word_embeddings=false`` at
``src/mini_llm_runtime/qwen_config.py:43-44``) and the sliding window (the reference
never reads ``sliding_window``); the window rule used is "a query at position p sees
the keys at positions p-window+1 .. p".
"""

from __future__ import annotations

import math

import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """qwen_model_runner.py:22-26 — x * rsqrt(mean(x^2) + eps) * w, eps inside the root."""
    x32 = x.float()
    variance = (x32 * x32).mean(dim=-1, keepdim=True)
    return weight.float() * (x32 * torch.rsqrt(variance + eps))


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float):
    """qwen_model_runner.py:45-57 — inv_freq[i] = theta^(-2i/D); angle = pos * inv_freq;
    the table repeats the D/2 angles twice (rotate-half layout)."""
    exponents = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    inv_freq = 1.0 / (theta ** exponents)
    angles = positions.float().unsqueeze(-1) * inv_freq.to(positions.device)
    table = torch.cat((angles, angles), dim=-1)
    return table.cos(), table.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """qwen_model_runner.py:34-36 — (x1, x2) -> (-x2, x1) with x1 the first half."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """qwen_model_runner.py:58-61 — x*cos + rotate_half(x)*sin; x is [heads, S, D]."""
    return x * cos.unsqueeze(0) + rotate_half(x) * sin.unsqueeze(0)


def split_heads(x: torch.Tensor, heads: int, head_dim: int) -> torch.Tensor:
    """qwen_model_runner.py:29-31 — [S, heads*D] -> [heads, S, D]; head h owns columns h*D.."""
    return x.reshape(x.shape[0], heads, head_dim).transpose(0, 1)


def causal_attention(q, k, v, *, window: int | None = None) -> torch.Tensor:
    """qwen_model_runner.py:64-72,157-177 — GQA by repeating each kv head over its group of
    adjacent query heads; scores = q k^T / sqrt(D); future keys masked; softmax in float32.
    q is [Hq, S, D], k and v are [Hkv, S, D]; all S tokens belong to one request.
    ``window`` (not in the reference) also masks keys older than p-window+1."""
    heads, length, head_dim = q.shape
    group = heads // k.shape[0]
    k = k.repeat_interleave(group, dim=0)
    v = v.repeat_interleave(group, dim=0)
    scores = torch.matmul(q, k.transpose(-2, -1)) / math.sqrt(head_dim)
    query_pos = torch.arange(length, device=q.device).unsqueeze(1)
    key_pos = torch.arange(length, device=q.device).unsqueeze(0)
    hidden = key_pos > query_pos
    if window is not None:
        hidden = hidden | (key_pos <= query_pos - window)
    scores = scores.masked_fill(hidden, float("-inf"))
    probabilities = torch.softmax(scores.float(), dim=-1)
    return torch.matmul(probabilities, v)


def attention_block(x, positions, tensors, prefix, cfg, *, window=None) -> torch.Tensor:
    """qwen_model_runner.py:88-103,178-183 — biased q/k/v projections, RoPE on q and k (not v),
    causal GQA attention, heads merged back to [S, Hq*D], o_proj without bias."""
    heads = cfg["num_attention_heads"]
    kv_heads = cfg["num_key_value_heads"]
    head_dim = cfg.get("head_dim") or cfg["hidden_size"] // heads
    p = prefix + ".self_attn."

    def linear(name, inp, bias=True):
        out = inp @ tensors[p + name + ".weight"].float().T
        if bias:
            out = out + tensors[p + name + ".bias"].float()
        return out

    q = split_heads(linear("q_proj", x), heads, head_dim)
    k = split_heads(linear("k_proj", x), kv_heads, head_dim)
    v = split_heads(linear("v_proj", x), kv_heads, head_dim)
    cos, sin = rope_tables(positions, head_dim, cfg["rope_theta"])
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    mixed = causal_attention(q, k, v, window=window)
    merged = mixed.transpose(0, 1).reshape(x.shape[0], heads * head_dim)
    return merged @ tensors[p + "o_proj.weight"].float().T


def swiglu_mlp(x, tensors, prefix) -> torch.Tensor:
    """qwen_model_runner.py:215-217 — down(silu(gate(x)) * up(x)), no biases."""
    p = prefix + ".mlp."
    gate = x @ tensors[p + "gate_proj.weight"].float().T
    up = x @ tensors[p + "up_proj.weight"].float().T
    return (torch.nn.functional.silu(gate) * up) @ tensors[p + "down_proj.weight"].float().T


def layer_window(cfg: dict, layer: int) -> int | None:
    """Not in the reference.  Qwen2's config.json keys: with ``use_sliding_window`` the layers
    from ``max_window_layers`` on see only the last ``sliding_window`` keys."""
    if not cfg.get("use_sliding_window", False):
        return None
    if layer < cfg.get("max_window_layers", 0):
        return None
    return int(cfg["sliding_window"])


def decoder_layer(x, positions, tensors, layer, cfg) -> torch.Tensor:
    """qwen_model_runner.py:199-218 — h = x + attn(norm(x)); out = h + mlp(norm(h))."""
    prefix = f"model.layers.{layer}"
    eps = cfg["rms_norm_eps"]
    normed = rms_norm(x, tensors[prefix + ".input_layernorm.weight"], eps)
    h = x + attention_block(normed, positions, tensors, prefix, cfg, window=layer_window(cfg, layer))
    normed = rms_norm(h, tensors[prefix + ".post_attention_layernorm.weight"], eps)
    return h + swiglu_mlp(normed, tensors, prefix)


def forward_logits(tensors: dict, cfg: dict, token_ids, *, return_layers: bool = False, rows=None):
    """qwen_model_runner.py:263-290 — embedding gather, the layers in order, final norm, then
    logits = x @ E^T (tied) or x @ lm_head^T (untied; ours).  Returns [S, vocab] float32 for
    one request given whole; every position's logits (``rows``: only those positions')."""
    table = tensors["model.embed_tokens.weight"]
    ids = torch.as_tensor(token_ids, dtype=torch.long, device=table.device)
    x = table[ids].float()
    positions = torch.arange(ids.shape[0], device=table.device)
    captured = []
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, positions, tensors, layer, cfg)
        captured.append(x)
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long, device=x.device)]
    x = rms_norm(x, tensors["model.norm.weight"], cfg["rms_norm_eps"])
    head = tensors["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else tensors["lm_head.weight"]
    logits = x @ head.float().T
    return (logits, captured) if return_layers else logits


def greedy_tokens(tensors: dict, cfg: dict, prompt, steps: int) -> list[int]:
    """tests/test_generation.py:14-28 of the reference — every step recomputes the whole
    sequence; argmax picks the lowest index on ties."""
    sequence = list(prompt)
    produced = []
    for _ in range(steps):
        logits = forward_logits(tensors, cfg, sequence)[-1]
        token = int(torch.argmax(logits))
        produced.append(token)
        sequence.append(token)
    return produced


def uniform_from_seed(seed: int, index: int) -> float:
    """The sampler's counter-based generator (ours; the reference samples greedily only,
    engine.py:222,246): splitmix64 of seed + (index+1) * golden ratio, top 24 bits / 2^24."""
    mask = (1 << 64) - 1
    z = (seed + (index + 1) * 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def temperature_sample(logits: torch.Tensor, temperature: float, uniform: float):
    """Ours: p = softmax(logits / T) in float32; the token is the first index whose
    cumulative probability exceeds uniform.  Returns (token, cdf) for boundary checks."""
    probabilities = torch.softmax(logits.float() / temperature, dim=-1)
    cdf = torch.cumsum(probabilities.double(), dim=-1)
    token = int(torch.searchsorted(cdf, torch.tensor(uniform, dtype=torch.float64), right=True))
    return min(token, logits.shape[-1] - 1), cdf
