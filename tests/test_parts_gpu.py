"""Each part of the decoder alone on the GPU, built from a ``PartSpec`` exactly as the model builds
it, against the plain function of the same part (``plain_qwen2``): norm (alone and fused with the
residual add), position encoding with the cache write, the attention mixer (whole prompt, then
continued from the cache), the feed-forward in both weight layouts, embedding, both heads, and the
pre-norm block.  Sizes differ from the tiny engines' and are no powers of two."""

from __future__ import annotations

import types

import pytest
import torch

import plain_qwen2 as plain
from harness import assert_close
from mini_llm_runtime_b200.cache import CacheManager
from mini_llm_runtime_b200.config import PartSpec
from mini_llm_runtime_b200.engine import ModelRunner, StepEntry
from mini_llm_runtime_b200.parts import build_part, part_factory

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def rnd(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


def stored(tensors):
    """Round to bfloat16 as a checkpoint would store them; the plain side reads the same values."""
    return {name: value.to(torch.bfloat16) for name, value in tensors.items()}


def context_for(need, dtype, tokens_per_step, page=8, mixer=None):
    """A cache for one entry and a function that opens a step of ``n`` rows for request "r".  The
    stand-in model has the one ``mixer`` (if any), so that the step carries its work lists."""
    cache = CacheManager([need], page_size=page, num_pages=32, max_requests=2, max_tokens_per_request=200,
                         dtype=dtype, device=DEVICE)
    blocks = [types.SimpleNamespace(mixer=mixer)] if mixer is not None else []
    stub = types.SimpleNamespace(device=torch.device(DEVICE), parts=lambda: [], blocks=blocks,
                                 spec=types.SimpleNamespace(vocab_size=1000, max_positions=4096))
    runner = ModelRunner(stub, cache)
    cache.create_request("r")

    def open_step(count):
        requests = cache.begin_step([("r", count)])
        return runner._build_context([StepEntry("r", [0] * count, [])], requests)

    return cache, open_step


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_part(dtype):
    spec = PartSpec("rms_norm", {"size": 200, "eps": 3e-5}, "n.")
    part = build_part("norm", spec, dtype)
    tensors = stored({"n.weight": 1 + rnd((200,), 1, 0.1)})
    assert set(part.tensors()) == {"n.weight"} and part.tensors()["n.weight"].shape == (200,)
    part.load(tensors, torch.device(DEVICE))
    x = rnd((7, 200), 2, 2.0).to(dtype)
    assert_close(part.forward(x.to(DEVICE)), plain.rms_norm(x, tensors["n.weight"], 3e-5), dtype, "norm")
    residual, delta = x.clone().to(DEVICE), rnd((7, 200), 3).to(dtype)
    got = part.add_forward(residual, delta.to(DEVICE))
    summed = (x.float() + delta.float()).to(dtype)
    assert torch.equal(residual.cpu(), summed)
    assert_close(got, plain.rms_norm(summed, tensors["n.weight"], 3e-5), dtype, "add + norm")


@pytest.mark.parametrize("dtype", DTYPES)
def test_rope_part_rotates_and_stores(dtype):
    from mini_llm_runtime_b200.parts import KVCacheNeed

    heads, kv_heads, head_dim, theta = 3, 1, 48, 50000.0
    part = build_part("position", PartSpec("rope_half", {"head_dim": head_dim, "theta": theta}), dtype)
    part.load({}, torch.device(DEVICE))
    cache, open_step = context_for(KVCacheNeed(kv_heads, head_dim), dtype, 13)
    ctx = open_step(13)
    qkv = rnd((13, (heads + 2 * kv_heads) * head_dim), 4).to(dtype)
    q = part.rotate_and_store(qkv.to(DEVICE), ctx, ctx.cache_view(0), heads, kv_heads, head_dim, True)
    cache.commit_step()
    split = qkv.float().view(13, heads + 2 * kv_heads, head_dim).transpose(0, 1)
    cos, sin = plain.rope_tables(torch.arange(13), head_dim, theta)
    want_q = plain.apply_rope(split[:heads], cos, sin).transpose(0, 1).reshape(13, -1)
    want_k = plain.apply_rope(split[heads:heads + kv_heads], cos, sin)
    assert_close(q, want_q, dtype, "rotated q")
    k_pool, v_pool, group = cache.entry_pools(0)
    pages = cache.get("r").pages[0]
    stored_k = torch.cat([k_pool[p] for p in pages], dim=1)[:, :13].float().cpu()     # [kv_heads, tokens, D]
    stored_v = torch.cat([v_pool[p] for p in pages], dim=1)[:, :13].float().cpu()
    assert_close(stored_k.reshape(13 * kv_heads, -1), want_k.reshape(13 * kv_heads, -1), dtype, "k in the pages")
    assert torch.equal(stored_v, split[heads + kv_heads:].to(dtype).float()), "v is stored unrotated"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 9])
def test_attention_mixer_whole_and_continued(dtype, window):
    hidden, heads, kv_heads, head_dim = 72, 6, 2, 16
    args = {"hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": head_dim,
            "qkv_bias": True, "out_bias": False, "window": window,
            "position": PartSpec("rope_half", {"head_dim": head_dim, "theta": 10000.0})}
    part = build_part("mixer", PartSpec("gqa_attention", args, "a."), dtype)
    tensors = stored({"a.q_proj.weight": rnd((96, hidden), 5, 0.2), "a.q_proj.bias": rnd((96,), 6, 0.2),
                      "a.k_proj.weight": rnd((32, hidden), 7, 0.2), "a.k_proj.bias": rnd((32,), 8, 0.2),
                      "a.v_proj.weight": rnd((32, hidden), 9, 0.2), "a.v_proj.bias": rnd((32,), 10, 0.2),
                      "a.o_proj.weight": rnd((hidden, 96), 11, 0.2)})
    assert set(part.tensors()) == set(tensors)
    part.load(tensors, torch.device(DEVICE))
    need = part.cache_need()
    assert (need.num_kv_heads, need.head_dim, need.window) == (kv_heads, head_dim, window)
    cache, open_step = context_for(need, dtype, 30, mixer=part)
    x = rnd((30, hidden), 12).to(dtype)
    cfg = {"num_attention_heads": heads, "num_key_value_heads": kv_heads, "hidden_size": hidden,
           "head_dim": head_dim, "rope_theta": 10000.0}
    plain_tensors = {"L.self_attn." + name[2:]: value for name, value in tensors.items()}
    want = plain.attention_block(x.float(), torch.arange(30), plain_tensors, "L", cfg, window=window)
    outputs = []
    for start, count in ((0, 17), (17, 1), (18, 12)):      # a portion, one decoded token, another portion
        ctx = open_step(count)
        outputs.append(part.forward(x[start:start + count].to(DEVICE), ctx, ctx.cache_view(0), True))
        cache.commit_step()
    assert_close(torch.cat(outputs), want, dtype, f"attention mixer window={window}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,inner", [(72, 104), (64, 192)])
def test_swiglu_part(dtype, hidden, inner):
    part = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inner}, "m."), dtype)
    tensors = stored({"m.gate_proj.weight": rnd((inner, hidden), 13, 0.3), "m.up_proj.weight": rnd((inner, hidden), 14, 0.3),
                      "m.down_proj.weight": rnd((hidden, inner), 15, 0.3)})
    part.load(tensors, torch.device(DEVICE))
    assert part.block == (64 if inner % 64 == 0 else inner)
    x = rnd((11, hidden), 16).to(dtype)
    plain_tensors = {"L.mlp." + name[2:]: value for name, value in tensors.items()}
    assert_close(part.forward(x.to(DEVICE), None), plain.swiglu_mlp(x.float(), plain_tensors, "L"), dtype, "swiglu")


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_heads(dtype):
    sizes = {"vocab_size": 203, "hidden_size": 40}
    embedding = build_part("embedding", PartSpec("token_embedding", sizes, "e."), dtype)
    table = stored({"e.weight": rnd((203, 40), 17)})
    embedding.load(table, torch.device(DEVICE))
    ids = torch.tensor([0, 202, 17, 17], dtype=torch.int32)
    rows = embedding.forward(ids.to(DEVICE))
    assert torch.equal(rows.float().cpu(), table["e.weight"].float()[ids.long()].to(dtype).float())
    x = rnd((5, 40), 18).to(dtype)
    tied = build_part("head", PartSpec("tied_head", sizes, "h."), dtype)
    tied.load({"model.embed_tokens.weight": table["e.weight"]}, torch.device(DEVICE))
    logits = tied.forward(x.to(DEVICE), embedding)
    assert logits.dtype == torch.float32
    assert_close(logits, x.float() @ table["e.weight"].float().T, dtype, "tied head")
    separate = build_part("head", PartSpec("linear_head", sizes, "h."), dtype)
    weight = stored({"h.weight": rnd((203, 40), 19)})
    separate.load(weight, torch.device(DEVICE))
    assert_close(separate.forward(x.to(DEVICE), embedding), x.float() @ weight["h.weight"].float().T, dtype, "untied head")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [21, 6])
def test_pre_norm_block(dtype, rows):
    """21 rows take the arrangement with norm kernels, 6 rows (in bfloat16, after the norms'
    weights were folded into the projections) the one where the products normalise and add."""
    hidden, heads, kv_heads, head_dim, inner, eps = 48, 3, 3, 16, 80, 1e-5
    mixer = build_part("mixer", PartSpec("gqa_attention", {
        "hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": head_dim, "qkv_bias": True,
        "out_bias": False, "window": None, "position": PartSpec("rope_half", {"head_dim": head_dim, "theta": 1e6})},
        "model.layers.0.self_attn."), dtype)
    feed_forward = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inner},
                                                       "model.layers.0.mlp."), dtype)
    norm1 = build_part("norm", PartSpec("rms_norm", {"size": hidden, "eps": eps}, "model.layers.0.input_layernorm."), dtype)
    norm2 = build_part("norm", PartSpec("rms_norm", {"size": hidden, "eps": eps},
                                        "model.layers.0.post_attention_layernorm."), dtype)
    block = part_factory("block", "pre_norm_residual")(mixer, feed_forward, norm1, norm2)
    tensors = {}
    for index, part in enumerate(block.parts()):
        for name, spec in part.tensors().items():
            base = rnd(spec.shape, 30 + len(tensors), 0.1)
            tensors[name] = base + 1 if spec.init == "norm" else base
    tensors = stored(tensors)
    for part in block.parts():
        part.load(tensors, torch.device(DEVICE))
    block.finish_load(dtype)
    assert block.folded == (dtype == torch.bfloat16)
    cache, open_step = context_for(mixer.cache_need(), dtype, rows, mixer=mixer)
    x = rnd((rows, hidden), 40).to(dtype)
    ctx = open_step(rows)
    residual, pending = block.forward(x.clone().to(DEVICE), None, ctx, ctx.cache_view(0), True)
    cache.commit_step()
    if pending is None:
        assert block.folded and rows <= 16
        pending = torch.zeros_like(residual)
    cfg = {"num_attention_heads": heads, "num_key_value_heads": kv_heads, "hidden_size": hidden, "head_dim": head_dim,
           "rope_theta": 1e6, "rms_norm_eps": eps, "num_hidden_layers": 1}
    want = plain.decoder_layer(x.float(), torch.arange(rows), tensors, 0, cfg)
    assert_close(residual.float() + pending.float(), want, dtype, "pre-norm block")
