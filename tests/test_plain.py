"""The plain implementation against the reference's own model code (committed golden outputs made
by tests/golden/make_reference_golden.py) and against hand-checked properties of each part."""

import os

import numpy as np
import torch

import plain_qwen2 as plain
from harness import random_prompt
from mini_llm_runtime_b200.models import build_model
from mini_llm_runtime_b200.weights import random_tensors
from tiny_configs import TINY_A, TINY_B, TINY_C, TINY_D

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def tensors_for(config, seed=5, dtype=torch.float32):
    return random_tensors(build_model(config, torch.float32).expected_tensors(), seed, dtype)


def test_tiny_a_matches_the_reference_runner():
    tensors = tensors_for(TINY_A)
    prompt = random_prompt(TINY_A.vocab_size, 33, 300)
    logits, layers = plain.forward_logits(tensors, TINY_A.to_dict(), prompt, return_layers=True)
    want_logits = torch.from_numpy(np.load(os.path.join(GOLDEN, "tiny_a_logits.npy")))
    want_layers = torch.from_numpy(np.load(os.path.join(GOLDEN, "tiny_a_layers.npy")))
    assert torch.allclose(torch.stack(layers), want_layers, atol=2e-6, rtol=1e-5)
    assert torch.allclose(logits, want_logits, atol=5e-6, rtol=1e-5)


def test_tiny_b_decoder_stack_matches_the_reference_layer_function():
    tensors = tensors_for(TINY_B)
    prompt = random_prompt(TINY_B.vocab_size, 40, 301)
    _, layers = plain.forward_logits(tensors, TINY_B.to_dict(), prompt, return_layers=True)
    want_layers = torch.from_numpy(np.load(os.path.join(GOLDEN, "tiny_b_layers.npy")))
    assert torch.allclose(torch.stack(layers), want_layers, atol=2e-6, rtol=1e-5)


def test_tiny_b_untied_head_is_the_reference_norm_times_the_head_matrix():
    tensors = tensors_for(TINY_B)
    prompt = random_prompt(TINY_B.vocab_size, 40, 301)
    logits = plain.forward_logits(tensors, TINY_B.to_dict(), prompt)
    want = torch.from_numpy(np.load(os.path.join(GOLDEN, "tiny_b_logits.npy")))
    assert torch.allclose(logits, want, atol=5e-6, rtol=1e-5)


def test_tiny_d_windowed_layers_match_the_reference_layer_function_under_a_window_mask():
    tensors = tensors_for(TINY_D)
    prompt = random_prompt(TINY_D.vocab_size, 150, 302)
    logits, layers = plain.forward_logits(tensors, TINY_D.to_dict(), prompt, return_layers=True)
    want_layers = torch.from_numpy(np.load(os.path.join(GOLDEN, "tiny_d_layers.npy")))
    want_logits = torch.from_numpy(np.load(os.path.join(GOLDEN, "tiny_d_logits.npy")))
    assert torch.allclose(torch.stack(layers)[:, 100:], want_layers, atol=5e-6, rtol=1e-5)
    assert torch.allclose(logits[-8:], want_logits, atol=1e-5, rtol=1e-5)
    # and the window matters there: without it the last layer's output differs
    no_window = dict(TINY_D.to_dict(), use_sliding_window=False)
    _, free = plain.forward_logits(tensors, no_window, prompt, return_layers=True)
    assert not torch.allclose(free[-1][100:], want_layers[-1], atol=1e-3)


def test_rms_norm_is_not_layer_norm():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]])
    weight = torch.tensor([1.0, 2.0, 1.0, 0.5])
    out = plain.rms_norm(x, weight, 1e-6)
    expected = weight * x / torch.sqrt(torch.tensor(50.0 / 4 + 1e-6))
    assert torch.allclose(out, expected, atol=1e-6)
    assert abs(float(out.mean())) > 0.1  # no mean-centering


def test_rotate_half_layout_and_identity_at_position_zero():
    x = torch.arange(8.0).reshape(1, 1, 8)
    assert plain.rotate_half(x).flatten().tolist() == [-4, -5, -6, -7, 0, 1, 2, 3]
    cos, sin = plain.rope_tables(torch.tensor([0]), 8, 10000.0)
    assert torch.equal(plain.apply_rope(x, cos, sin), x)
    cos, sin = plain.rope_tables(torch.tensor([3]), 8, 10000.0)
    rotated = plain.apply_rope(x, cos, sin)
    assert torch.allclose(rotated.norm(), x.norm(), atol=1e-5)  # a rotation keeps the length
    assert torch.allclose(cos[0, :4], cos[0, 4:])  # the D/2 angles are repeated


def test_attention_is_causal_and_groups_adjacent_heads():
    generator = torch.Generator().manual_seed(0)
    q = torch.randn(4, 6, 8, generator=generator)
    k = torch.randn(2, 6, 8, generator=generator)
    v = torch.randn(2, 6, 8, generator=generator)
    out = plain.causal_attention(q, k, v)
    assert torch.allclose(out[:, 0], v.repeat_interleave(2, dim=0)[:, 0])  # first row sees only itself
    changed = v.clone()
    changed[:, 5] += 1.0  # the future of rows 0..4
    assert torch.equal(plain.causal_attention(q, k, changed)[:, :5], out[:, :5])
    changed = v.clone()
    changed[1] += 1.0  # kv head 1 serves query heads 2 and 3 only
    again = plain.causal_attention(q, k, changed)
    assert torch.equal(again[:2], out[:2]) and not torch.equal(again[2:], out[2:])


def test_window_hides_old_keys():
    generator = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(1, 10, 4, generator=generator) for _ in range(3))
    windowed = plain.causal_attention(q, k, v, window=3)
    changed = v.clone()
    changed[:, 0:5] += 5.0
    again = plain.causal_attention(q, k, changed, window=3)
    assert torch.equal(again[:, 7:], windowed[:, 7:])      # rows 7.. see keys 5.. only
    assert not torch.equal(again[:, 6], windowed[:, 6])    # row 6 still sees key 4
    assert torch.allclose(plain.causal_attention(q, k, v, window=100), plain.causal_attention(q, k, v))


def test_layer_window_follows_max_window_layers():
    cfg = TINY_C.to_dict()
    assert [plain.layer_window(cfg, i) for i in range(4)] == [None, None, 21, 21]
    assert plain.layer_window(TINY_A.to_dict(), 0) is None


def test_untied_head_and_greedy_recompute():
    tensors = tensors_for(TINY_B, dtype=torch.bfloat16)
    prompt = random_prompt(TINY_B.vocab_size, 9, 2)
    logits = plain.forward_logits(tensors, TINY_B.to_dict(), prompt)
    assert logits.shape == (9, TINY_B.vocab_size)
    tied = dict(TINY_B.to_dict(), tie_word_embeddings=True)
    assert not torch.allclose(logits, plain.forward_logits(tensors, tied, prompt))
    produced = plain.greedy_tokens(tensors, TINY_B.to_dict(), prompt, 3)
    assert produced[0] == int(torch.argmax(logits[-1])) and len(produced) == 3


def test_plain_sampler():
    assert 0.0 <= plain.uniform_from_seed(7, 0) < 1.0
    assert plain.uniform_from_seed(7, 0) != plain.uniform_from_seed(7, 1) != plain.uniform_from_seed(8, 1)
    logits = torch.tensor([0.0, 0.0, 10.0, 0.0])
    assert plain.temperature_sample(logits, 1.0, 0.5)[0] == 2
    assert plain.temperature_sample(logits, 1.0, 0.0)[0] == 0
    assert plain.temperature_sample(logits, 1.0, 0.99999)[0] in (2, 3)
