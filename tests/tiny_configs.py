"""The tiny configurations every test uses.  A and B are the two the benchmark description
names; they differ in every size and option.  C adds what neither has: a sliding window on some
layers (two cache groups), a head_dim that config.json gives explicitly and that differs from
hidden/heads, and a page size that does not divide the window."""

from mini_llm_runtime_b200.config import Qwen2Config

TINY_A = Qwen2Config(
    vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
    num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512,
    rms_norm_eps=1e-6, rope_theta=10000.0, hidden_act="silu", tie_word_embeddings=True)
PAGE_A = 16

TINY_B = Qwen2Config(
    vocab_size=384, hidden_size=96, intermediate_size=200, num_hidden_layers=3,
    num_attention_heads=3, num_key_value_heads=1, max_position_embeddings=1024,
    rms_norm_eps=1e-5, rope_theta=1000000.0, hidden_act="silu", tie_word_embeddings=False)
PAGE_B = 8

TINY_C = Qwen2Config(
    vocab_size=203, hidden_size=80, intermediate_size=112, num_hidden_layers=4,
    num_attention_heads=6, num_key_value_heads=3, max_position_embeddings=640,
    rms_norm_eps=3e-6, rope_theta=50000.0, hidden_act="silu", tie_word_embeddings=False,
    head_dim=48, use_sliding_window=True, sliding_window=21, max_window_layers=2)
PAGE_C = 16

TINY = {"A": (TINY_A, PAGE_A), "B": (TINY_B, PAGE_B), "C": (TINY_C, PAGE_C)}
