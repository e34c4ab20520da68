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

# D and E have the head sizes (64, 128) and page sizes (powers of two) that the tensor-core attention
# kernels with bulk-copy loaders take, an intermediate size that is a multiple of 64 (gate and up
# interleaved for the fused SwiGLU epilogue), and widths that are multiples of 8 (tensor-core
# products); D has a window on its second layer, E has no grouping (one query head per kv head).
TINY_D = Qwen2Config(
    vocab_size=328, hidden_size=192, intermediate_size=256, num_hidden_layers=2,
    num_attention_heads=3, num_key_value_heads=1, max_position_embeddings=768,
    rms_norm_eps=1e-6, rope_theta=100000.0, hidden_act="silu", tie_word_embeddings=True,
    head_dim=64, use_sliding_window=True, sliding_window=70, max_window_layers=1)
PAGE_D = 16

TINY_E = Qwen2Config(
    vocab_size=264, hidden_size=160, intermediate_size=192, num_hidden_layers=2,
    num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=512,
    rms_norm_eps=1e-5, rope_theta=10000.0, hidden_act="silu", tie_word_embeddings=False,
    head_dim=128)
PAGE_E = 32

TINY = {"A": (TINY_A, PAGE_A), "B": (TINY_B, PAGE_B), "C": (TINY_C, PAGE_C), "D": (TINY_D, PAGE_D),
        "E": (TINY_E, PAGE_E)}
