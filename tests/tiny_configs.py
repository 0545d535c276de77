"""Tiny configurations of the architecture for the tests, and their workloads.

The first three differ in every size and option: layers, width, heads and groups
(4:1, 6:2, 5:5), head size (16, 32, 48), feed-forward width, vocabulary (one a
prime), rotary base, norm eps, tied or untied head, window (none, none, 40 keys
on two of three layers), page size.  Sizes that are no power of two: 96, 224,
384, 80, 136, 331, 6 and 5 heads, head size 48.
"""

import random

from tinyvllm_b200.models import Qwen3Config

TINY_CONFIGS = {
    "a": Qwen3Config(
        vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=1, head_dim=16, max_position_embeddings=1024,
        rope_theta=10_000.0, rms_norm_eps=1e-6, tie_word_embeddings=True),
    "b": Qwen3Config(
        vocab_size=384, hidden_size=96, intermediate_size=224, num_hidden_layers=3,
        num_attention_heads=6, num_key_value_heads=2, head_dim=32, max_position_embeddings=2048,
        rope_theta=1_000_000.0, rms_norm_eps=1e-5, tie_word_embeddings=False),
    "c": Qwen3Config(
        vocab_size=331, hidden_size=80, intermediate_size=136, num_hidden_layers=3,
        num_attention_heads=5, num_key_value_heads=5, head_dim=48, max_position_embeddings=1536,
        rope_theta=500_000.0, rms_norm_eps=3e-6, tie_word_embeddings=False,
        layer_windows=(40, None, 40)),
    # head sizes the tiled bfloat16 kernels take: 64 (groups of 2, a window) and 128 (groups of 4)
    "d": Qwen3Config(
        vocab_size=211, hidden_size=128, intermediate_size=192, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, head_dim=64, max_position_embeddings=1024,
        rope_theta=100_000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
        layer_windows=(None, 100)),
    "e": Qwen3Config(
        vocab_size=300, hidden_size=160, intermediate_size=256, num_hidden_layers=2,
        num_attention_heads=8, num_key_value_heads=2, head_dim=128, max_position_embeddings=1024,
        rope_theta=1_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=False),
}
SEEDS = {"a": 0, "b": 1, "c": 2, "d": 3, "e": 4}
PAGE_SIZES = {"a": 4, "b": 8, "c": 16, "d": 16, "e": 32}


def random_tokens(vocab: int, count: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(count)]


# what tests/golden/make_golden.py runs through the reference's own code
GOLDEN_WORKLOADS = {
    "a": {"seed": 0, "page_size": 4, "pages": 24, "chunk": 5, "new_tokens": 8,
          "prompts": [random_tokens(256, n, 100 + n) for n in (1, 7, 19)]},
    "b": {"seed": 1, "page_size": 8, "pages": 40, "chunk": 7, "new_tokens": 12,
          "prompts": [random_tokens(384, n, 200 + n) for n in (3, 16, 31, 50)]},
}
