"""Sizes that are no power of two, end to end: whatever config.json allows either runs right or is
refused with a clear error, in 32-bit and in bfloat16, for whole prompts, decoded tails and mixed
batches.  Head sizes in steps of 16 that no tiled kernel takes (80, 112, 144, 240), groups of 3, 5
and 7 query heads, widths whose rows are no whole number of 16-byte words (66, 90, 100), odd
vocabularies, pages of 5 tokens, a window on one of two layers."""

import pytest
import torch

import replay_helpers as rh
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu

# hidden, intermediate, q heads, kv heads, head size, vocabulary, page size, window of the first layer
SHAPES = [
    (72, 100, 3, 3, 16, 257, 4, None),
    (90, 130, 6, 2, 80, 301, 8, None),
    (100, 200, 5, 1, 112, 199, 16, 33),
    (136, 264, 7, 7, 144, 513, 32, None),
    (200, 312, 10, 2, 240, 1000, 16, None),
    (1000, 1504, 6, 2, 128, 777, 16, None),
    (264, 520, 9, 3, 64, 1031, 16, 70),
    (96, 96, 2, 1, 256, 130, 64, None),
    (66, 70, 2, 2, 32, 97, 5, None),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("shape", SHAPES, ids=[f"h{s[0]}-{s[2]}x{s[4]}" for s in SHAPES])
def test_odd_sizes_run_right(shape, dtype, tmp_path):
    from tinyvllm_b200.config.registry import read_model_config
    from tinyvllm_b200.engine.model import Model
    from tinyvllm_b200.engine.step import StepRunner
    from tinyvllm_b200.models import Qwen3Config
    from tinyvllm_b200.weights.random_init import write_model_folder

    hidden, inter, heads, kv_heads, head_dim, vocab, page, window = shape
    config = Qwen3Config(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=2,
                         num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
                         max_position_embeddings=1024, rope_theta=10000.0, rms_norm_eps=1e-6,
                         tie_word_embeddings=vocab % 2 == 1, layer_windows=(window, None) if window else None)
    folder = write_model_folder(tmp_path / "model", config, seed=hidden)
    model = Model(read_model_config(folder).to_spec(), device="cuda:0", dtype=dtype).load(folder)
    runner = StepRunner(model, page_size=page, num_pages=-(-2000 // page), max_requests=8)
    requests = {f"r{n}": random_tokens(vocab, n, n) for n in (1, 9, 70, 300, 130)}
    expected = rh.oracle(folder, requests, dtype)
    for mode, steps in (("whole", rh.whole(requests)), ("tail", rh.tail_by_one(requests, tail=12)),
                        ("mixed", rh.mixed(requests, seed=3))):
        with torch.inference_mode():
            got = rh.run_steps(runner, steps)
        rh.compare(got, expected, dtype, what=f"{shape} {mode}")
    assert all(pool.free_count == pool.num_pages for pool in runner.manager.pools)


def test_sizes_no_kernel_takes_are_refused_clearly(tmp_path):
    from tinyvllm_b200.config.registry import read_model_config
    from tinyvllm_b200.engine.model import Model
    from tinyvllm_b200.models import Qwen3Config

    for head_dim, message in ((24, "steps of 16"), (272, "up to 256")):
        config = Qwen3Config(vocab_size=64, hidden_size=48, intermediate_size=64, num_hidden_layers=1,
                             num_attention_heads=2, num_key_value_heads=1, head_dim=head_dim,
                             max_position_embeddings=64, rope_theta=10000.0, rms_norm_eps=1e-6,
                             tie_word_embeddings=True)
        with pytest.raises(ValueError, match=message):
            Model(config.to_spec(), device="cuda:0", dtype=torch.bfloat16)
