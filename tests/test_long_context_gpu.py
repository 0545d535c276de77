"""A context of several thousand tokens: prompt portions of 2,048 tokens (as the scheduler cuts
them) and then decoded tokens, against the whole-sequence oracle.  The attention kernels walk
dozens of key blocks and chunk edges here, the decode kernel cuts its keys into pieces of more
than a thousand, and one layer's window lets go of most pages on the way."""

import pytest
import torch

import replay_helpers as rh
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu

LENGTH = 9000
TAIL = 24


def long_config():
    from tinyvllm_b200.models import Qwen3Config

    return Qwen3Config(vocab_size=200, hidden_size=128, intermediate_size=192, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=16384,
                       rope_theta=1_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                       layer_windows=(None, 700))


@pytest.fixture(scope="module")
def long_folder(tmp_path_factory):
    from tinyvllm_b200.weights.random_init import write_model_folder

    return write_model_folder(tmp_path_factory.mktemp("long"), long_config(), seed=77)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_long_context_prefill_in_portions_then_decode(dtype, long_folder):
    from tinyvllm_b200.config.registry import read_model_config
    from tinyvllm_b200.engine.model import Model
    from tinyvllm_b200.engine.step import StepRunner

    tokens = random_tokens(200, LENGTH, 5)
    requests = {"long": tokens}
    steps = []
    place = 0
    while place < LENGTH - TAIL:
        count = min(2048, LENGTH - TAIL - place)
        # logits at the first, a middle and the last places of every portion
        want = sorted({0, 1, count // 2, count - 2, count - 1})
        steps.append({"step": len(steps), "entries": [{"id": "long", "tokens": tokens[place:place + count],
                                                       "want": want}], "end": []})
        place += count
    for position in range(place, LENGTH):
        steps.append({"step": len(steps), "entries": [{"id": "long", "tokens": [tokens[position]], "want": [0]}],
                      "end": ["long"] if position == LENGTH - 1 else []})
    model = Model(read_model_config(long_folder).to_spec(), device="cuda:0", dtype=dtype).load(long_folder)
    runner = StepRunner(model, page_size=16, num_pages=-(-LENGTH // 16) + 2, max_requests=2)
    with torch.inference_mode():
        got = rh.run_steps(runner, steps)
    assert len(got) == 5 * 5 + TAIL
    # the windowed layer's group gave back the pages its window had passed while the request ran
    assert all(pool.free_count == pool.num_pages for pool in runner.manager.pools)
    expected = rh.oracle(long_folder, requests, dtype, positions=rh.wanted_positions(steps))
    rh.compare(got, expected, dtype, what="long context")
