"""The stream-k tcgen05 product inside the engine.  The launcher gives it weights of 400 MB and more,
which no test model has; here the threshold is taken away, so that every bfloat16 product of 17 to
64 rows, the gate/up product with its activation and the float32 head go through it, and the logits
are compared with the oracle for whole prompts, portions, decoded tails and mixed batches."""

import pytest
import torch

import replay_helpers as rh
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(64, 136, 4, 2, 16, 300), (264, 520, 6, 2, 64, 1031)],
                         ids=["h64", "h264"])
def test_products_through_the_stream_kernel(shape, tmp_path, monkeypatch):
    from tinyvllm_b200.config.registry import read_model_config
    from tinyvllm_b200.engine.model import Model
    from tinyvllm_b200.engine.step import StepRunner
    from tinyvllm_b200.models import Qwen3Config
    from tinyvllm_b200.ops import gemm, kernels
    from tinyvllm_b200.weights.random_init import write_model_folder

    hidden, inter, heads, kv_heads, head_dim, vocab = shape
    config = Qwen3Config(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=2,
                         num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
                         max_position_embeddings=512, rope_theta=10000.0, rms_norm_eps=1e-6,
                         tie_word_embeddings=False)
    folder = write_model_folder(tmp_path / "model", config, seed=hidden)
    model = Model(read_model_config(folder).to_spec(), device="cuda:0", dtype=torch.bfloat16).load(folder)
    runner = StepRunner(model, page_size=16, num_pages=80, max_requests=6)
    requests = {f"r{n}": random_tokens(vocab, n, n) for n in (20, 33, 64, 50, 47)}
    expected = rh.oracle(folder, requests, torch.bfloat16)
    monkeypatch.setattr(gemm, "STREAM_MIN_WEIGHT_BYTES", 0)
    calls = []
    real = kernels.gemm_stream
    monkeypatch.setattr(kernels, "gemm_stream", lambda *a, **k: (calls.append(a[2] if len(a) > 2 else k.get("mode", 0)),
                                                                 real(*a, **k))[1])
    for mode, steps in (("whole", rh.whole(requests)), ("portions", rh.portions(requests, seed=2, sizes=(17, 20, 31))),
                        ("tail", rh.tail_by_one(requests, tail=6)), ("mixed", rh.mixed(requests, seed=3))):
        with torch.inference_mode():
            got = rh.run_steps(runner, steps)
        rh.compare(got, expected, torch.bfloat16, what=f"stream {shape} {mode}")
    assert kernels.gemm_stream_status() == 0
    # bfloat16 products, the activation and the float32 head all went that way
    assert {kernels.GEMM_BF16, kernels.GEMM_F32, kernels.GEMM_SILU} <= set(calls)
    assert all(pool.free_count == pool.num_pages for pool in runner.manager.pools)
