"""Properties of the plain implementation itself.  No GPU."""

import math

import torch

import plain_qwen3 as plain
from tiny_configs import random_tokens


def test_logits_at_a_position_do_not_depend_on_later_tokens(model_folders):
    for name in ("a", "c"):
        cfg, weights = plain.read_config(model_folders[name]), plain.read_weights(model_folders[name])
        tokens = random_tokens(cfg["V"], 90, 4)
        full = plain.forward(cfg, weights, tokens)
        short = plain.forward(cfg, weights, tokens[:50])
        assert torch.allclose(full[:50], short, atol=1e-6, rtol=1e-5)


def test_window_limits_what_a_query_sees():
    torch.manual_seed(0)
    q, k, v = torch.randn(12, 2, 8), torch.randn(12, 1, 8), torch.randn(12, 1, 8)
    full = plain.causal_attention(q, k, v, 0.3, None, torch.float32)
    wide = plain.causal_attention(q, k, v, 0.3, 12, torch.float32)
    assert torch.allclose(full, wide)
    narrow = plain.causal_attention(q, k, v, 0.3, 3, torch.float32)
    assert torch.allclose(narrow[:3], full[:3])              # the first three positions see everything
    # position 7 with window 3 sees keys 5, 6, 7 only
    alone = plain.causal_attention(q[7:8], k[5:8], v[5:8], 0.3, None, torch.float32,
                                   q_positions=torch.tensor([2]))
    assert torch.allclose(narrow[7], alone[0], atol=1e-6)
    one = plain.causal_attention(q, k, v, 0.3, 1, torch.float32)
    assert torch.allclose(one, v.expand(12, 2, 8), atol=1e-6)   # window 1: the token's own value


def test_rotation_keeps_norms_and_depends_on_distance_only():
    cos, sin = plain.rope_tables(16, 64, 10_000.0)
    torch.manual_seed(1)
    x = torch.randn(1, 1, 16).expand(40, 1, 16)
    y = torch.randn(1, 1, 16).expand(40, 1, 16)
    rx = plain.rotate_half_split(x, cos[:40], sin[:40], torch.float32)
    ry = plain.rotate_half_split(y, cos[:40], sin[:40], torch.float32)
    assert torch.allclose(rx.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    dots = [(rx[p + 3, 0] * ry[p, 0]).sum().item() for p in range(30)]
    assert max(dots) - min(dots) < 1e-4
    assert cos[0].eq(1).all() and sin[0].eq(0).all()
    assert math.isclose(cos[1, 1].item(), math.cos(10_000.0 ** (-2 / 16)), rel_tol=1e-6)


def test_norm_and_activation_formulas():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    y = plain.rms_norm(x, w, 0.0, torch.float32)
    rms = math.sqrt((9 + 16) / 2)
    assert torch.allclose(y, torch.tensor([[3 / rms * 2, 4 / rms * 0.5]]))
    y2, m = plain.add_rms_norm(x, torch.tensor([[1.0, -1.0]]), w, 0.0, torch.float32)
    assert torch.equal(m, torch.tensor([[4.0, 3.0]]))
    g = torch.tensor([[0.0, 2.0, 5.0, -1.0]])
    out = plain.swiglu(g, torch.float32)
    assert torch.allclose(out, torch.tensor([[0.0, 2 / (1 + math.exp(-2)) * -1.0]]))


def test_bfloat16_rounding_points_change_little_but_something(model_folders):
    cfg, weights = plain.read_config(model_folders["b"]), plain.read_weights(model_folders["b"])
    tokens = random_tokens(cfg["V"], 40, 5)
    exact = plain.forward(cfg, weights, tokens)
    rounded = plain.forward(cfg, weights, tokens, torch.bfloat16)
    error = (exact - rounded).abs().max().item() / exact.abs().max().item()
    assert 1e-4 < error < 5e-2


def test_run_list_with_a_repeated_layer_and_a_borrowed_cache(model_folders):
    cfg, weights = plain.read_config(model_folders["a"]), plain.read_weights(model_folders["a"])
    tokens = random_tokens(cfg["V"], 20, 6)
    plainly = plain.forward(cfg, weights, tokens)
    same = plain.forward(cfg, weights, tokens, order=[(0, None), (1, None)])
    assert torch.equal(plainly, same)
    twice = plain.forward(cfg, weights, tokens, order=[(0, None), (1, None), (0, None)])
    borrowed = plain.forward(cfg, weights, tokens, order=[(0, None), (1, None), (0, 0)])
    assert not torch.allclose(twice, plainly) and not torch.allclose(twice, borrowed)


def test_philox_known_answer_and_noise_range():
    # Random123 known-answer test for philox4x32-10 with counter and key of all ones bits
    out = plain.philox4x32((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2)
    assert out == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert plain.philox4x32((0, 0, 0, 0), (0, 0)) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    noise = plain.exponential_noise(3, 5, 1001)
    assert noise.shape == (1001,) and (noise > 0).all() and torch.isfinite(noise).all()
    assert 0.9 < noise.mean().item() < 1.1
    assert not torch.equal(noise, plain.exponential_noise(3, 6, 1001))


def test_sampling_rules():
    logits = torch.tensor([0.1, 3.0, 2.9, -1.0, 2.95, 0.0])
    assert plain.sample(logits, 0.0, 0, 1.0, 0, 0) == 1
    picks = {plain.sample(logits, 1.0, 2, 1.0, seed, 0) for seed in range(60)}
    assert picks == {1, 4}                                    # top-k 2 keeps the two largest
    probabilities = torch.softmax(logits, 0)
    top_p = (probabilities[1] + probabilities[4]).item() + 1e-3
    picks = {plain.sample(logits, 1.0, 0, top_p, seed, 0) for seed in range(80)}
    assert picks == {1, 4, 2}        # the mass before token 2 does not exceed top_p: it stays; the rest go
    picks = {plain.sample(logits, 1.0, 0, 1e-6, seed, 0) for seed in range(20)}
    assert picks == {1}                                       # the first token always stays
    counts = torch.zeros(6)
    for seed in range(3000):
        counts[plain.sample(logits, 0.7, 0, 1.0, seed, 1)] += 1
    expected = torch.softmax(logits / 0.7, 0)
    assert (counts / 3000 - expected).abs().max().item() < 0.03
