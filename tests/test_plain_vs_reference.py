"""The plain implementation against logits recorded from the reference's own code.

tests/golden/make_golden.py produced the files (its header says what of the
reference ran and what was stood in for).  Not a GPU test."""

from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from tiny_configs import GOLDEN_WORKLOADS

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", sorted(GOLDEN_WORKLOADS))
def test_plain_matches_reference_logits(name, model_folders):
    data = np.load(GOLDEN / f"reference_logits_{name}.npz")
    cfg = plain.read_config(model_folders[name])
    weights = plain.read_weights(model_folders[name])
    workload = GOLDEN_WORKLOADS[name]
    for index, prompt in enumerate(workload["prompts"]):
        assert data[f"prompt_{index}"].tolist() == prompt
        generated = data[f"tokens_{index}"].tolist()
        golden = torch.from_numpy(data[f"logits_{index}"])
        sequence = prompt + generated[:-1]
        logits = plain.forward(cfg, weights, sequence)
        ours = logits[len(prompt) - 1:]
        assert ours.shape == golden.shape
        scale = golden.abs().max().item()
        assert (ours - golden).abs().max().item() <= 2e-5 * scale
        assert ours.argmax(-1).tolist() == generated
        assert plain.greedy_generate(cfg, weights, prompt, 3) == generated[:3]


# --------------------------------------------------------------------------------------------
# The four pointwise formulas against the reference's own CUDA kernels
# (tests/golden/make_pointwise_golden.py ran tinyvllm/kernels/pointwise.cu on a B200 and saved
# inputs and outputs).  float32: equal to rounding of the last place; bfloat16: bit for bit.
# --------------------------------------------------------------------------------------------
POINTWISE = np.load(GOLDEN / "reference_pointwise.npz")
DTYPE_OF = {"f32": torch.float32, "bf16": torch.bfloat16}


def saved(name: str) -> torch.Tensor:
    return torch.from_numpy(POINTWISE[name]).to(torch.float32)


def same(ours: torch.Tensor, golden: torch.Tensor, tag: str, what: str) -> None:
    assert ours.shape == golden.shape, what
    if tag == "bf16":
        # every value the reference rounds is rounded at the same place: the same bfloat16 bits
        wrong = (ours != golden).nonzero()
        assert wrong.numel() == 0, f"{what}: {wrong.shape[0]} values differ, first at {wrong[0].tolist()}"
    else:
        # float32: the kernel's rsqrtf and expf and the order of its sums may differ in the last places
        limit = 4e-6 * golden.abs().clamp_min(1.0)
        assert ((ours - golden).abs() <= limit).all(), f"{what}: {(ours - golden).abs().max().item():.3e}"


@pytest.mark.parametrize("tag", ["f32", "bf16"])
@pytest.mark.parametrize("width", [48, 128, 200, 1024])
@pytest.mark.parametrize("eps_tag", ["a", "b"])
def test_plain_norms_match_the_reference_kernels(tag, width, eps_tag):
    dt = DTYPE_OF[tag]
    case = f"norm_{tag}_w{width}_{eps_tag}"
    eps = float(POINTWISE[f"{case}_eps"])
    x, residual, weight = saved(f"{case}_x"), saved(f"{case}_residual"), saved(f"{case}_weight")
    same(plain.rms_norm(x, weight, eps, dt), saved(f"{case}_out"), tag, f"rms_norm {case}")
    normed, summed = plain.add_rms_norm(x, residual, weight, eps, dt)
    same(summed, saved(f"{case}_add_sum"), tag, f"add_rms_norm sum {case}")
    same(normed, saved(f"{case}_add_out"), tag, f"add_rms_norm {case}")


@pytest.mark.parametrize("tag", ["f32", "bf16"])
@pytest.mark.parametrize("inter", [24, 100, 3072])
def test_plain_swiglu_matches_the_reference_kernel(tag, inter):
    case = f"silu_{tag}_i{inter}"
    same(plain.swiglu(saved(f"{case}_x"), DTYPE_OF[tag]), saved(f"{case}_out"), tag, case)


@pytest.mark.parametrize("tag", ["f32", "bf16"])
@pytest.mark.parametrize("head_dim", [16, 48, 128])
def test_plain_qk_norm_rope_matches_the_reference_kernel(tag, head_dim):
    dt = DTYPE_OF[tag]
    case = f"rope_{tag}_d{head_dim}"
    eps = float(POINTWISE[f"{case}_eps"])
    q, k = plain.qk_norm_rope(saved(f"{case}_q"), saved(f"{case}_k"), saved(f"{case}_q_weight"),
                              saved(f"{case}_k_weight"), saved(f"{case}_cos"), saved(f"{case}_sin"), eps, dt)
    same(q, saved(f"{case}_q_out"), tag, f"{case} q")
    same(k, saved(f"{case}_k_out"), tag, f"{case} k")
