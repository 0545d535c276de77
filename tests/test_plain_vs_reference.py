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
