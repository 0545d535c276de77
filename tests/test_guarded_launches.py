"""Kernels with bounded waits report through a status word that the host reads after a step.  A
step replayed from a CUDA graph launches them without passing through their Python wrappers, so
the replay tells the wrappers' module; the status functions are replaced here (no GPU)."""

import pytest

from tinyvllm_b200.ops import kernels


@pytest.fixture
def fake_status(monkeypatch):
    state = {"gemm": 0, "attention": 0, "reads": []}

    def gemm_status():
        kernels._gemm_tc_unchecked = False
        state["reads"].append("gemm")
        value, state["gemm"] = state["gemm"], 0
        return value

    def attention_status():
        kernels._attention_tc_unchecked = False
        state["reads"].append("attention")
        value, state["attention"] = state["attention"], 0
        return value

    monkeypatch.setattr(kernels, "gemm_tc_status", gemm_status)
    monkeypatch.setattr(kernels, "attention_prefill_tc_status", attention_status)
    monkeypatch.setattr(kernels, "_gemm_tc_unchecked", False)
    monkeypatch.setattr(kernels, "_attention_tc_unchecked", False)
    return state


def test_nothing_is_read_when_no_guarded_kernel_ran(fake_status):
    kernels.check_finished_launches()
    kernels.note_guarded_launches(False, False)
    kernels.check_finished_launches()
    assert fake_status["reads"] == []


def test_a_replayed_graph_makes_the_next_check_read_the_status_words(fake_status):
    kernels.note_guarded_launches(True, False)
    kernels.check_finished_launches()
    assert fake_status["reads"] == ["gemm"]
    kernels.check_finished_launches()                      # read once per replay
    assert fake_status["reads"] == ["gemm"]
    kernels.note_guarded_launches(True, True)
    fake_status["attention"] = 3                           # a wait inside the replayed kernel gave up
    with pytest.raises(kernels.KernelError, match="attention_prefill_tc.*code 3"):
        kernels.check_finished_launches()
    assert fake_status["reads"] == ["gemm", "gemm", "attention"]


def test_a_wait_that_gave_up_in_the_product_kernel_is_reported(fake_status):
    kernels.note_guarded_launches(True, False)
    fake_status["gemm"] = 2
    with pytest.raises(kernels.KernelError, match="gemm_tc.*code 2"):
        kernels.check_finished_launches()
