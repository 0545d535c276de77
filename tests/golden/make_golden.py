"""Makes tests/golden/reference_logits_*.npz: RicardoMin/tiny-vLLM's own model code on the CPU.

Run by hand where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/tiny-vLLM

It imports the reference's model (tinyvllm/models/qwen3.py), scheduler, block
manager, batch builder and executor with its "reference" attention backend
(tinyvllm/runtime/attention.py:12-151) in float32 on the CPU, loads a tiny
random model folder through the reference's own checkpoint reader
(tinyvllm/checkpoint.py:84-143), generates greedily with chunked prefill, and
records the logits of every sampled position.  tests/test_plain_vs_reference.py
compares the plain implementation with these files.

Two things are not the reference's own code here, because they cannot run on
this CPU as shipped:
* its four pointwise operations are CUDA only (tinyvllm/layers.py:12-16,
  tinyvllm/models/qwen3.py:16); they are replaced by the functions of
  tests/plain_qwen3.py here; those four formulas are checked against the reference's own
  kernels separately (make_pointwise_golden.py, run on a GPU, reference_pointwise.npz);
* its configuration loader goes through a transformers version that is not
  installed; the configuration object is built with ``Qwen3Config.from_hf`` from
  a plain namespace of the same keys (tinyvllm/models/qwen3.py:123-201).
Everything else (weight routing and packing, rotary tables, layer arrangement,
attention with its masks, cache writes and gathers, scheduling, head) is the
reference's code.
"""

from __future__ import annotations

import sys
import tempfile
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

import plain_qwen3 as plain  # noqa: E402
from tiny_configs import GOLDEN_WORKLOADS, TINY_CONFIGS  # noqa: E402
from tinyvllm_b200.models import Qwen3Config  # noqa: E402
from tinyvllm_b200.weights.random_init import write_model_folder  # noqa: E402


def install_cpu_pointwise():
    import tinyvllm.layers as layers
    import tinyvllm.models.qwen3 as qwen3

    f32 = torch.float32

    def rms_norm(x, weight, eps):
        return plain.rms_norm(x.to(f32), weight.to(f32), eps, x.dtype).to(x.dtype)

    def add_rms_norm(x, residual, weight, eps):
        y, m = plain.add_rms_norm(x.to(f32), residual.to(f32), weight.to(f32), eps, x.dtype)
        return y.to(x.dtype), m.to(x.dtype)

    def silu_and_mul(x):
        return plain.swiglu(x.to(f32), x.dtype).to(x.dtype)

    def qk_norm_rope(q, k, qw, kw, cos, sin, q_eps, k_eps):
        c, s = cos[:, 0, :].to(f32), sin[:, 0, :].to(f32)
        qo = plain.rotate_half_split(plain.rms_norm(q.to(f32), qw.to(f32), q_eps, q.dtype), c, s, q.dtype)
        ko = plain.rotate_half_split(plain.rms_norm(k.to(f32), kw.to(f32), k_eps, k.dtype), c, s, k.dtype)
        return qo.to(q.dtype).contiguous(), ko.to(k.dtype).contiguous()

    layers.rms_norm, layers.add_rms_norm, layers.silu_and_mul = rms_norm, add_rms_norm, silu_and_mul
    qwen3.qk_norm_rope = qk_norm_rope


def run_reference(model_dir: Path, config: Qwen3Config, workload: dict):
    from tinyvllm.checkpoint import load_weights
    from tinyvllm.engine import Engine, GenerateRequest
    from tinyvllm.executor import Executor
    from tinyvllm.models.qwen3 import Qwen3Config as RefConfig, Qwen3ForCausalLM
    from tinyvllm.request import SamplingParams
    from tinyvllm.sampling import TorchSampler
    from tinyvllm.scheduler import Scheduler

    namespace = types.SimpleNamespace(
        model_type="qwen3", hidden_act="silu", eos_token_id=None,
        vocab_size=config.vocab_size, hidden_size=config.hidden_size,
        intermediate_size=config.intermediate_size, num_hidden_layers=config.num_hidden_layers,
        max_position_embeddings=config.max_position_embeddings,
        num_attention_heads=config.num_attention_heads,
        num_key_value_heads=config.num_key_value_heads, head_dim=config.head_dim,
        rope_theta=config.rope_theta, rms_norm_eps=config.rms_norm_eps,
        tie_word_embeddings=config.tie_word_embeddings)
    model = Qwen3ForCausalLM(RefConfig.from_hf(namespace), device="cpu", dtype=torch.float32)
    load_weights(model, model_dir)
    model.eval()

    recorded: dict[int, list[np.ndarray]] = {}

    class Recorder(TorchSampler):
        def sample(self, logits, sampling_params, request_ids):
            for row, request_id in zip(logits, request_ids):
                recorded.setdefault(request_id, []).append(row.to(torch.float32).numpy().copy())
            return super().sample(logits, sampling_params, request_ids)

    page, pages = workload["page_size"], workload["pages"]
    executor = Executor(model, block_size=page, num_blocks=pages, max_model_len=config.max_position_embeddings,
                        sampler=Recorder(), max_num_seqs=4, attention_backend="reference",
                        enforce_eager=True)
    scheduler = Scheduler(max_active_requests=4, max_step_requests=4, max_scheduled_tokens=64,
                          prefill_chunk_size=workload["chunk"],
                          max_model_len=config.max_position_embeddings,
                          prefill_reserve_tokens=0, prefill_reserve_requests=0, kv_block_size=page,
                          kv_num_blocks=pages, eos_token_ids=None, enable_prefix_caching=False)
    engine = Engine(scheduler, executor)
    sampling = SamplingParams(max_new_tokens=workload["new_tokens"], temperature=0.0, ignore_eos=True)
    outputs = engine.generate([GenerateRequest(tuple(p), sampling) for p in workload["prompts"]])
    result = {}
    for index, output in enumerate(outputs):
        result[f"tokens_{index}"] = np.asarray(output.output_token_ids, dtype=np.int64)
        result[f"logits_{index}"] = np.stack(recorded[output.request_id])
        result[f"prompt_{index}"] = np.asarray(workload["prompts"][index], dtype=np.int64)
    return result


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py /path/to/tiny-vLLM")
    reference_root = Path(sys.argv[1])
    sys.path.insert(0, str(reference_root))
    install_cpu_pointwise()
    for name, workload in GOLDEN_WORKLOADS.items():
        config = TINY_CONFIGS[name]
        with tempfile.TemporaryDirectory() as folder:
            write_model_folder(folder, config, seed=workload["seed"])
            with torch.inference_mode():
                result = run_reference(Path(folder), config, workload)
        np.savez_compressed(HERE / f"reference_logits_{name}.npz", **result)
        print(name, {k: v.shape for k, v in result.items() if k.startswith("logits")})


if __name__ == "__main__":
    main()
