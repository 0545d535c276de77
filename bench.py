"""Decode and prefill throughput of the engine at Qwen3-0.6B dimensions on one B200.

``python bench.py --gpus 1 --steps K --warmup W`` prints ONE JSON line.  A step is
one decode step of a batch of 8 requests whose contexts start at 2,048 tokens
(context limit 4,096), random weights, bfloat16.

* ``value``: decoded tokens per second, device-timed with CUDA events over K replays
  of the decode step (metadata of every step uploaded from pinned memory, no host
  synchronisation between steps).
* ``e2e``: the same through the public token-level API (``Engine.submit`` /
  ``Engine.step``), which every step uploads the step's inputs from pinned host
  memory and copies the sampled tokens back to pinned host memory (the engine
  plans up to 32 decode steps at once, keeps two launched ahead of the one it
  reads, and a call of ``step`` returns the tokens of one of them).
* ``prefill``: one prompt of 2,048 tokens through the step function.
* ``roofline``: bytes a decode step must read (every weight once + the cache of the
  live requests) / time / measured HBM bandwidth.
* ``points``: decode at batch 1 and 64.

Every step reads more than the 126 MB of L2 (weights alone are 1.19 GB), so the
inputs are larger than L2 and no flush is needed between timed steps.
"""

from __future__ import annotations

import argparse
import json
import random
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MODEL = dict(vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
             num_attention_heads=16, num_key_value_heads=8, head_dim=128,
             max_position_embeddings=40960, rope_theta=1_000_000.0, rms_norm_eps=1e-6,
             tie_word_embeddings=True)
CONTEXT_LIMIT = 4096
PROMPT_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            flat = {}

            def walk(node):
                if isinstance(node, dict):
                    for key, value in node.items():
                        if isinstance(value, (int, float)) and key in FALLBACK_PEAKS:
                            flat.setdefault(key, float(value))
                        else:
                            walk(value)
                elif isinstance(node, list):
                    for value in node:
                        walk(value)

            walk(data)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return {**FALLBACK_PEAKS, **flat}, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.process = None
        self.lines: list[str] = []

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.process = None

    def _read(self) -> None:
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def mark(self) -> int:
        return len(self.lines)

    def stop(self) -> None:
        if self.process is not None:
            self.process.terminate()

    def summary(self, first: int = 0, last: int | None = None) -> dict:
        sm, sm_max, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines[first:last]:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                sm.append(int(parts[0]))
                sm_max = max(sm_max, int(parts[1]))
            except ValueError:
                continue
            for name, value in zip(names, parts[2:]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": sm_max or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args) -> int:
    """The unmodified reference through its own public API, or one line saying why not."""
    line = {"impl": "reference"}
    try:
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        import tinyvllm  # noqa: F401
        from tinyvllm.models.qwen3 import Qwen3Config as ReferenceConfig

        with tempfile.TemporaryDirectory() as folder:
            (Path(folder) / "config.json").write_text(json.dumps(
                {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", **MODEL,
                 "hidden_act": "silu", "attention_bias": False}))
            ReferenceConfig.from_model_dir(folder)
        line["unavailable"] = ("the reference loads, but its engine needs a tokenizer and a checkpoint "
                               "folder that cannot be had offline")
    except ModuleNotFoundError as exc:
        line["unavailable"] = f"the reference is not installed under baseline/_ref ({exc})"
    except Exception as exc:  # noqa: BLE001  (whatever its own loader raises is the reason)
        line["unavailable"] = ("its own config loader refuses every model folder under the installed "
                               f"transformers (it pins 4.51, not in the wheelhouse): {exc}")
    print(json.dumps(line))
    return 0


def random_prompt(rng: random.Random, count: int) -> list[int]:
    return [rng.randrange(MODEL["vocab_size"]) for _ in range(count)]


def new_tokens_of(steps: int, warmup: int) -> int:
    """Tokens a request of the decode measurement may generate: the warm-up and the timed steps of
    either measurement, and room for the steps a run has launched ahead when it is cut off."""
    return steps + warmup + 64


def clear_engine(engine) -> None:
    """Cancel whatever the engine holds and let a run in flight end, so that every page is back."""
    scheduler = engine.scheduler
    for request_id in list(scheduler.waiting) + list(scheduler.prefilling) + list(scheduler.decoding):
        engine.cancel(request_id)
    while engine.in_run:                # the steps launched ahead are read; the run's pages go back
        engine.step()
    scheduler.take_finished()


def make_engine(folder: str, layers: int, max_num_seqs: int, dtype: str = "bfloat16", eager: bool = False,
                new_tokens: int = 512):
    from tinyvllm_b200 import EngineConfig
    from tinyvllm_b200.engine.engine import Engine
    from tinyvllm_b200.models import Qwen3Config

    config = Qwen3Config(**{**MODEL, "num_hidden_layers": layers})
    Path(folder, "config.json").write_text(json.dumps(config.to_json()))
    kv_bytes_per_token = 2 * layers * MODEL["num_key_value_heads"] * MODEL["head_dim"] * 2
    context = max(CONTEXT_LIMIT, PROMPT_TOKENS + new_tokens + 16)     # more steps than the workload's 256 fit too
    kv_budget = kv_bytes_per_token * (max_num_seqs * (PROMPT_TOKENS + new_tokens + 64) + 4096)
    engine_config = EngineConfig(
        model=folder, dtype=dtype, weights="random", seed=0, max_model_len=context,
        max_num_seqs=max_num_seqs, max_num_batched_tokens=max(4096, max_num_seqs),
        prefill_chunk_size=2048, prefill_reserve_tokens=0, prefill_reserve_requests=0,
        kv_block_size=16, kv_cache_memory_bytes=kv_budget,
        graph_batch_sizes=(max_num_seqs,), enforce_eager=eager)
    return Engine.from_config(engine_config)


def decode_bytes(engine, batch: int, mean_context: float) -> float:
    from tinyvllm_b200.engine.step import StepRunner

    weights = engine.runner.model.weight_bytes()
    per_token = StepRunner.bytes_per_token(engine.runner.model, engine.runner.dtype)
    return weights + batch * mean_context * per_token


def prefill_flops(layers: int, tokens: int) -> float:
    h, i, v = MODEL["hidden_size"], MODEL["intermediate_size"], MODEL["vocab_size"]
    nq, nkv, d = MODEL["num_attention_heads"], MODEL["num_key_value_heads"], MODEL["head_dim"]
    linear = layers * (h * (nq + 2 * nkv) * d + nq * d * h + h * 2 * i + i * h)
    attention = layers * 2 * nq * d * (tokens * (tokens + 1) / 2)     # QK^T and PV over the causal half
    return 2.0 * tokens * linear + 2.0 * attention + 2.0 * h * v


def run_decode(engine, batch: int, steps: int, warmup: int, sampler: ClockSampler | None):
    """(device tokens/s, ms/step, e2e tokens/s, h2d bytes, d2h bytes, launches/step, mean ctx, clocks)."""
    import torch

    from tinyvllm_b200 import SamplingParams
    from tinyvllm_b200.ops import kernels

    rng = random.Random(batch)
    sampling = SamplingParams(max_new_tokens=new_tokens_of(steps, warmup), ignore_eos=True)

    def fresh_batch():
        """``batch`` requests with their prompts in the cache, about to decode their second token."""
        clear_engine(engine)
        for _ in range(batch):
            engine.submit(random_prompt(rng, PROMPT_TOKENS), sampling)
        while engine.scheduler.prefilling or engine.scheduler.waiting:      # untimed prefill
            engine.step()
        assert len(engine.scheduler.decoding) == batch

    fresh_batch()

    # ---- end to end through the public API: submit/step with host tokens in and out
    for _ in range(warmup):
        engine.step()
    graph_steps_before = engine.graph_steps
    torch.cuda.synchronize()
    start_wall = time.perf_counter()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    e2e_steps = 0
    while e2e_steps < steps:            # a call of step() may run several decode steps back to back
        before = engine.graph_steps
        events = engine.step()
        ran = engine.graph_steps - before
        assert ran >= 1 and len(events.tokens) == batch * ran, "decode steps did not replay graphs"
        e2e_steps += ran
    end.record()
    torch.cuda.synchronize()
    e2e_ms = max(start.elapsed_time(end), (time.perf_counter() - start_wall) * 1e3)
    assert engine.graph_steps - graph_steps_before == e2e_steps
    bucket = engine.graphs.bucket_for(batch)
    h2d_bytes = bucket.host.numel() * 4
    d2h_bytes = batch * 4

    # ---- device-timed: K replays, inputs uploaded each step, no host synchronisation; a new batch,
    # so that both measurements walk the same contexts
    fresh_batch()
    scheduler = engine.scheduler
    plans = []
    for _ in range(warmup + steps):
        scheduled = scheduler.schedule()
        plans.append(scheduled)
        # commit with arbitrary tokens: only the bookkeeping advances, nothing is run here
        scheduler.commit(scheduled, {item.request_id: rng.randrange(MODEL["vocab_size"])
                                     for item in scheduled.items})
    from tinyvllm_b200.engine.step import StepEntry

    def replay(scheduled):
        entries = [StepEntry(item.request_id, (rng.randrange(MODEL["vocab_size"]),), (0,))
                   for item in scheduled.items]
        params = [scheduler.requests[item.request_id].sampling for item in scheduled.items]
        engine.graphs.run(scheduled.cache_plan, entries, params, [0] * len(entries))

    contexts = []
    for scheduled in plans[:warmup]:
        replay(scheduled)
    torch.cuda.synchronize()
    launches_before = kernels.launch_count()
    mark = sampler.mark() if sampler else 0
    start.record()
    for scheduled in plans[warmup:]:
        contexts.append(statistics.mean(item.start + 1 for item in scheduled.items))
        replay(scheduled)
    end.record()
    torch.cuda.synchronize()
    clocks = sampler.summary(mark, sampler.mark()) if sampler else None
    device_ms = start.elapsed_time(end)
    assert kernels.launch_count() == launches_before      # everything ran from the graph
    clear_engine(engine)
    return {
        "tokens_per_s": batch * steps / (device_ms / 1e3), "ms_per_step": device_ms / steps,
        "e2e_tokens_per_s": batch * e2e_steps / (e2e_ms / 1e3), "h2d": h2d_bytes, "d2h": d2h_bytes,
        "launches_per_step": engine.graphs.launches_per_step(batch),
        "mean_context": statistics.mean(contexts), "clocks": clocks,
    }


def run_prefill(engine, repeats: int = 5):
    import torch

    from tinyvllm_b200.engine.step import StepEntry

    rng = random.Random(99)
    runner = engine.runner
    times = []
    with torch.inference_mode():
        for index in range(repeats + 2):
            rid = f"prefill{index}"
            runner.open(rid)
            entry = StepEntry(rid, tuple(random_prompt(rng, PROMPT_TOKENS)), (PROMPT_TOKENS - 1,))
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runner.run([entry])
            end.record()
            torch.cuda.synchronize()
            runner.close(rid)
            if index >= 2:
                times.append(start.elapsed_time(end))
    return statistics.median(times)


def eager_profile(args, warmup: int) -> int:
    """Decode steps and one prefill through the eager path, so that a profiler sees every kernel."""
    import torch

    from tinyvllm_b200 import SamplingParams

    rng = random.Random(0)
    with tempfile.TemporaryDirectory() as folder:
        engine = make_engine(folder, args.layers, args.batch, eager=True, new_tokens=new_tokens_of(args.steps, warmup))
        sampling = SamplingParams(max_new_tokens=warmup + args.steps + 4, ignore_eos=True)
        for _ in range(args.batch):
            engine.submit(random_prompt(rng, PROMPT_TOKENS), sampling)
        while engine.scheduler.prefilling or engine.scheduler.waiting:
            engine.step()
        torch.cuda.synchronize()
        for _ in range(warmup + args.steps):
            engine.step()
        torch.cuda.synchronize()
        clear_engine(engine)
        print("eager profile run: ok", run_prefill(engine, repeats=1), "ms prefill")
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--layers", type=int, default=MODEL["num_hidden_layers"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    parser.add_argument("--eager-profile", action="store_true",
                        help="no graphs: run warm-up + steps decode steps and one prefill kernel by "
                             "kernel, for a profiler; prints no bench line")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not built (this engine is single-GPU)")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    warmup = max(args.warmup, 3)

    import torch

    if args.eager_profile:
        return eager_profile(args, warmup)
    peak, peak_source = peaks()
    sampler = ClockSampler()
    sampler.start()
    with tempfile.TemporaryDirectory() as folder:
        engine = make_engine(folder, args.layers, max(args.batch, 1), new_tokens=new_tokens_of(args.steps, warmup))
        main_run = run_decode(engine, args.batch, args.steps, warmup, sampler)
        prefill_ms = run_prefill(engine)
        weight_bytes = engine.runner.model.weight_bytes()
        bytes_step = decode_bytes(engine, args.batch, main_run["mean_context"])
        points = {}
        del engine
        torch.cuda.empty_cache()
        if not args.no_points:
            for batch in (1, 64):
                with tempfile.TemporaryDirectory() as other:
                    point_engine = make_engine(other, args.layers, batch, new_tokens=new_tokens_of(args.steps, warmup))
                    result = run_decode(point_engine, batch, args.steps, warmup, None)
                    points[f"decode_b{batch}"] = round(result["tokens_per_s"], 1)
                    points[f"decode_b{batch}_e2e"] = round(result["e2e_tokens_per_s"], 1)
                    del point_engine
                    torch.cuda.empty_cache()
    sampler.stop()

    achieved_gbs = bytes_step / (main_run["ms_per_step"] / 1e3) / 1e9
    flops = prefill_flops(args.layers, PROMPT_TOKENS)
    line = {
        "metric": "decode tok/s @ batch 8 (Qwen3-0.6B dims, bf16, context from 2,048)",
        "value": round(main_run["tokens_per_s"], 1),
        "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, random weights N(0, 0.02)",
        "impl": "ours",
        "config": {
            "model": "Qwen3-0.6B dims", "layers": args.layers, "layers_of_config": MODEL["num_hidden_layers"],
            "hidden": MODEL["hidden_size"], "q_heads": MODEL["num_attention_heads"],
            "kv_heads": MODEL["num_key_value_heads"], "head_dim": MODEL["head_dim"],
            "intermediate": MODEL["intermediate_size"], "vocab": MODEL["vocab_size"],
            "tied": True, "global_batch": args.batch, "seq_len": CONTEXT_LIMIT,
            "prompt_tokens": PROMPT_TOKENS, "kv_block_size": 16, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (weights 1.19 GB read every step)",
            "cuda_graphs": True, "peaks": peak_source,
        },
        "e2e": {"value": round(main_run["e2e_tokens_per_s"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": main_run["h2d"], "d2h_bytes_per_step": main_run["d2h"]},
        "gpu_launches": main_run["launches_per_step"] * args.steps,
        "prefill": {"value": round(PROMPT_TOKENS / (prefill_ms / 1e3), 1), "tokens": PROMPT_TOKENS,
                    "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": peak["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved_gbs / peak["hbm_gbs"], 4),
                     "bytes_per_step": int(bytes_step), "weight_bytes": int(weight_bytes)},
        "points": points,
        "clocks": main_run["clocks"],
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
