"""Throughput of the engine on one B200: decode and prefill at Qwen3-0.6B dimensions (the
default, the headline), and the serving workloads of the 8B and 32B dimensions.

``python bench.py --gpus 1 --steps K --warmup W`` prints ONE JSON line.  A step is one decode
step of a batch of 8 requests whose contexts start at 2,048 tokens (context limit 4,096), random
weights, bfloat16.

* ``value``: decoded tokens per second, device-timed with CUDA events over K replays of the
  decode step (the metadata of every step uploaded from pinned memory, no host synchronisation
  between steps).
* ``e2e``: the same through the public token-level API (``Engine.submit`` / ``Engine.step``),
  which every step uploads the step's inputs from pinned host memory and copies the sampled
  tokens back to pinned host memory (the engine plans up to 32 decode steps at once, keeps two
  launched ahead of the one it reads, and a call of ``step`` returns the tokens of one of them).
* ``prefill``: one prompt of 2,048 tokens through the step function.
* ``roofline``: bytes a decode step must read (every weight once + the cache of the live
  requests) / time / measured HBM bandwidth.
* ``points``: decode at batch 1 and 64; decode at batch 8 from a context of 16,384 tokens (with its
  fraction of the HBM roofline), a prefill of 8,192 tokens (with its fraction of the tensor peak) and
  decode of one request alone at a context of 32,768.

Every step reads more than the 126 MB of L2 (the weights alone are 1.19 GB), so the inputs are
larger than L2 and no flush is needed between timed steps.

``--workload 8b`` / ``--workload 32b`` run the request mixes of those sizes at full depth through
``Engine.step`` (64 requests with prompts of 128 to 4,096 tokens and 128 new tokens, half of them
sampled at temperature 0.8, 2,048 prompt tokens a step; 8 requests with prompts of 4,096 to
16,384 tokens and 256 new tokens) and print one JSON line with tokens per second, the time of a
decode step with every request live and its fraction of the HBM roofline.  ``--workload
arrivals`` replays 16 requests that arrive 20 ms apart at the 0.6B sizes (time to first token and
time per output token).

``--impl reference`` runs the unmodified reference installed under ``baseline/_ref`` on the same
decode workload through its own engine, or prints one line saying why it cannot.
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

MODELS = {
    "0.6b": dict(vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
                 num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                 max_position_embeddings=40960, rope_theta=1_000_000.0, rms_norm_eps=1e-6,
                 tie_word_embeddings=True),
    "8b": dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
               num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               max_position_embeddings=40960, rope_theta=1_000_000.0, rms_norm_eps=1e-6,
               tie_word_embeddings=False),
    "32b": dict(vocab_size=151936, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64,
                num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                max_position_embeddings=40960, rope_theta=1_000_000.0, rms_norm_eps=1e-6,
                tie_word_embeddings=False),
}
MODEL = MODELS["0.6b"]
CONTEXT_LIMIT = 4096
PROMPT_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
METRIC = "decode tok/s @ batch 8 (Qwen3-0.6B dims, bf16, context from 2,048)"


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
    """nvidia-smi clocks and throttle reasons while the timed regions run."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.process = None
        self.lines: list[str] = []
        self.spans: list[tuple[int, int]] = []

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

    def span(self, first: int) -> None:
        """The samples from ``first`` to now were taken under a timed region."""
        self.spans.append((first, len(self.lines)))

    def stop(self) -> None:
        if self.process is not None:
            self.process.terminate()

    def summary(self) -> dict:
        sm, sm_max, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        chosen = [line for first, last in self.spans for line in self.lines[first:last]]
        for line in chosen or self.lines[-3:]:
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


def random_prompt(rng: random.Random, count: int, vocab: int = MODEL["vocab_size"]) -> list[int]:
    return [rng.randrange(vocab) for _ in range(count)]


# --------------------------------------------------------------------------- the reference arm
def reference_arm(args) -> int:
    """The unmodified reference from ``baseline/_ref`` on the decode workload: the same model sizes
    with random weights, ``--batch`` prompts of 2,048 tokens prefilled untimed, then K decode steps
    through its own ``Engine.step`` (its scheduler, executor, CUDA kernels and decode graphs).
    Nothing of this repository's package is imported here.  If the reference cannot run on this
    machine, one line says why, in its own words."""
    import types

    line = {"impl": "reference", "metric": METRIC, "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: uniform random token ids, random weights N(0, 0.02)"}
    warmup, steps, batch = max(args.warmup, 3), args.steps, args.batch
    stage = "import"
    try:
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        import torch
        from tinyvllm.engine import Engine
        from tinyvllm.executor import Executor
        from tinyvllm.models.qwen3 import Qwen3Config, Qwen3ForCausalLM
        from tinyvllm.request import SamplingParams
        from tinyvllm.scheduler import Scheduler

        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is visible")
        stage = "model"
        layers = args.layers
        config = Qwen3Config.from_hf(types.SimpleNamespace(
            model_type="qwen3", hidden_act="silu", eos_token_id=None,
            **{**MODEL, "num_hidden_layers": layers}))
        with torch.inference_mode():
            model = Qwen3ForCausalLM(config, device="cuda", dtype=torch.bfloat16)
            generator = torch.Generator(device="cuda").manual_seed(0)
            for _, parameter in model.named_parameters():
                if parameter.dim() >= 2:
                    parameter.normal_(0.0, 0.02, generator=generator)
                else:
                    parameter.fill_(1.0)
            model.eval()
        stage = "engine (its CUDA kernels are built here)"
        new_tokens = steps + warmup + 64
        block = 16
        blocks = batch * (-(-(PROMPT_TOKENS + new_tokens + 64) // block)) + 256
        budget = max(4096, batch)
        executor = Executor(model, block_size=block, num_blocks=blocks, max_model_len=CONTEXT_LIMIT,
                            max_num_seqs=batch, attention_backend="cuda", enforce_eager=False)
        scheduler = Scheduler(max_active_requests=batch, max_step_requests=batch, max_scheduled_tokens=budget,
                              prefill_chunk_size=2048, max_model_len=CONTEXT_LIMIT, prefill_reserve_tokens=0,
                              prefill_reserve_requests=0, kv_block_size=block, kv_num_blocks=blocks,
                              eos_token_ids=None, enable_prefix_caching=False)
        engine = Engine(scheduler, executor)
        stage = "prefill"
        rng = random.Random(batch)
        sampling = SamplingParams(max_new_tokens=new_tokens, temperature=0.0, ignore_eos=True)
        ids = [engine.submit(random_prompt(rng, PROMPT_TOKENS), sampling) for _ in range(batch)]
        started = set()
        while len(started) < batch:                      # untimed: until every request has its first token
            for event in engine.step().token_events:
                started.add(event.request_id)
        stage = "decode"
        sampler = ClockSampler()
        sampler.start()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        mark = sampler.mark()
        wall = time.perf_counter()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        tokens = 0
        for _ in range(steps):
            tokens += len(engine.step().token_events)
        end.record()
        torch.cuda.synchronize()
        elapsed_ms = max(start.elapsed_time(end), (time.perf_counter() - wall) * 1e3)
        sampler.span(mark)
        sampler.stop()
        if tokens != batch * steps:
            raise RuntimeError(f"{tokens} tokens came back from {steps} steps of {batch} requests")
        value = tokens / (elapsed_ms / 1e3)
        line.update({
            "value": round(value, 1), "ms_per_step": round(elapsed_ms / steps, 4),
            "config": {"model": "Qwen3-0.6B dims", "layers": layers, "layers_of_config": MODEL["num_hidden_layers"],
                       "global_batch": batch, "seq_len": CONTEXT_LIMIT, "prompt_tokens": PROMPT_TOKENS,
                       "kv_block_size": block, "attention_backend": "cuda", "cuda_graphs": True,
                       "parallelism": "single GPU", "timed": "Engine.step of the reference, host tokens in and out"},
            # the reference has no device-only loop: its one number is end to end
            "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": None,
                    "d2h_bytes_per_step": batch * 8},
            "clocks": sampler.summary(),
        })
        for request_id in ids:
            engine.cancel(request_id)
    except ModuleNotFoundError as exc:
        line = {"impl": "reference",
                "unavailable": f"the reference is not installed under baseline/_ref ({exc})"}
    except Exception as exc:  # noqa: BLE001  (whatever the reference raises is the reason)
        reason = " ".join(f"{type(exc).__name__}: {exc}".split())
        line = {"impl": "reference",
                "unavailable": f"the reference's own code refused at stage '{stage}': {reason[:400]}"}
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------- this engine
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
                new_tokens: int = 512, prompt_tokens: int = PROMPT_TOKENS):
    from tinyvllm_b200 import EngineConfig
    from tinyvllm_b200.engine.engine import Engine
    from tinyvllm_b200.models import Qwen3Config

    config = Qwen3Config(**{**MODEL, "num_hidden_layers": layers})
    Path(folder, "config.json").write_text(json.dumps(config.to_json()))
    kv_bytes_per_token = 2 * layers * MODEL["num_key_value_heads"] * MODEL["head_dim"] * 2
    context = max(CONTEXT_LIMIT, prompt_tokens + new_tokens + 16)     # more steps than the workload's 256 fit too
    kv_budget = kv_bytes_per_token * (max_num_seqs * (prompt_tokens + new_tokens + 64) + 8192 + 4096)
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


LONG_CONTEXT = 16384           # context of the long-context decode point
LONG_PREFILL = 8192            # tokens of the long prefill point
LONE_CONTEXT = 32768           # context of the point with one request alone


def prefill_flops(layers: int, tokens: int) -> float:
    h, i, v = MODEL["hidden_size"], MODEL["intermediate_size"], MODEL["vocab_size"]
    nq, nkv, d = MODEL["num_attention_heads"], MODEL["num_key_value_heads"], MODEL["head_dim"]
    linear = layers * (h * (nq + 2 * nkv) * d + nq * d * h + h * 2 * i + i * h)
    attention = layers * 2 * nq * d * (tokens * (tokens + 1) / 2)     # QK^T and PV over the causal half
    return 2.0 * tokens * linear + 2.0 * attention + 2.0 * h * v


def run_decode(engine, batch: int, steps: int, warmup: int, sampler: ClockSampler | None,
               prompt_tokens: int = PROMPT_TOKENS):
    """Device-timed and end-to-end decode of ``batch`` requests; a dict of the figures."""
    import torch

    from tinyvllm_b200 import SamplingParams
    from tinyvllm_b200.engine.step import StepEntry
    from tinyvllm_b200.ops import kernels

    rng = random.Random(batch)
    sampling = SamplingParams(max_new_tokens=new_tokens_of(steps, warmup), ignore_eos=True)

    def fresh_batch():
        """``batch`` requests with their prompts in the cache, about to decode their second token."""
        clear_engine(engine)
        for _ in range(batch):
            engine.submit(random_prompt(rng, prompt_tokens), sampling)
        while engine.scheduler.prefilling or engine.scheduler.waiting:      # untimed prefill
            engine.step()
        assert len(engine.scheduler.decoding) == batch

    fresh_batch()

    # ---- end to end through the public API: submit/step with host tokens in and out
    for _ in range(warmup):
        engine.step()
    graph_steps_before = engine.graph_steps
    torch.cuda.synchronize()
    mark = sampler.mark() if sampler else 0
    start_wall = time.perf_counter()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    e2e_steps = 0
    while e2e_steps < steps:            # a call of step() returns the tokens of the decode steps it read
        before = engine.graph_steps
        events = engine.step()
        ran = engine.graph_steps - before
        assert ran >= 1 and len(events.tokens) == batch * ran, "decode steps did not replay graphs"
        e2e_steps += ran
    end.record()
    torch.cuda.synchronize()
    e2e_ms = max(start.elapsed_time(end), (time.perf_counter() - start_wall) * 1e3)
    if sampler:
        sampler.span(mark)
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
    if sampler:
        sampler.span(mark)
    device_ms = start.elapsed_time(end)
    assert kernels.launch_count() == launches_before      # everything ran from the graph
    kernels.check_finished_launches()
    clear_engine(engine)
    return {
        "tokens_per_s": batch * steps / (device_ms / 1e3), "ms_per_step": device_ms / steps,
        "e2e_tokens_per_s": batch * e2e_steps / (e2e_ms / 1e3), "h2d": h2d_bytes, "d2h": d2h_bytes,
        "launches_per_step": engine.graphs.launches_per_step(batch),
        "mean_context": statistics.mean(contexts),
    }


def run_prefill(engine, repeats: int = 5, tokens: int = PROMPT_TOKENS):
    import torch

    from tinyvllm_b200.engine.step import StepEntry

    rng = random.Random(99)
    runner = engine.runner
    times = []
    with torch.inference_mode():
        for index in range(repeats + 2):
            rid = f"prefill{tokens}-{index}"
            runner.open(rid)
            entry = StepEntry(rid, tuple(random_prompt(rng, tokens)), (tokens - 1,))
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
        engine.close()
    return 0


def headline(args, warmup: int) -> int:
    import gc

    import torch

    peak, peak_source = peaks()
    sampler = ClockSampler()
    sampler.start()
    with tempfile.TemporaryDirectory() as folder:
        engine = make_engine(folder, args.layers, max(args.batch, 1), new_tokens=new_tokens_of(args.steps, warmup))
        main_run = run_decode(engine, args.batch, args.steps, warmup, sampler)
        clocks = sampler.summary()
        prefill_ms = run_prefill(engine)
        weight_bytes = engine.runner.model.weight_bytes()
        bytes_step = decode_bytes(engine, args.batch, main_run["mean_context"])
        points = {}
        engine.close()
        del engine
        gc.collect()
        torch.cuda.empty_cache()
        if not args.no_points:
            for batch in (1, 64):
                with tempfile.TemporaryDirectory() as other:
                    point_engine = make_engine(other, args.layers, batch, new_tokens=new_tokens_of(args.steps, warmup))
                    result = run_decode(point_engine, batch, args.steps, warmup, None)
                    points[f"decode_b{batch}"] = round(result["tokens_per_s"], 1)
                    points[f"decode_b{batch}_e2e"] = round(result["e2e_tokens_per_s"], 1)
                    point_engine.close()
                    del point_engine
                    gc.collect()
                    torch.cuda.empty_cache()
            # further context lengths: decode at batch 8 from a context of 16,384 and a prefill of 8,192
            with tempfile.TemporaryDirectory() as other:
                long_steps = min(args.steps, 32)
                long_engine = make_engine(other, args.layers, 8, new_tokens=new_tokens_of(long_steps, warmup),
                                          prompt_tokens=LONG_CONTEXT)
                result = run_decode(long_engine, 8, long_steps, warmup, None, prompt_tokens=LONG_CONTEXT)
                long_bytes = decode_bytes(long_engine, 8, result["mean_context"])
                points["decode_b8_ctx16k"] = round(result["tokens_per_s"], 1)
                points["decode_b8_ctx16k_hbm_frac"] = round(
                    long_bytes / (result["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"], 4)
                long_ms = run_prefill(long_engine, repeats=3, tokens=LONG_PREFILL)
                points["prefill_8192"] = round(LONG_PREFILL / (long_ms / 1e3), 1)
                points["prefill_8192_frac"] = round(
                    prefill_flops(args.layers, LONG_PREFILL) / (long_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)
                long_engine.close()
                del long_engine
                gc.collect()
                torch.cuda.empty_cache()
            # one request alone with a context of 32,768 (the decode attention cuts it over several
            # clusters a kv head, so that more than 64 of the SMs read its keys)
            with tempfile.TemporaryDirectory() as other:
                lone_steps = min(args.steps, 32)
                lone_engine = make_engine(other, args.layers, 1, new_tokens=new_tokens_of(lone_steps, warmup),
                                          prompt_tokens=LONE_CONTEXT)
                result = run_decode(lone_engine, 1, lone_steps, warmup, None, prompt_tokens=LONE_CONTEXT)
                lone_bytes = decode_bytes(lone_engine, 1, result["mean_context"])
                points["decode_b1_ctx32k"] = round(result["tokens_per_s"], 1)
                points["decode_b1_ctx32k_hbm_frac"] = round(
                    lone_bytes / (result["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"], 4)
                lone_engine.close()
                del lone_engine
                gc.collect()
                torch.cuda.empty_cache()
    sampler.stop()

    achieved_gbs = bytes_step / (main_run["ms_per_step"] / 1e3) / 1e9
    flops = prefill_flops(args.layers, PROMPT_TOKENS)
    line = {
        "metric": METRIC,
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
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------- serving workloads of the other sizes
SERVING = {
    # requests, shortest and longest prompt, new tokens, context limit, half of the requests sampled
    "8b": dict(requests=64, shortest=128, longest=4096, new_tokens=128, max_model_len=8192, sampled=True),
    "32b": dict(requests=8, shortest=4096, longest=16384, new_tokens=256, max_model_len=32768, sampled=False),
}


def serving_workload(args) -> int:
    """The request mix of the 8B or 32B sizes through ``Engine.step``: chunked prefill under 2,048
    prompt tokens a step beside the decodes, every request to its last token; one JSON line."""
    import torch

    from tinyvllm_b200 import EngineConfig, SamplingParams
    from tinyvllm_b200.engine.engine import Engine
    from tinyvllm_b200.engine.step import StepRunner
    from tinyvllm_b200.models import Qwen3Config
    from tinyvllm_b200.ops import kernels

    which = args.workload
    work = SERVING[which]
    dims = dict(MODELS[which])
    layers_of_config = dims["num_hidden_layers"]
    if args.layers_given:
        dims["num_hidden_layers"] = args.layers
    layers = dims["num_hidden_layers"]
    peak, peak_source = peaks()
    requests, new = work["requests"], work["new_tokens"]
    with tempfile.TemporaryDirectory() as folder:
        Path(folder, "config.json").write_text(json.dumps(Qwen3Config(**dims).to_json()))
        kv_per_token = 2 * layers * dims["num_key_value_heads"] * dims["head_dim"] * 2
        sizes = tuple(s for s in (1, 2, 4, 8, 16, 32, 64) if s <= requests)
        config = EngineConfig(
            model=folder, dtype="bfloat16", weights="random", seed=0, max_model_len=work["max_model_len"],
            max_num_seqs=requests, max_num_batched_tokens=2048 + 64, prefill_chunk_size=2048,
            prefill_reserve_tokens=0, prefill_reserve_requests=0, kv_block_size=16,
            kv_cache_memory_bytes=kv_per_token * requests * (work["longest"] + new + 64),
            gpu_memory_utilization=0.95, graph_batch_sizes=sizes)
        began = time.perf_counter()
        engine = Engine.from_config(config)
        start_up_s = time.perf_counter() - began
        weight_bytes = engine.runner.model.weight_bytes()
        rng = random.Random(3)
        prompt_tokens = 0
        for index in range(requests):
            count = rng.randrange(work["shortest"], work["longest"] + 1)
            prompt_tokens += count
            if work["sampled"] and index % 2:
                sampling = SamplingParams(max_new_tokens=new, temperature=0.8, seed=index, ignore_eos=True)
            else:
                sampling = SamplingParams(max_new_tokens=new, ignore_eos=True)
            engine.submit(random_prompt(rng, count, dims["vocab_size"]), sampling)
        sampler = ClockSampler()
        sampler.start()
        torch.cuda.synchronize()
        mark = sampler.mark()
        began = time.perf_counter()
        done, first_token_s = {}, None
        full_ms, full_steps, full_context = 0.0, 0, []
        scheduler = engine.scheduler
        while engine.has_unfinished():
            all_decode = not scheduler.waiting and not scheduler.prefilling and len(scheduler.decoding) == requests
            if all_decode:
                # a decode step with every request live, timed by itself (the wait costs the run a
                # little of its overlap between host and device)
                torch.cuda.synchronize()
                context = sum(scheduler.requests[r].computed_tokens + 1 for r in scheduler.decoding)
                before, at = engine.steps_run, time.perf_counter()
            events = engine.step()
            if all_decode:
                torch.cuda.synchronize()
                ran = engine.steps_run - before
                if ran == 1:
                    full_ms += (time.perf_counter() - at) * 1e3
                    full_steps += 1
                    full_context.append(context)
            if first_token_s is None and events.tokens:
                first_token_s = time.perf_counter() - began
            for output in events.finished:
                done[output.request_id] = output
        torch.cuda.synchronize()
        seconds = time.perf_counter() - began
        sampler.span(mark)
        sampler.stop()
        kernels.check_finished_launches()
        assert len(done) == requests and all(len(o.output_token_ids) == new for o in done.values())
        engine.runner.manager.check()
        assert all(pool.free_count == pool.num_pages for pool in engine.runner.manager.pools)
        decode_ms = full_ms / full_steps if full_steps else None
        hbm = None
        if decode_ms:
            per_token = StepRunner.bytes_per_token(engine.runner.model, engine.runner.dtype)
            bytes_step = weight_bytes + statistics.mean(full_context) * per_token
            achieved = bytes_step / (decode_ms / 1e3) / 1e9
            hbm = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                   "frac": round(achieved / peak["hbm_gbs"], 4), "bytes_per_step": int(bytes_step)}
        line = {
            "metric": f"serving workload, Qwen3-{which.upper()} dims, bf16: new tokens/s over the whole run",
            "value": round(requests * new / seconds, 1), "unit": "tokens/s", "n_gpus": 1,
            "higher_is_better": True, "dtype": "bf16", "impl": "ours",
            "data": "synthetic: uniform random token ids, random weights N(0, 0.02)",
            "seconds": round(seconds, 3), "prompt_tokens_per_s": round(prompt_tokens / seconds, 1),
            "first_token_s": round(first_token_s or 0.0, 3),
            "decode_ms_per_step": round(decode_ms, 3) if decode_ms else None,
            "decode_tokens_per_s": round(requests / decode_ms * 1e3, 1) if decode_ms else None,
            "roofline": hbm,
            "config": {"model": f"Qwen3-{which.upper()} dims", "layers": layers, "layers_of_config": layers_of_config,
                       "requests": requests, "prompt_tokens": prompt_tokens, "new_tokens": new,
                       "shortest_prompt": work["shortest"], "longest_prompt": work["longest"],
                       "seq_len": work["max_model_len"], "prefill_tokens_per_step": 2048,
                       "half_sampled_at_0.8": work["sampled"], "kv_block_size": 16, "peaks": peak_source,
                       "weight_gb": round(weight_bytes / 1e9, 2), "start_up_s": round(start_up_s, 1)},
            "steps": engine.steps_run, "graph_steps": engine.graph_steps,
            "device_gb_peak": round(torch.cuda.max_memory_allocated() / 1e9, 1),
            "clocks": sampler.summary(),
        }
        engine.close()
    print(json.dumps(line))
    return 0


def arrivals_workload(args) -> int:
    """16 requests with prompts of 64 or 512 tokens and 64 new tokens that arrive 20 ms apart, at the
    0.6B sizes, through ``Engine.submit(arrival_ns=)`` and ``Engine.step``: time to first token, time
    per output token and output tokens per second."""
    import torch

    from tinyvllm_b200 import SamplingParams

    requests, new, gap_ns = 16, 64, 20_000_000
    rng = random.Random(16)
    with tempfile.TemporaryDirectory() as folder:
        engine = make_engine(folder, args.layers, requests, new_tokens=new)
        prompts = [random_prompt(rng, 64 if index % 2 == 0 else 512) for index in range(requests)]
        sampling = SamplingParams(max_new_tokens=new, ignore_eos=True)
        results = []
        for _ in range(3):                             # the first pass settles graphs and allocations
            torch.cuda.synchronize()
            origin = time.monotonic_ns()
            ids = [engine.submit(prompt, sampling, arrival_ns=origin + index * gap_ns)
                   for index, prompt in enumerate(prompts)]
            done = {}
            while engine.has_unfinished():
                events = engine.step()
                for output in events.finished:
                    done[output.request_id] = output
                if not events.tokens and not events.finished:
                    ahead = engine.scheduler.next_arrival_ns
                    if ahead is not None:
                        time.sleep(max(0.0, (ahead - time.monotonic_ns()) / 1e9))
            torch.cuda.synchronize()
            finish = max(done[i].finished_ns for i in ids)
            ttft = [(done[i].first_token_ns - done[i].arrival_ns) / 1e6 for i in ids]
            tpot = [(done[i].finished_ns - done[i].first_token_ns) / 1e6 / (new - 1) for i in ids]
            results.append({"ttft_ms": statistics.mean(ttft), "tpot_ms": statistics.mean(tpot),
                            "tokens_per_s": requests * new / ((finish - origin) / 1e9)})
        engine.close()
    best = results[-1]
    print(json.dumps({
        "metric": "arrivals: 16 requests, 64/512 -> 64 tokens, 20 ms apart (Qwen3-0.6B dims, bf16)",
        "value": round(best["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True,
        "dtype": "bf16", "impl": "ours", "ttft_ms": round(best["ttft_ms"], 3), "tpot_ms": round(best["tpot_ms"], 3),
        "passes": [{k: round(v, 3) for k, v in r.items()} for r in results],
        "data": "synthetic: uniform random token ids, random weights N(0, 0.02)",
        "config": {"model": "Qwen3-0.6B dims", "layers": args.layers, "requests": requests, "new_tokens": new,
                   "arrival_gap_ms": 20, "note": "the arrival schedule bounds tokens/s from above"}}))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--workload", choices=("0.6b", "8b", "32b", "arrivals"), default="0.6b",
                        help="0.6b: the decode and prefill measurement (default); 8b, 32b: the serving "
                             "workloads of those sizes at full depth; arrivals: 16 requests 20 ms apart")
    parser.add_argument("--layers", type=int, default=None,
                        help="fewer layers than the configuration has (both numbers are in the line)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    parser.add_argument("--eager-profile", action="store_true",
                        help="no graphs: run warm-up + steps decode steps and one prefill kernel by "
                             "kernel, for a profiler; prints no bench line")
    args = parser.parse_args()
    args.layers_given = args.layers is not None
    if args.layers is None:
        args.layers = MODEL["num_hidden_layers"]
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not built (this engine is single-GPU)")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    sys.path.insert(0, str(ROOT))
    warmup = max(args.warmup, 3)
    if args.workload in SERVING:
        return serving_workload(args)
    if args.workload == "arrivals":
        return arrivals_workload(args)
    if args.eager_profile:
        return eager_profile(args, warmup)
    return headline(args, warmup)


if __name__ == "__main__":
    sys.exit(main())
