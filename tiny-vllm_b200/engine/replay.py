"""Trace replay: given token ids through the step function, logits to disk.

Reads one JSON object a line,
``{"step": n, "entries": [{"id": ..., "tokens": [...], "want": [...]}], "end": [...]}``,
runs each step through :class:`StepRunner` (the model, cache and kernels that
generation uses), writes ``<out>/<step>.f32`` (little-endian float32,
``[wanted, vocab]``) for steps in which something is wanted, and prints
``done <step>``.  It samples nothing.  The reference ships no such tool (its
charts mention an "offline token-level replay", assets/performance.svg:995).
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

from ..config.registry import read_model_config
from ..ops import kernels
from .model import Model
from .step import StepEntry, StepRunner

PAGE_SIZE = 16
MAX_LIVE_REQUESTS = 16


def build_runner(model_dir, dtype: str, max_tokens: int, *, page_size: int = PAGE_SIZE,
                 device: str = "cuda:0") -> StepRunner:
    """Model of ``model_dir`` with a page pool for ``max_tokens`` tokens in every group."""
    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    if not torch.cuda.is_available():
        raise RuntimeError("trace replay runs the CUDA kernels and needs a GPU; none is visible")
    config = read_model_config(model_dir)
    model = Model(config.to_spec(), device=device, dtype=torch_dtype).load(model_dir)
    pages = -(-max_tokens // page_size)
    return StepRunner(model, page_size=page_size, num_pages=pages, max_requests=MAX_LIVE_REQUESTS)


def replay(runner: StepRunner, lines, out_dir: Path, *, report=print) -> None:
    out_dir.mkdir(parents=True, exist_ok=True)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            if not runner.manager.is_open(item["id"]):
                runner.open(item["id"])
            entries.append(StepEntry(item["id"], tuple(item["tokens"]), tuple(item.get("want", ()))))
        if entries:
            logits = runner.run(entries)
            if logits is not None:
                array = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                kernels.check_finished_launches()
                array.tofile(out_dir / f"{step}.f32")
        for request_id in record.get("end", []):
            if runner.manager.is_open(request_id):
                runner.close(request_id)
        report(f"done {step}")


def main(argv=None) -> int:
    import argparse

    parser = argparse.ArgumentParser(
        prog="trace_run", description="feed token ids through the model step by step, write logits")
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), required=True)
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to 64)")
    parser.add_argument("--page-size", type=int, default=PAGE_SIZE)
    args = parser.parse_args(argv)
    if args.max_tokens <= 0 or args.page_size <= 0:
        parser.error("--max-tokens and --page-size must be positive")
    print(f"[trace_run] loading {args.model} ({args.dtype})", file=sys.stderr, flush=True)
    runner = build_runner(args.model, args.dtype, args.max_tokens, page_size=args.page_size)
    torch.backends.cuda.matmul.allow_tf32 = False
    with torch.inference_mode():
        replay(runner, sys.stdin, Path(args.out),
               report=lambda text: (sys.stdout.write(text + "\n"), sys.stdout.flush()))
    return 0
