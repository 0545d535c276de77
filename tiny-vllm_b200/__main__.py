"""Command line: ``python -m tinyvllm_b200 --model DIR --prompt-ids 1,2,3``.

Option names, meanings and defaults are those of ``python -m tinyvllm``
(tinyvllm/__main__.py:58-163) where the engine has the feature: --model,
--prompt (repeatable), --dtype, --max-new-tokens, --temperature, --top-k,
--top-p, --seed, --ignore-eos, --enforce-eager, --max-model-len, --max-num-seqs,
--max-num-batched-tokens, --prefill-chunk-size, --kv-cache-mib, --stream (here:
one JSON line per token id as it comes; the reference streams the text of one
prompt); prefill reservations are zero as there (:137-138).  Added: --prompt-ids
(token ids, the engine's native input), --random-weights SEED, --kv-block-size,
float32 as a dtype.  Not offered: chat, attention backends, prefix caching.
Prints one JSON object ``{"outputs": [...]}`` (:155-163).
"""

from __future__ import annotations

import argparse
import json
import sys
from dataclasses import asdict
from pathlib import Path

from .config.engine import EngineConfig
from .engine.llm import LLM
from .sampling.params import SamplingParams


def _ids(text: str) -> list[int]:
    try:
        return [int(part) for part in text.replace(",", " ").split()]
    except ValueError:
        raise argparse.ArgumentTypeError(f"not a list of token ids: {text!r}") from None


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(prog="python -m tinyvllm_b200",
                                     description="Generate tokens with a local model folder")
    parser.add_argument("--model", type=Path, required=True)
    inputs = parser.add_mutually_exclusive_group(required=True)
    inputs.add_argument("--prompt", action="append", help="raw prompt text; repeat for a batch "
                        "(needs tokenizer.json in the model folder)")
    inputs.add_argument("--prompt-ids", action="append", type=_ids,
                        help="prompt as token ids, e.g. 1,2,3; repeat for a batch")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    parser.add_argument("--max-new-tokens", type=int, default=64)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--top-k", type=int, default=0)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--ignore-eos", action="store_true")
    parser.add_argument("--enforce-eager", action="store_true",
                        help="Disable CUDA Graph capture to save memory and startup time")
    parser.add_argument("--max-model-len", type=int, default=2048)
    parser.add_argument("--max-num-seqs", type=int, default=4)
    parser.add_argument("--max-num-batched-tokens", type=int, default=1024,
                        help="Total prefill and decode query-token limit per engine step")
    parser.add_argument("--prefill-chunk-size", type=int, default=512,
                        help="Per-request prefill query-token limit per engine step")
    parser.add_argument("--kv-cache-mib", type=int, default=512)
    parser.add_argument("--kv-block-size", type=int, default=16)
    parser.add_argument("--stream", action="store_true",
                        help="print every token id as it is generated, one JSON object a line, before the outputs")
    parser.add_argument("--random-weights", type=int, metavar="SEED", default=None,
                        help="ignore model.safetensors and draw the weights from this seed")
    args = parser.parse_args(argv)

    sampling = SamplingParams(
        max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_k=args.top_k,
        top_p=args.top_p, seed=args.seed, ignore_eos=args.ignore_eos)
    config = EngineConfig(
        model=args.model, dtype=args.dtype, enforce_eager=args.enforce_eager,
        max_model_len=args.max_model_len, max_num_seqs=args.max_num_seqs,
        max_num_batched_tokens=args.max_num_batched_tokens,
        prefill_chunk_size=min(args.prefill_chunk_size, args.max_num_batched_tokens),
        prefill_reserve_tokens=0, prefill_reserve_requests=0,
        kv_cache_memory_bytes=args.kv_cache_mib * 1024**2, kv_block_size=args.kv_block_size,
        weights="random" if args.random_weights is not None else "checkpoint",
        seed=args.random_weights or 0)
    prompts = args.prompt if args.prompt is not None else args.prompt_ids
    with LLM(config) as llm:
        if args.stream:
            # one line per token as it comes, then the outputs as without the flag
            outputs = [None] * len(prompts)
            for index, item in llm.stream(prompts, sampling):
                if isinstance(item, int):
                    print(json.dumps({"prompt": index, "token_id": item}), flush=True)
                else:
                    outputs[index] = item
        else:
            outputs = llm.generate(prompts, sampling)
    records = [{**asdict(output), "completion_token_count": output.completion_token_count,
                "total_token_count": output.total_token_count} for output in outputs]
    print(json.dumps({"outputs": records}, ensure_ascii=False))


if __name__ == "__main__":
    main(sys.argv[1:])
