"""Traces for the replay tests, and the comparison with the plain implementation.

A trace is a list of steps ``{"step", "entries": [{"id", "tokens", "want"}], "end"}``
in the format of ``bin/trace_run``.  Every generator below cuts the same
requests differently; ``collect`` turns the logits of a run into
{(request, position): row} so that all cuts compare with one oracle.
"""

from __future__ import annotations

import random

import numpy as np
import torch

import plain_qwen3 as plain

TOLERANCE = {
    # largest |difference| allowed, as a fraction of the largest |logit| of the sequence.  Observed on a
    # B200 over every configuration and way of cutting: float32 up to 1.1e-6 at the tiny sizes and 7.1e-6
    # at the layer widths of the 8B and 32B sizes (sums over 12,288 and 25,600 terms in another order
    # than the oracle's); bfloat16 up to 1.5e-2 (both follow the same rounding points; the engine's
    # products sum in another order and its attention rounds probabilities per tile).
    torch.float32: 1.2e-5,
    torch.bfloat16: 2.5e-2,
}
# mean |difference| of a row, averaged over the rows; observed up to 1.0e-6 and 2.0e-3
MEAN_TOLERANCE = {torch.float32: 2e-6, torch.bfloat16: 3e-3}


def whole(requests: dict) -> list[dict]:
    """Each request alone and whole: one step, logits everywhere."""
    steps = []
    for n, (rid, tokens) in enumerate(requests.items()):
        steps.append({"step": n, "entries": [{"id": rid, "tokens": list(tokens),
                                              "want": list(range(len(tokens)))}], "end": [rid]})
    return steps


def tail_by_one(requests: dict, tail: int = 32) -> list[dict]:
    """Most of a request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(tokens[:head]),
                                                       "want": [head - 1]}], "end": []})
        for p in range(head, len(tokens)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [tokens[p]],
                                                           "want": [0]}],
                          "end": [rid] if p == len(tokens) - 1 else []})
        if head == len(tokens):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests: dict, seed: int, sizes=(2, 3, 5, 8, 13, 31, 64, 100)) -> list[dict]:
    """Portions of changing size, down to two tokens; logits everywhere."""
    rng = random.Random(seed)
    steps = []
    for rid, tokens in requests.items():
        p = 0
        while p < len(tokens):
            n = min(rng.choice(sizes), len(tokens) - p)
            if len(tokens) - p - n == 1:       # never leave a single token behind: portions are >= 2
                n += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(tokens[p:p + n]),
                                                           "want": list(range(n))}],
                          "end": [rid] if p + n == len(tokens) else []})
            p += n
    return steps


def mixed(requests: dict, seed: int, *, live: int = 4, decode_tail: int = 12,
          sizes=(2, 3, 7, 16, 40)) -> list[dict]:
    """Up to ``live`` requests at a time: portions of some beside single tokens of others;
    a request sometimes sits a step out.  The last ``decode_tail`` tokens of a request come
    one by one.  Ends free pages that later requests take again."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    running: dict = {}
    steps = []
    while waiting or running:
        while waiting and len(running) < live:
            rid, tokens = waiting.pop(0)
            running[rid] = [list(tokens), 0]
        entries, ended = [], []
        for rid, state in list(running.items()):
            tokens, p = state
            if len(running) > 1 and rng.random() < 0.2:
                continue                        # sits this step out
            left = len(tokens) - p
            n = 1 if left <= decode_tail else min(rng.choice(sizes), left - decode_tail)
            entries.append({"id": rid, "tokens": tokens[p:p + n], "want": list(range(n))})
            state[1] = p + n
            if state[1] == len(tokens):
                ended.append(rid)
                del running[rid]
        if not entries:
            continue
        rng.shuffle(entries)
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def live_token_need(steps: list[dict], round_to: int = 64) -> int:
    """The --max-tokens a trace needs: the most tokens live requests hold, each
    request's count rounded up to ``round_to``."""
    held: dict = {}
    peak = 0
    for step in steps:
        for entry in step["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    return peak


def run_steps(runner, steps: list[dict]) -> dict:
    """Drive a StepRunner through a trace; {(request, position): float32 row}."""
    from tinyvllm_b200.engine.step import StepEntry

    out: dict = {}
    position: dict = {}
    for step in steps:
        entries = []
        for item in step["entries"]:
            if not runner.manager.is_open(item["id"]):
                runner.open(item["id"])
            entries.append(StepEntry(item["id"], tuple(item["tokens"]), tuple(item["want"])))
        logits = runner.run(entries)
        rows = None if logits is None else logits.float().cpu()
        cursor = 0
        for item in step["entries"]:
            start = position.get(item["id"], 0)
            for place in item["want"]:
                out[(item["id"], start + place)] = rows[cursor]
                cursor += 1
            position[item["id"]] = start + len(item["tokens"])
        for rid in step["end"]:
            runner.close(rid)
            position.pop(rid, None)
        runner.manager.check()
    return out


def read_trace_output(steps: list[dict], out_dir, vocab: int) -> dict:
    """The same mapping from the <step>.f32 files bin/trace_run wrote."""
    out: dict = {}
    position: dict = {}
    for step in steps:
        wanted = sum(len(e["want"]) for e in step["entries"])
        rows = None
        if wanted:
            rows = torch.from_numpy(
                np.fromfile(out_dir / f"{step['step']}.f32", dtype="<f4").reshape(wanted, vocab).copy())
        cursor = 0
        for item in step["entries"]:
            start = position.get(item["id"], 0)
            for place in item["want"]:
                out[(item["id"], start + place)] = rows[cursor]
                cursor += 1
            position[item["id"]] = start + len(item["tokens"])
        for rid in step["end"]:
            position.pop(rid, None)
    return out


_oracle_cache: dict = {}


class SomeRows:
    """The oracle's logits at chosen positions of one sequence: ``self[position]`` is a row."""

    def __init__(self, positions, rows: torch.Tensor) -> None:
        self.rows = {position: rows[i] for i, position in enumerate(positions)}
        self.largest = rows.abs().max().item()

    def __getitem__(self, position):
        return self.rows[position]


def logit_scale(expected) -> float:
    return expected.largest if isinstance(expected, SomeRows) else expected.abs().max().item()


def oracle(folder, requests: dict, dtype: torch.dtype, order=None, positions=None, weights=None) -> dict:
    """{request: logits [T, V]} of the plain implementation (cached per folder and dtype).  With
    ``positions`` = {request: positions} only those rows are made (a wide vocabulary)."""
    cfg = plain.read_config(folder)
    weights = weights if weights is not None else plain.read_weights(folder)
    out = {}
    for rid, tokens in requests.items():
        chosen = None if positions is None else tuple(sorted(positions[rid]))
        key = (str(folder), dtype, tuple(tokens), None if order is None else tuple(order), chosen)
        if key not in _oracle_cache:
            logits = plain.forward(cfg, weights, tokens, dtype, order=order, rows=chosen)
            _oracle_cache[key] = logits if chosen is None else SomeRows(chosen, logits)
        out[rid] = _oracle_cache[key]
    return out


def thin(steps: list[dict], keep_every: int, tail: int = 24) -> list[dict]:
    """The same trace with logits wanted only at every ``keep_every``-th place of a portion and at
    its last ``tail`` places (a wide vocabulary makes every row expensive)."""
    thinned = []
    for step in steps:
        entries = []
        for entry in step["entries"]:
            count = len(entry["tokens"])
            want = [p for p in entry["want"] if p % keep_every == 0 or p >= count - tail]
            entries.append({**entry, "want": want})
        thinned.append({**step, "entries": entries})
    return thinned


def wanted_positions(steps: list[dict]) -> dict:
    """{request: positions at which the trace wants logits}."""
    found: dict = {}
    position: dict = {}
    for step in steps:
        for entry in step["entries"]:
            start = position.get(entry["id"], 0)
            found.setdefault(entry["id"], set()).update(start + p for p in entry["want"])
            position[entry["id"]] = start + len(entry["tokens"])
    return found


def compare(got: dict, expected: dict, dtype: torch.dtype, *, what: str = "") -> float:
    """Every produced row against the oracle; the first wrong position is named."""
    assert got, f"{what}: no logits were produced"
    worst = 0.0
    total, count = 0.0, 0
    for (rid, position), row in sorted(got.items(), key=lambda kv: (str(kv[0][0]), kv[0][1])):
        want = expected[rid][position]
        scale = logit_scale(expected[rid])
        assert torch.isfinite(row).all(), f"{what}: request {rid} position {position}: not finite"
        diff = (row - want).abs()
        err = diff.max().item() / scale
        total += diff.mean().item() / scale
        count += 1
        assert err <= TOLERANCE[dtype], (
            f"{what}: request {rid} position {position}: |diff| {err:.3e} of the logit scale "
            f"(allowed {TOLERANCE[dtype]:.1e})")
        worst = max(worst, err)
    assert total / count <= MEAN_TOLERANCE[dtype], (
        f"{what}: mean |diff| {total / count:.3e} of the logit scale (allowed {MEAN_TOLERANCE[dtype]:.1e})")
    return worst
