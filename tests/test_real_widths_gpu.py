"""The engine against the plain implementation at the layer widths of real models.

The tiny configurations never reach the kernels' real-size choices: the tcgen05 product at
thousands of columns, library products for weights of tens of megabytes, eight query heads of a
key-value head in one CTA of the decode attention, clusters of eight CTAs a request, a vocabulary
of 151,936 in the head.  Here two layers of the Qwen3-0.6B sizes (full vocabulary, tied head), two
of the 8B sizes, one of the 32B sizes (query width 8192 beside a hidden width of 5120, untied
head) and one of the 14B sizes (five query heads on a key-value head) are replayed in every way of cutting, in 32-bit and in bfloat16, and compared with the
whole-sequence oracle.  Weights are stored in bfloat16 so that both paths and the oracle read the
same values; logits are wanted at a subset of the places to keep the oracle affordable.
"""

import pytest
import torch

import replay_helpers as rh
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
PAGE = 16


def wide_configs():
    from tinyvllm_b200.models import Qwen3Config

    common = dict(max_position_embeddings=2048, rope_theta=1_000_000.0, rms_norm_eps=1e-6, head_dim=128)
    return {
        "w06": Qwen3Config(vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=2,
                           num_attention_heads=16, num_key_value_heads=8, tie_word_embeddings=True, **common),
        "w8": Qwen3Config(vocab_size=6000, hidden_size=4096, intermediate_size=12288, num_hidden_layers=2,
                          num_attention_heads=32, num_key_value_heads=8, tie_word_embeddings=False, **common),
        "w32": Qwen3Config(vocab_size=5000, hidden_size=5120, intermediate_size=25600, num_hidden_layers=1,
                           num_attention_heads=64, num_key_value_heads=8, tie_word_embeddings=False, **common),
        # the 14B sizes: five q heads on a kv head (the decode kernel's tile for eight, five rows used)
        "w14": Qwen3Config(vocab_size=4000, hidden_size=5120, intermediate_size=17408, num_hidden_layers=1,
                           num_attention_heads=40, num_key_value_heads=8, tie_word_embeddings=False, **common),
    }


NAMES = ("w06", "w8", "w32", "w14")
LENGTHS = (6, 150, 70, 300, 41, 120, 33)


@pytest.fixture(scope="module")
def wide_folders(tmp_path_factory):
    from tinyvllm_b200.weights.random_init import write_model_folder

    made = {}

    def get(name):
        if name not in made:
            made[name] = write_model_folder(tmp_path_factory.mktemp(f"wide_{name}"), wide_configs()[name],
                                            seed=len(name) + 7, dtype=torch.bfloat16)
        return made[name]

    return get


@pytest.fixture(scope="module")
def wide_runners(wide_folders):
    """One runner at a time (the 32B layer alone is 2 GB in 32-bit)."""
    from tinyvllm_b200.config.registry import read_model_config
    from tinyvllm_b200.engine.model import Model
    from tinyvllm_b200.engine.step import StepRunner

    held = {}

    def get(name, dtype, pages=None, max_requests=8):
        key = (name, dtype, pages, max_requests)
        if key not in held:
            held.clear()
            torch.cuda.empty_cache()
            folder = wide_folders(name)
            model = Model(read_model_config(folder).to_spec(), device="cuda:0", dtype=dtype).load(folder)
            held[key] = StepRunner(model, page_size=PAGE, num_pages=pages or 120, max_requests=max_requests)
        return held[key]

    yield get
    held.clear()
    torch.cuda.empty_cache()


def requests_of(name):
    vocab = wide_configs()[name].vocab_size
    return {f"{name}-{n}": random_tokens(vocab, n, 2000 + n) for n in LENGTHS}


_weights = {}


def check(name, dtype, steps, got, wide_folders, what):
    folder = wide_folders(name)
    if name not in _weights:
        _weights.clear()
        import plain_qwen3 as plain
        _weights[name] = plain.read_weights(folder)
    expected = rh.oracle(folder, requests_of(name), dtype, positions=rh.wanted_positions(steps),
                         weights=_weights[name])
    return rh.compare(got, expected, dtype, what=f"{what} {name}")


def trace_whole(requests):
    return rh.thin(rh.whole(requests), keep_every=7), None


def trace_tail(requests):
    """Decode steps of one request: the fused decode kernel with all q heads of a kv head in one CTA
    and its context cut over a cluster, and the small-batch products (or the library's, by size)."""
    return rh.tail_by_one(requests, tail=20), None


def trace_portions(requests):
    return rh.thin(rh.portions(requests, seed=5, sizes=(2, 9, 33, 64, 130)), keep_every=5, tail=6), None


def trace_mixed(requests):
    """Portions beside decoded tokens of up to four live requests, with so few pages that they are
    used again."""
    steps = rh.mixed(requests, seed=3, sizes=(2, 17, 40, 128))
    held, pages = {}, 0
    for step in steps:
        for entry in step["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        pages = max(pages, sum(-(-n // PAGE) for n in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    assert pages * PAGE < sum(len(t) for t in requests.values())
    return rh.thin(steps, keep_every=6, tail=4), pages


MODES = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions, "mixed": trace_mixed}
CASES = [(name, dtype, mode) for name in NAMES for dtype in DTYPES for mode in MODES]


@pytest.mark.parametrize("name,dtype,mode", CASES,
                         ids=[f"{n}-{'f32' if d == torch.float32 else 'bf16'}-{m}" for n, d, m in CASES])
def test_every_way_of_cutting_at_real_widths(name, dtype, mode, wide_runners, wide_folders):
    steps, pages = MODES[mode](requests_of(name))
    runner = wide_runners(name, dtype) if pages is None else wide_runners(name, dtype, pages=pages, max_requests=4)
    with torch.inference_mode():
        got = rh.run_steps(runner, steps)
    assert all(pool.free_count == pool.num_pages for pool in runner.manager.pools)
    check(name, dtype, steps, got, wide_folders, mode)


@pytest.mark.parametrize("name", ["w06", "w32"])
def test_decode_graphs_with_padding_rows_against_the_oracle(name, wide_runners, wide_folders, monkeypatch):
    """Three requests decode in a graph captured for four rows (one row is padding), in bfloat16: the
    logits the graph leaves are the oracle's and, to rounding in the head, those of the same steps
    run eagerly.  (The eager steps cut every context into as many pieces as the graph of four rows
    does: the number fitted to three rows would merge partial sums in another order, which is a
    difference of rounding in the attention, not of the padding row that this test is about.)"""
    from tinyvllm_b200.engine.graphs import DecodeGraphs
    from tinyvllm_b200.engine.step import StepEntry
    from tinyvllm_b200.ops import attention as attention_ops
    from tinyvllm_b200.sampling.params import SamplingParams

    monkeypatch.setattr(attention_ops, "FEW_ROWS", 0)

    dtype = torch.bfloat16
    requests = {rid: tokens for rid, tokens in list(requests_of(name).items())[1:4]}      # 150, 70, 300 tokens
    tail = 10
    rows = {}
    eager_rows = {}
    for use_graphs in (False, True):
        runner = wide_runners(name, dtype, pages=121 if use_graphs else 122, max_requests=4)
        graphs = None
        if use_graphs:
            graphs = DecodeGraphs(runner, [4], max_model_len=runner.max_model_len)
            graphs.capture()
        with torch.inference_mode():
            for rid, tokens in requests.items():
                runner.open(rid)
                runner.run([StepEntry(rid, tuple(tokens[:-tail]), ())])
            for step in range(tail):
                entries = [StepEntry(rid, (tokens[len(tokens) - tail + step],), (0,))
                           for rid, tokens in requests.items()]
                if graphs is None:
                    logits = runner.run(entries)
                else:
                    plan = runner.plan(entries)
                    _, logits = graphs.run(plan, entries, [SamplingParams()] * 3, [0] * 3)
                    runner.manager.commit(plan)
                target = rows if use_graphs else eager_rows
                for index, (rid, tokens) in enumerate(requests.items()):
                    target[(rid, len(tokens) - tail + step)] = logits[index].float().cpu().clone()
            for rid in requests:
                runner.close(rid)
    assert rows.keys() == eager_rows.keys()
    for key in rows:
        # the same request beside two others or beside two others and a padding row: the library
        # product of the head may sum in another order for three rows than for four
        scale = eager_rows[key].abs().max().item()
        assert (rows[key] - eager_rows[key]).abs().max().item() <= 1e-4 * scale, key
    folder = wide_folders(name)
    import plain_qwen3 as plain
    if name not in _weights:
        _weights.clear()
        _weights[name] = plain.read_weights(folder)
    positions = {rid: {p for (r, p) in rows if r == rid} for rid in requests}
    expected = rh.oracle(folder, requests, dtype, positions=positions, weights=_weights[name])
    rh.compare(rows, expected, dtype, what=f"decode graph {name}")
