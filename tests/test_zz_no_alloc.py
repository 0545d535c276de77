"""The attention entry point that allocates nothing, called through its exported C symbol.

``tvb_attention_rows_static`` is for programs that may not allocate device memory once they
run (a host that gave the whole GPU to its own pool, a plug-in under a fixed budget): the
scratch that the split mode of the row attention kernel needs lives inside the library
instead of being passed in.  This test calls the symbol with ctypes, twice in a row with
different inputs (the scratch keeps the first call's contents), and compares each result
with the existing entry point, ``tvb_attention_rows``, given a scratch buffer of its own.
It also checks that a batch too large for the built-in scratch is refused, not run.

The file is collected last so that a run stopping at the first failure has already run
every other test."""

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F32, BF16 = 0, 1


def library():
    from tinyvllm_b200.ops.build import load_library

    lib = load_library("attention_rows")
    common = [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]
    tail = [c_int] * 7 + [c_float, c_int, c_void_p]
    lib.tvb_attention_rows.argtypes = common + [c_void_p] + tail        # ... out, scratch, max_chunks, ...
    lib.tvb_attention_rows.restype = c_int
    lib.tvb_attention_rows_static.argtypes = common + tail              # ... out, max_chunks, ...
    lib.tvb_attention_rows_static.restype = c_int
    lib.tvb_attention_rows_static_capacity.restype = c_longlong
    lib.tvb_attention_rows_static_error.argtypes = [c_int]
    lib.tvb_attention_rows_static_error.restype = ctypes.c_char_p
    return lib


def make_case(dtype, seed, *, nq=6, nkv=2, d=48, page=8, lengths=(700, 33, 300), tokens_each=3):
    g = torch.Generator().manual_seed(seed)
    pages = sum(-(-n // page) for n in lengths) + 2
    order = torch.randperm(pages, generator=g).tolist()
    kc = torch.randn(pages, nkv, page, d, generator=g).to(dtype)
    vc = torch.randn(pages, nkv, page, d, generator=g).to(dtype)
    blocks = max(-(-n // page) for n in lengths)
    tables = torch.zeros(len(lengths), blocks, dtype=torch.int32)
    token_row, positions = [], []
    for r, n in enumerate(lengths):
        for b in range(-(-n // page)):
            tables[r, b] = order.pop()
        for p in range(max(0, n - tokens_each), n):
            token_row.append(r), positions.append(p)
    q = torch.randn(len(positions), nq * d, generator=g).to(dtype)
    to_dev = lambda t: t.to(DEV).contiguous()
    return dict(q=to_dev(q), kc=to_dev(kc), vc=to_dev(vc), tables=to_dev(tables),
                token_row=to_dev(torch.tensor(token_row, dtype=torch.int32)),
                positions=to_dev(torch.tensor(positions, dtype=torch.int32)),
                nq=nq, nkv=nkv, d=d, page=page, max_position=max(positions))


def call(lib, case, dtype, *, static, max_chunks, scratch=None):
    tokens = case["positions"].shape[0]
    out = torch.full((tokens, case["nq"] * case["d"]), float("nan"), dtype=dtype, device=DEV)
    head = [case["q"].data_ptr(), case["nq"] * case["d"], case["kc"].data_ptr(), case["vc"].data_ptr(),
            case["tables"].data_ptr(), case["tables"].shape[1], case["token_row"].data_ptr(),
            case["positions"].data_ptr(), out.data_ptr()]
    tail = [max_chunks, tokens, case["nq"], case["nkv"], case["d"], case["page"], 0, case["d"] ** -0.5,
            F32 if dtype == torch.float32 else BF16, torch.cuda.current_stream().cuda_stream]
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    if static:
        code = lib.tvb_attention_rows_static(*head, *tail)
    else:
        code = lib.tvb_attention_rows(*head, scratch.data_ptr(), *tail)
    torch.cuda.synchronize()
    call.device_memory_taken = free_before - torch.cuda.mem_get_info()[0]
    return code, out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_static_entry_point_matches_the_one_with_a_scratch_argument(dtype):
    lib = library()
    assert lib.tvb_attention_rows_static_capacity() == 4 * 1024 * 1024
    limit = 3e-6 if dtype == torch.float32 else 8e-3          # the tolerances of test_kernels_gpu.py
    for seed, lengths in ((1, (700, 33, 300)), (2, (90, 515, 260, 5))):    # two calls in a row
        case = make_case(dtype, seed, lengths=lengths)
        max_chunks = case["max_position"] // 256 + 1
        tokens = case["positions"].shape[0]
        need = tokens * case["nq"] * max_chunks * (case["d"] + 2)
        scratch = torch.empty(need, dtype=torch.float32, device=DEV)
        code, want = call(lib, case, dtype, static=False, max_chunks=max_chunks, scratch=scratch)
        assert code == 0
        code, got = call(lib, case, dtype, static=True, max_chunks=max_chunks)
        assert code == 0, lib.tvb_attention_rows_static_error(code).decode()
        assert call.device_memory_taken == 0                 # the device's free memory did not move
        assert torch.isfinite(got.float()).all()
        scale = want.float().abs().max().item()
        assert (got.float() - want.float()).abs().max().item() <= limit * scale


def test_static_entry_point_refuses_what_does_not_fit():
    lib = library()
    case = make_case(torch.float32, 3)
    code, out = call(lib, case, torch.float32, static=True, max_chunks=60000)
    assert code == -2 and torch.isnan(out).all()              # refused before anything ran
    assert b"do not fit" in lib.tvb_attention_rows_static_error(code)
    code, _ = call(lib, case, torch.float32, static=True, max_chunks=0)
    assert code == -1
