"""The entry point for callers that cannot allocate device memory (a plug-in inside another
program's memory budget, a loop that may not take the allocator's lock): decode attention whose
scratch is a fixed array inside the library, ``zb_paged_decode_no_alloc``.

It is called here through its exported C symbol, straight from the shared library, twice in a row
(the second call finds the first call's partial results still in the shared array), and its output
is compared with the ordinary entry point's, which takes a scratch buffer from the caller.  A
problem too large for the built-in array must be refused with the code the header names.

This file sorts last on purpose: should it fail, a run that stops at the first failure has
already run every other test."""

import ctypes
import math
import random
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

NH, NKV, HD, PAGE = 16, 8, 128, 16
SCRATCH_BYTES = 4 << 20
ERR_SCRATCH_TOO_SMALL = 4


def make_case(device, contexts, seed, nh=NH, nkv=NKV):
    """Random queries and a paged cache holding ``contexts[r] + 1`` positions for row r."""
    g = torch.Generator().manual_seed(seed)
    rows = len(contexts)
    totals = [c + 1 for c in contexts]
    pages_needed = sum(-(-n // PAGE) for n in totals)
    num_pages = pages_needed + 2
    order = list(range(1, num_pages))
    random.Random(seed).shuffle(order)
    width = max(-(-n // PAGE) for n in totals)
    table = torch.zeros((rows, width), dtype=torch.int32)
    cursor = 0
    for r, n in enumerate(totals):
        need = -(-n // PAGE)
        table[r, :need] = torch.tensor(order[cursor:cursor + need], dtype=torch.int32)
        cursor += need
    cache = torch.randn((num_pages, 2, nkv, PAGE, HD), generator=g).to(torch.bfloat16).to(device)
    q = torch.randn((rows, nh * HD), generator=g).to(torch.bfloat16).to(device)
    return dict(
        nh=nh, nkv=nkv, q=q, cache=cache, table=table.to(device), num_pages=num_pages,
        rows=torch.arange(rows, dtype=torch.int32, device=device),
        row_q_start=torch.arange(rows, dtype=torch.int32, device=device),
        row_ctx=torch.tensor(contexts, dtype=torch.int32, device=device))


def load_symbol():
    from zephyr_b200.kernels.build import build_library

    lib = ctypes.CDLL(str(build_library()))
    fn = lib.zb_paged_decode_no_alloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                   c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p]
    lib.zb_paged_decode_no_alloc_bytes_needed.restype = c_longlong
    lib.zb_paged_decode_no_alloc_bytes_needed.argtypes = [c_int, c_int, c_int, c_int, c_int, c_int]
    lib.zb_paged_decode_no_alloc_error.restype = ctypes.c_char_p
    lib.zb_paged_decode_no_alloc_error.argtypes = [c_int]
    return lib


def call_no_alloc(lib, case, out, status, split_size, max_splits, n_rows=None):
    n_rows = case["rows"].numel() if n_rows is None else n_rows
    return lib.zb_paged_decode_no_alloc(
        out.data_ptr(), case["q"].data_ptr(), case["cache"].data_ptr(), case["table"].data_ptr(),
        case["table"].shape[1], PAGE, case["num_pages"], case["table"].shape[0], case["rows"].data_ptr(), n_rows,
        case["row_q_start"].data_ptr(), case["row_ctx"].data_ptr(), case["nh"], case["nkv"], HD, 0, 1.0 / math.sqrt(HD), split_size,
        max_splits, status.data_ptr(), torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("split", ["fixed", "balanced"])
def test_no_alloc_entry_point_matches_the_ordinary_one(cuda_device, split):
    from zephyr_b200.kernels import ops

    lib = load_symbol()
    split_size = ops.DECODE_SPLIT_SIZE if split == "fixed" else 0
    # Two different problems in a row: the second finds the first one's partial results in the array.
    for seed, contexts in ((1, [0, 255, 256, 1000, 77]), (2, [600, 3, 2047])):
        case = make_case(cuda_device, contexts, seed)
        max_splits = math.ceil((max(contexts) + 1) / (split_size or 32))
        status = ops.new_status(cuda_device)
        expected = torch.zeros_like(case["q"])
        ops.paged_decode(case["q"], case["cache"], case["table"], case["rows"], case["row_q_start"], case["row_ctx"],
                         max(contexts) + 1, NH, NKV, HD, 0, 1.0 / math.sqrt(HD), status, out=expected,
                         split_size=split_size)
        got = torch.full_like(case["q"], float("nan"))
        assert 0 < lib.zb_paged_decode_no_alloc_bytes_needed(len(contexts), NH, NKV, HD, split_size, max_splits) \
            <= SCRATCH_BYTES
        rc = call_no_alloc(lib, case, got, status, split_size, max_splits)
        assert rc == 0, lib.zb_paged_decode_no_alloc_error(rc).decode()
        torch.cuda.synchronize()
        ops.check_status(status)
        # The same kernel on the same inputs, cut in the same way and merged in the same order: every
        # bit agrees, wherever the scratch lies.
        assert torch.equal(got, expected)


def test_no_alloc_entry_point_refuses_what_does_not_fit(cuda_device):
    from zephyr_b200.kernels import ops

    lib = load_symbol()
    case = make_case(cuda_device, [10, 20], 3)
    out = torch.zeros_like(case["q"])
    status = ops.new_status(cuda_device)
    too_many_splits = SCRATCH_BYTES // (2 * NH * (HD + 2) * 4) + 1
    assert lib.zb_paged_decode_no_alloc_bytes_needed(2, NH, NKV, HD, ops.DECODE_SPLIT_SIZE, too_many_splits) > SCRATCH_BYTES
    rc = call_no_alloc(lib, case, out, status, ops.DECODE_SPLIT_SIZE, too_many_splits)
    assert rc == ERR_SCRATCH_TOO_SMALL
    assert b"4 MiB" in lib.zb_paged_decode_no_alloc_error(rc)
    torch.cuda.synchronize()
    assert out.abs().max() == 0         # nothing was launched


def test_no_alloc_entry_point_sizes_balanced_items_by_the_group(cuda_device):
    """With balanced items the partial results number two per CTA and query head of a group, whatever
    the rows are: a group of 16 heads of size 128 needs more than the array holds and is refused
    before anything is cleared or launched, although the fixed-split formula would call it tiny."""
    from zephyr_b200.kernels import ops

    lib = load_symbol()
    nh, nkv = 32, 2
    case = make_case(cuda_device, [40, 300], 4, nh=nh, nkv=nkv)
    out = torch.zeros_like(case["q"])
    status = ops.new_status(cuda_device)
    max_splits = math.ceil(301 / 32)
    assert lib.zb_paged_decode_no_alloc_bytes_needed(2, nh, nkv, HD, ops.DECODE_SPLIT_SIZE, 2) <= SCRATCH_BYTES
    assert lib.zb_paged_decode_no_alloc_bytes_needed(2, nh, nkv, HD, 0, max_splits) > SCRATCH_BYTES
    assert call_no_alloc(lib, case, out, status, 0, max_splits) == ERR_SCRATCH_TOO_SMALL
    torch.cuda.synchronize()
    ops.check_status(status)
    assert out.abs().max() == 0         # nothing was launched
    # The same shape with fixed splits fits and runs.
    expected = torch.zeros_like(case["q"])
    ops.paged_decode(case["q"], case["cache"], case["table"], case["rows"], case["row_q_start"], case["row_ctx"],
                     301, nh, nkv, HD, 0, 1.0 / math.sqrt(HD), status, out=expected, split_size=ops.DECODE_SPLIT_SIZE)
    assert call_no_alloc(lib, case, out, status, ops.DECODE_SPLIT_SIZE, 2) == 0
    torch.cuda.synchronize()
    ops.check_status(status)
    assert torch.equal(out, expected)
