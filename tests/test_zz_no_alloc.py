"""The allocation-free decode attention entry point, called through its exported C symbol.

Some callers of the kernel library cannot allocate device memory at all: a host program that gave
the whole GPU to its own pool at start-up, a serving loop in which an allocation (and the device-wide
synchronisation it may bring) is forbidden once requests flow, a plug-in that only ever receives raw
pointers.  For them ``tb_attention_decode_noalloc`` keeps the per-split partial results in a 16 MiB
array inside the library image.  This test calls it the way such a caller would (ctypes on the shared
library, raw pointers, no Python wrapper), twice in a row on different inputs, because the array is
shared by all calls and keeps the previous call's contents, and checks each result against the
ordinary entry point, which takes its scratch buffers from the caller, and against the plain
whole-sequence attention of the test suite.

The file sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""

import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from tesseract_b200.csrc.build import load_library

    lib = load_library("attention_noalloc")
    lib.tb_attention_noalloc_floats_needed.restype = ctypes.c_int64
    lib.tb_attention_noalloc_strerror.restype = ctypes.c_char_p
    return lib


def _call(lib, case, nh, nkv, d, page_size, window, scale, splits, claimed_head_dim=None):
    rows = case["q"].shape[0]
    new, lengths = case["new"], case["lengths"]
    row_start = torch.tensor(np.concatenate([[0], np.cumsum(new)]), dtype=torch.int32, device="cuda")
    seq_begin = torch.tensor([n - q for n, q in zip(lengths, new)], dtype=torch.int32, device="cuda")
    q = case["q"].cuda().view(rows, nh * d)
    cache, table = case["cache"].cuda(), case["table"].cuda()
    out = torch.full((rows, nh * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    p, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    status = lib.tb_attention_decode_noalloc(
        p(q.data_ptr()), i64(q.stride(0)), p(out.data_ptr()), i64(out.stride(0)), p(cache.data_ptr()),
        p(row_start.data_ptr()), p(seq_begin.data_ptr()), p(table.data_ptr()), i32(table.stride(0)),
        i32(len(lengths)), i32(rows), i32(max(new)), i32(nh), i32(nkv), i32(claimed_head_dim or d), i32(page_size),
        i32(window),
        ctypes.c_float(scale), i32(splits), p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return status, out


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from tests.test_kernels_gpu import paged_case, plain_paged_attention, run_attention_mma

    lib = _library()
    nh, nkv, d, page_size = 32, 8, 64, 16
    scale = 1.0 / math.sqrt(d)
    calls = [([700, 64, 65, 1], [1, 1, 1, 1], 12, 11), ([2100, 300, 31], [1, 2, 1], 9, 12)]   # more than 8 splits use the scratch
    for lengths, new, splits, seed in calls:          # the second call finds the first call's leftovers
        case = paged_case(torch.bfloat16, lengths, new, nh, nkv, d, page_size, seed=seed)
        want = run_attention_mma(case, nh, nkv, d, page_size, 0, scale, splits)
        status, got = _call(lib, case, nh, nkv, d, page_size, 0, scale, splits)
        assert status == 0, lib.tb_attention_noalloc_strerror(status).decode()
        assert not torch.isnan(got.float()).any()
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        plain = plain_paged_attention(case, scale).reshape(got.shape)
        torch.testing.assert_close(got.cpu().double(), plain, rtol=2e-2, atol=2e-2)


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from tests.test_kernels_gpu import paged_case

    lib = _library()
    limit = 4 * 1024 * 1024
    # (splits, sequences, kv heads, head size): sixteen folded rows of 64 + 2 floats per (split, sequence, kv head)
    assert lib.tb_attention_noalloc_floats_needed(12, 4, 8, 64) == 12 * 4 * 8 * 16 * (64 + 2)
    assert lib.tb_attention_noalloc_floats_needed(8, 4000, 8, 64) == 0          # up to 8 splits use no scratch
    assert lib.tb_attention_noalloc_floats_needed(32, 64, 8, 64) > limit
    case = paged_case(torch.bfloat16, [40] * 64, [1] * 64, 32, 8, 64, 16, seed=1)
    status, out = _call(lib, case, 32, 8, 64, 16, 0, 0.125, 32)
    assert status == -5 and torch.isnan(out.float()).all()          # refused, and nothing was launched
    assert b"16 MiB" in lib.tb_attention_noalloc_strerror(status)
    status, _ = _call(lib, paged_case(torch.bfloat16, [40], [1], 4, 2, 16, 16, seed=2), 4, 2, 16, 16, 0, 0.2, 2,
                      claimed_head_dim=20)
    assert status == -3                                              # a head size the kernels do not take


def test_no_alloc_entry_point_takes_any_size_that_needs_no_scratch():
    """Up to eight splits meet inside a thread-block cluster: the static array is not touched, so its limit does
    not apply, however many sequences the call has (here more than the array could serve with nine splits)."""
    from tests.test_kernels_gpu import paged_case, run_attention_mma

    lib = _library()
    nh, nkv, d, page_size, splits = 8, 8, 64, 16, 8
    lengths = [130 + (k % 7) for k in range(600)]
    assert 9 * len(lengths) * nkv * 16 * (d + 2) > 4 * 1024 * 1024
    case = paged_case(torch.bfloat16, lengths, [1] * len(lengths), nh, nkv, d, page_size, seed=3)
    want = run_attention_mma(case, nh, nkv, d, page_size, 0, 0.125, splits)
    status, got = _call(lib, case, nh, nkv, d, page_size, 0, 0.125, splits)
    assert status == 0, lib.tb_attention_noalloc_strerror(status).decode()
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
