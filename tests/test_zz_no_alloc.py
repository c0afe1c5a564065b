"""The allocation-free entry point, sddmm_count_cols_noalloc, against the existing
sddmm_plan_count_cols on the same inputs.

It is for callers that must not enter the CUDA allocator (all device memory owned
by someone else's pool, no tolerance for cudaMalloc's device-wide synchronisation,
code running inside a foreign callback).  Its scratch is a fixed array inside the
library that every call on a GPU shares and that still holds the previous call's
marks, so the check is made on two calls in a row whose column sets differ: the
second answer is only right if the first call's marks were cleared.  The result is
an integer count, so agreement is exact.

This file sorts last so that a run which stops at the first failure has already
been through every other test.
"""
import numpy as np
import pytest
import torch

from sddmm_gpu_b200 import api

pytestmark = pytest.mark.gpu


def _reference_count(handle, M, N, rows, cols):
    plan = handle.plan_coo(M, N, rows, cols, 8)
    try:
        return plan.count_cols()
    finally:
        plan.close()


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    handle = api.Handle(0)   # own handle: the test must also pass alone in a fresh process
    try:
        g = torch.Generator(device="cuda")
        g.manual_seed(1234)
        M, N, nnz = 5000, 300_000, 400_000
        rows = torch.sort(torch.randint(0, M, (nnz,), generator=g, device="cuda", dtype=torch.int32)).values
        # first call: columns spread over the whole range; second: a narrow band, so
        # stale marks from the first call would inflate the second count
        cols_a = torch.randint(0, N, (nnz,), generator=g, device="cuda", dtype=torch.int32)
        cols_b = torch.randint(1000, 1500, (nnz,), generator=g, device="cuda", dtype=torch.int32)
        torch.cuda.synchronize()
        want_a = _reference_count(handle, M, N, rows, cols_a)
        want_b = _reference_count(handle, M, N, rows, cols_b)
        got_a = api.count_cols_noalloc(cols_a, N)
        got_b = api.count_cols_noalloc(cols_b, N)
        assert got_a == want_a == int(torch.unique(cols_a).numel())
        assert got_b == want_b == int(torch.unique(cols_b).numel())
        assert got_b <= 500 < got_a
        # again, on a caller's stream, and the empty matrix
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        assert api.count_cols_noalloc(cols_a, N, cuda_stream=side.cuda_stream) == want_a
        assert api.count_cols_noalloc(cols_a[:0], N, nnz=0) == 0
    finally:
        handle.close()


def test_indices_outside_the_matrix_are_ignored():
    """-1 and N are not columns of the matrix: neither is counted and neither is written."""
    N = 1000
    cols = torch.tensor([-1, 0, 5, 5, N - 1, N, N + 7, -2 ** 31], dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    assert api.count_cols_noalloc(cols, N) == 3
    # the mark just behind the matrix stayed clear: a matrix one column wider sees column N once
    assert api.count_cols_noalloc(cols, N + 1) == 4


def test_sizes_beyond_the_builtin_scratch_are_rejected():
    cols = torch.zeros(4, dtype=torch.int32, device="cuda")
    with pytest.raises(api.SddmmError) as e:
        api.count_cols_noalloc(cols, api.NOALLOC_MAX_COLS + 1)
    assert e.value.status == api.INVALID_ARG
    assert "SDDMM_NOALLOC_MAX_COLS" in str(e.value)
    # the limit itself is accepted
    assert api.count_cols_noalloc(cols, api.NOALLOC_MAX_COLS) == 1
