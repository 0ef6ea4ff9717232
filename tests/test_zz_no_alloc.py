"""The allocation-free attention entry point, called through its exported C symbol.

Some users of the kernels cannot allocate device memory when they need attention: the GPU's
memory is all handed out already, or they sit in a loop that must not touch an allocator, or
they use the library without PyTorch.  For them ``pylon_paged_attention_mma_static``
(``csrc/attention_static.cu``) keeps the scratch for partial results and the counters in
fixed arrays inside the library.  This test calls that symbol with raw pointers, twice in a row on different
inputs (the array keeps what the last call left, so the second call shows whether stale
contents matter), and compares with the ordinary entry point, which gets its scratch from
the caller.  It also checks that a job too large for the built-in scratch is refused.

The file name sorts last on purpose: if this test fails in a run that stops at the first
failure, every other test has already run.
"""
from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

HEAD_DIM = 64


def load_static_library():
    from pylon_b200.kernels import build

    library = build.load("attention_static.cu", {"PYLON_HEAD_DIM": HEAD_DIM})
    function = library.pylon_paged_attention_mma_static
    function.argtypes = [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                         c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_void_p]
    function.restype = c_int
    library.pylon_static_scratch_floats.restype = c_longlong
    library.pylon_attention_scratch_floats.argtypes = [c_int, c_int, c_int, c_int, c_int, c_int]
    library.pylon_attention_scratch_floats.restype = c_longlong
    return library


def call_static(library, fused, cache, nq, nkv, window, splits, out):
    pointer = lambda tensor: c_void_p(tensor.data_ptr())
    return library.pylon_paged_attention_mma_static(
        pointer(fused), fused.stride(0), pointer(cache.k_pages), pointer(cache.v_pages), pointer(out), pointer(cache.q_start),
        pointer(cache.kv_len), pointer(cache.table), cache.table.shape[1], cache.page_size, cache.k_pages.shape[0], nq, nkv,
        int(window or 0), 1.0 / math.sqrt(HEAD_DIM), len(cache.kv_lens), cache.tokens, max(cache.q_lens), splits,
        c_void_p(torch.cuda.current_stream().cuda_stream),
    )


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from pylon_b200.kernels import ops
    from test_kernels_gpu import Paged

    library = load_static_library()
    assert library.pylon_static_scratch_floats() == 4 * 1024 * 1024
    nq, nkv = 8, 2
    cases = [
        # kv_lens, q_lens, page size, window, splits: decoded tokens, then a mix with a prompt portion
        ([300, 64, 65, 7, 1, 129], [1, 1, 1, 1, 1, 1], 64, None, 4),
        ([200, 90, 33], [70, 1, 2], 16, 50, 3),
    ]
    for number, (kv_lens, q_lens, page, window, splits) in enumerate(cases):
        torch.manual_seed(77 + number)
        cache = Paged(kv_lens, q_lens, nkv, HEAD_DIM, page, torch.bfloat16, seed=number)
        fused = torch.randn(cache.tokens, (nq + 2 * nkv) * HEAD_DIM, device="cuda").to(torch.bfloat16)
        expected = ops.paged_attention(
            fused, cache.k_pages, cache.v_pages, cache.positions, cache.token_row, cache.q_start, cache.kv_len, cache.table, nq,
            max(q_lens), max(kv_lens), window=window, num_splits=splits,
        )
        out = torch.full((cache.tokens, nq * HEAD_DIM), float("nan"), dtype=torch.bfloat16, device="cuda")
        code = call_static(library, fused, cache, nq, nkv, window, splits, out)
        assert code == 0, library.pylon_last_error().decode()
        torch.cuda.synchronize()
        torch.testing.assert_close(out.float(), expected.float(), rtol=2e-2, atol=2e-2)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from test_kernels_gpu import Paged

    library = load_static_library()
    nq, nkv = 8, 2
    cache = Paged([40], [40], nkv, HEAD_DIM, 16, torch.bfloat16)
    fused = torch.randn(cache.tokens, (nq + 2 * nkv) * HEAD_DIM, device="cuda").to(torch.bfloat16)
    out = torch.zeros((cache.tokens, nq * HEAD_DIM), dtype=torch.bfloat16, device="cuda")
    # claim a job of 100,000 tokens and 64 splits: far beyond 4 Mi floats; nothing may be launched
    needed = library.pylon_attention_scratch_floats(64, 100_000, nq, 1, nkv, 0)   # one long row: no blocks for decoded rows
    assert needed > library.pylon_static_scratch_floats()
    pointer = lambda tensor: c_void_p(tensor.data_ptr())
    code = library.pylon_paged_attention_mma_static(
        pointer(fused), fused.stride(0), pointer(cache.k_pages), pointer(cache.v_pages), pointer(out), pointer(cache.q_start),
        pointer(cache.kv_len), pointer(cache.table), cache.table.shape[1], cache.page_size, cache.k_pages.shape[0], nq, nkv, 0,
        1.0 / math.sqrt(HEAD_DIM), 1, 100_000, 40, 64, c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    assert code == -1
    text = library.pylon_last_error().decode()
    assert "scratch" in text and str(needed) in text
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0
