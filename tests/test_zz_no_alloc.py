"""The allocation-free attention entry point, called through its exported C symbol.

Some users of the kernels cannot allocate device memory when they need attention: the GPU's
memory is all handed out already, or they sit in a loop that must not touch an allocator, or
they use the library without PyTorch.  For them ``pylon_paged_attention_mma_static``
(``csrc/attention_static.cu``) keeps the scratch for partial results and the counters in
fixed arrays inside the library.  This test calls that symbol with raw pointers, several times in a
row on different inputs and then on the first again (the arrays keep what the last call left, so
the later calls show whether stale contents matter), and compares with a plain statement of
attention and with the ordinary entry point, which gets its scratch from the caller.  After every
call the library's error word must be zero.  It also checks that a job too large for the built-in
scratch is refused, and that the counters can be put back after an error (written from the host).

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


def load_static_library(head_dim: int = HEAD_DIM):
    from pylon_b200.kernels import build

    library = build.load("attention_static.cu", {"PYLON_HEAD_DIM": head_dim})
    function = library.pylon_paged_attention_mma_static
    function.argtypes = [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                         c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_void_p]
    function.restype = c_int
    library.pylon_static_scratch_floats.restype = c_longlong
    library.pylon_attention_scratch_floats.argtypes = [c_int, c_int, c_int, c_int, c_int, c_int]
    library.pylon_attention_scratch_floats.restype = c_longlong
    library.pylon_static_error_word.restype = c_int
    library.pylon_static_reset.restype = c_int
    library.pylon_static_inject.argtypes = [c_int, ctypes.c_uint, c_int]
    library.pylon_static_inject.restype = c_int
    return library


def call_static(library, fused, cache, nq, nkv, window, splits, out, head_dim: int = HEAD_DIM):
    pointer = lambda tensor: c_void_p(tensor.data_ptr())
    return library.pylon_paged_attention_mma_static(
        pointer(fused), fused.stride(0), pointer(cache.k_pages), pointer(cache.v_pages), pointer(out), pointer(cache.q_start),
        pointer(cache.kv_len), pointer(cache.table), cache.table.shape[1], cache.page_size, cache.k_pages.shape[0], nq, nkv,
        int(window or 0), 1.0 / math.sqrt(head_dim), len(cache.kv_lens), cache.tokens, max(cache.q_lens), splits,
        c_void_p(torch.cuda.current_stream().cuda_stream),
    )


CASES = [
    # head size, kv_lens, q_lens, page size, window, splits
    (64, [300, 64, 65, 7, 1, 129], [1, 1, 1, 1, 1, 1], 64, None, 4),        # decoded tokens
    (64, [200, 90, 33], [70, 1, 2], 16, 50, 3),                             # a prompt portion beside them, a window
    (128, [700, 1030, 257], [1, 1, 1], 256, None, 1),                       # the serving geometry: head size 128, pages of 256
    (64, [900] * 40, [1] * 40, 64, None, 1),                                # 80 (row, KV head) pairs: runs that cross pairs
]


def run_case(libraries, number, nq=8, nkv=2):
    from pylon_b200.kernels import ops
    from test_kernels_gpu import Paged, attention_reference

    head_dim, kv_lens, q_lens, page, window, splits = CASES[number]
    library = libraries[head_dim]
    torch.manual_seed(77 + number)
    cache = Paged(kv_lens, q_lens, nkv, head_dim, page, torch.bfloat16, seed=number)
    fused = torch.randn(cache.tokens, (nq + 2 * nkv) * head_dim, device="cuda").to(torch.bfloat16)
    out = torch.full((cache.tokens, nq * head_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
    code = call_static(library, fused, cache, nq, nkv, window, splits, out, head_dim)
    assert code == 0, library.pylon_last_error().decode()
    torch.cuda.synchronize()
    assert library.pylon_static_error_word() == 0
    plain = attention_reference(fused[:, : nq * head_dim].reshape(cache.tokens, nq, head_dim), cache, nq, nkv, head_dim, window, 1.0 / math.sqrt(head_dim))
    torch.testing.assert_close(out.double(), plain, rtol=2e-2, atol=2e-2)
    ordinary = ops.paged_attention(
        fused, cache.k_pages, cache.v_pages, cache.positions, cache.token_row, cache.q_start, cache.kv_len, cache.table, nq,
        max(q_lens), max(kv_lens), window=window, num_splits=splits,
    )
    torch.testing.assert_close(out.float(), ordinary.float(), rtol=2e-2, atol=2e-2)
    return library


def test_static_scratch_entry_point_matches_plain_attention_call_after_call():
    libraries = {64: load_static_library(64), 128: load_static_library(128)}
    assert libraries[64].pylon_static_scratch_floats() == 4 * 1024 * 1024
    for number in (0, 1, 2, 3, 0, 3, 1):    # the first case again after the others: the same counters and scratch slots
        run_case(libraries, number)


def test_static_counters_can_be_put_back_after_an_error():
    """A kernel that gives up leaves the error word set and counters of the rows it shared above zero.  Both are
    written from the host here (no kernel is made to give up); after pylon_static_reset() the next call is right."""
    libraries = {64: load_static_library(64), 128: load_static_library(128)}
    library = run_case(libraries, 0)
    assert library.pylon_static_inject(0, 1, 1) == 0 and library.pylon_static_inject(5, 2, 1) == 0
    assert library.pylon_static_error_word() == 1
    assert library.pylon_static_reset() == 0
    assert library.pylon_static_error_word() == 0
    run_case(libraries, 0)
    run_case(libraries, 3)


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
