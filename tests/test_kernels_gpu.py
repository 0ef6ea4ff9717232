"""Each CUDA kernel alone against a plain PyTorch float32/float64 statement of the same
operation, at sizes other than the engine's tiny models."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEVICE = "cuda"


def tolerance(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(1234)


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab, width, tokens", [(1000, 2560, 37), (77, 50, 5), (151_936, 96, 3)])
def test_embed_gather(dtype, vocab, width, tokens):
    from pylon_b200.kernels import ops

    table = torch.randn(vocab, width, device=DEVICE).to(dtype)
    ids = torch.randint(0, vocab, (tokens,), device=DEVICE, dtype=torch.int32)
    ids[0], ids[-1] = vocab - 1, 0
    out = ops.embed_gather(ids, table)
    assert out.dtype == torch.float32
    torch.testing.assert_close(out, table[ids.long()].float(), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens, width, eps", [(19, 2560, 1e-6), (3, 100, 1e-5), (2, 5000, 1e-3), (1, 7, 1e-6)])
def test_add_rmsnorm(dtype, tokens, width, eps):
    from pylon_b200.kernels import ops

    residual = torch.randn(tokens, width, device=DEVICE) * 3
    delta = torch.randn(tokens, width, device=DEVICE).to(dtype)
    weight = torch.rand(width, device=DEVICE) + 0.5
    expected_sum = residual.double() + delta.double()
    expected = expected_sum / torch.sqrt((expected_sum**2).mean(-1, keepdim=True) + eps) * weight.double()
    work = residual.clone()
    out = ops.add_rmsnorm(work, delta, weight, eps, dtype)
    torch.testing.assert_close(work.double(), expected_sum, rtol=1e-6, atol=1e-6)      # the residual sum stays 32-bit
    torch.testing.assert_close(out.double(), expected, **tolerance(dtype))
    # without a delta the residual is left as it is
    work2 = residual.clone()
    out2 = ops.add_rmsnorm(work2, None, weight, eps, dtype)
    plain = residual.double() / torch.sqrt((residual.double() ** 2).mean(-1, keepdim=True) + eps) * weight.double()
    torch.testing.assert_close(out2.double(), plain, **tolerance(dtype))
    assert torch.equal(work2, residual)
    # a row selection normalises those rows of (residual + delta) and writes nothing back
    rows = torch.tensor([tokens - 1, 0], device=DEVICE, dtype=torch.int32)
    work3 = residual.clone()
    out3 = ops.add_rmsnorm(work3, delta, weight, eps, dtype, rows=rows)
    torch.testing.assert_close(out3.double(), expected[rows.long()], **tolerance(dtype))
    assert torch.equal(work3, residual)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens, inter", [(5, 9728), (3, 100), (2, 7), (64, 24)])
def test_swiglu(dtype, tokens, inter):
    from pylon_b200.kernels import ops

    gate_up = (torch.randn(tokens, 2 * inter, device=DEVICE) * 2).to(dtype)
    out = ops.swiglu(gate_up)
    g, u = gate_up[:, :inter].double(), gate_up[:, inter:].double()
    torch.testing.assert_close(out.double(), g * torch.sigmoid(g) * u, **tolerance(dtype))


@pytest.mark.parametrize("m, n, k", [(1, 300, 77), (5, 64, 64), (70, 130, 2560), (129, 1000, 33), (3, 151_936 // 8, 96)])
def test_gemm_f32_is_true_32_bit(m, n, k):
    from pylon_b200.kernels import ops

    x = torch.randn(m, k, device=DEVICE)
    w = torch.randn(n, k, device=DEVICE)
    y = ops.linear(x, w)
    expected = x.double() @ w.double().T
    # a TF32 product would be off by ~1e-3 relative; float32 accumulation stays near 1e-6
    error = (y.double() - expected).abs().max() / expected.abs().max()
    assert float(error) < 2e-6, float(error)
    # a row's result does not depend on the other rows of the launch
    alone = ops.linear(x[:1].contiguous(), w)
    assert torch.equal(alone[0], y[0])


@pytest.mark.parametrize("m, n, k", [(1, 256, 128), (8, 6144, 2560), (40, 1000, 96), (300, 320, 224)])
def test_linear_bf16(m, n, k):
    from pylon_b200.kernels import ops

    x = torch.randn(m, k, device=DEVICE).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEVICE) * 0.05).to(torch.bfloat16)
    expected = x.double() @ w.double().T
    torch.testing.assert_close(ops.linear(x, w).double(), expected, rtol=2e-2, atol=2e-2)
    wide = ops.linear(x, w, out_dtype=torch.float32)
    assert wide.dtype == torch.float32
    torch.testing.assert_close(wide.double(), expected, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 31, 64])
@pytest.mark.parametrize("n, k", [(100, 64), (2560, 4096), (77, 1000), (333, 264)])
def test_skinny_gemm_every_row_count(m, n, k):
    """The weight-streaming kernel on its own, for every tile configuration it has, with row
    and k counts that do not fill its tiles."""
    from pylon_b200.kernels import ops

    x = torch.randn(m, k, device=DEVICE).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEVICE) * 0.05).to(torch.bfloat16)
    expected = x.double() @ w.double().T
    torch.testing.assert_close(ops.linear_skinny(x, w, torch.float32).double(), expected, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(ops.linear_skinny(x, w).double(), expected, rtol=2e-2, atol=2e-2)
    # a strided view of a wider buffer works too (row stride a multiple of 8)
    wide = torch.randn(m, k + 16, device=DEVICE).to(torch.bfloat16)
    view = wide[:, 8 : 8 + k]
    torch.testing.assert_close(ops.linear_skinny(view, w, torch.float32).double(), view.double() @ w.double().T, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("m", [1, 7, 8, 9, 20, 32, 33, 64, 70])
@pytest.mark.parametrize("inter, k", [(9728, 2560), (224, 96), (24, 64)])
def test_linear_swiglu_with_interleaved_weights(m, inter, k):
    """silu(x gate^T) * (x up^T) from weights stacked in alternating groups of 8 rows: fused in
    the product's kernel for few rows (every tile count of the TMA-fed kernel), product plus
    SwiGLU kernel for more."""
    from pylon_b200.kernels import ops

    gate = (torch.randn(inter, k, device=DEVICE) * 0.05).to(torch.bfloat16)
    up = (torch.randn(inter, k, device=DEVICE) * 0.05).to(torch.bfloat16)
    x = torch.randn(m, k, device=DEVICE).to(torch.bfloat16)
    stacked = ops.interleave_gate_up(gate, up)
    assert torch.equal(stacked[:8], gate[:8]) and torch.equal(stacked[8:16], up[:8]) and torch.equal(stacked[16:24], gate[8:16])
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    want = g * torch.sigmoid(g) * u
    torch.testing.assert_close(ops.linear_swiglu(x, stacked).double(), want, rtol=2e-2, atol=2e-2)
    if m <= 64:   # the TMA-fed kernel itself, also where the dispatch prefers the library
        torch.testing.assert_close(ops.linear_stream(x, stacked, swiglu=True).double(), want, rtol=2e-2, atol=2e-2)
        assert int(ops.stream_error_word(torch.device(DEVICE)).item()) == 0
    # the SwiGLU kernel alone on interleaved columns, both dtypes
    for dtype in (torch.bfloat16, torch.float32):
        columns = torch.randn(m, 2 * inter, device=DEVICE).to(dtype)
        pairs = columns.double().reshape(m, inter // 8, 2, 8)
        g2, u2 = pairs[:, :, 0].reshape(m, inter), pairs[:, :, 1].reshape(m, inter)
        torch.testing.assert_close(ops.swiglu(columns, interleaved=True).double(), g2 * torch.sigmoid(g2) * u2, **tolerance(dtype))


@pytest.mark.parametrize("m, n, k", [(128, 256, 64), (256, 512, 128), (300, 320, 224), (2048, 2560, 4096), (1000, 6144, 2560), (129, 136, 72)])
def test_tcgen05_gemm(m, n, k):
    """The TMA + tcgen05 product against float64, with row, column and k counts that do not
    fill its tiles; its bounded waits must never have run out."""
    from pylon_b200.kernels import ops

    x = torch.randn(m, k, device=DEVICE).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEVICE) * 0.05).to(torch.bfloat16)
    y = ops.linear_tcgen05(x, w)
    torch.testing.assert_close(y.double(), x.double() @ w.double().T, rtol=2e-2, atol=2e-2)
    assert int(ops.tcgen05_error_word(x.device).item()) == 0


@pytest.mark.parametrize("columns", [288, 256, 192, 160, 128])
def test_tcgen05_gemm_every_tile_width(columns):
    """Each tile width on its own (the choice by size would never take some of them here),
    with edges inside a tile in both directions, plain and with the SwiGLU epilogue, and
    with strided views as operands."""
    from pylon_b200.kernels import ops

    ops.tcgen05_force_tile(columns)
    try:
        # the last: more tiles than SMs at every width, so that blocks take a second tile (with 288 columns: into the one accumulator)
        for m, n, k in [(128, 256, 64), (300, 328, 224), (130, 72, 64), (700, 1224, 512), (2100, 2560, 320)]:
            x = torch.randn(m, k + 8, device=DEVICE).to(torch.bfloat16)[:, :k]
            w = (torch.randn(n, k + 16, device=DEVICE) * 0.05).to(torch.bfloat16)[:, 8:8 + k]
            torch.testing.assert_close(ops.linear_tcgen05(x, w).double(), x.double() @ w.double().T, rtol=2e-2, atol=2e-2)
        for m, inter, k in [(256, 128, 64), (300, 104, 96), (600, 1000, 512)]:
            gate = (torch.randn(inter, k, device=DEVICE) * 0.05).to(torch.bfloat16)
            up = (torch.randn(inter, k, device=DEVICE) * 0.05).to(torch.bfloat16)
            x = torch.randn(m, k, device=DEVICE).to(torch.bfloat16)
            g, u = x.double() @ gate.double().T, x.double() @ up.double().T
            got = ops.linear_tcgen05(x, ops.interleave_gate_up(gate, up), swiglu=True)
            torch.testing.assert_close(got.double(), g * torch.sigmoid(g) * u, rtol=2e-2, atol=2e-2)
        assert int(ops.tcgen05_error_word(torch.device(DEVICE)).item()) == 0
    finally:
        ops.tcgen05_force_tile(0)


@pytest.mark.parametrize("columns", [128, 256, 288])
def test_tcgen05_gemm_tile_before_a_partly_empty_row_tile(columns):
    """A last row tile whose lower quarters lie outside the matrix stores nothing for them; the tile a block wrote just
    before it must still come out whole (its last store may still be reading its buffer when the block moves on).  Few
    steps of k and several tiles a block make the window wide; two inputs take turns, so that what an earlier call left
    in shared or tensor memory is never the right answer."""
    from pylon_b200.kernels import ops

    m, n, k = 4000, 2560, 128
    xs = [torch.randn(m, k, device=DEVICE).to(torch.bfloat16) for _ in range(2)]
    ws = [(torch.randn(n, k, device=DEVICE) * 0.05).to(torch.bfloat16) for _ in range(2)]
    wants = [x.float() @ w.float().T for x, w in zip(xs, ws)]
    ops.tcgen05_force_tile(columns)
    try:
        for turn in range(40):
            got = ops.linear_tcgen05(xs[turn % 2], ws[turn % 2])
            wrong = (got.float() - wants[turn % 2]).abs() > 0.1
            assert not bool(wrong.any()), f"turn {turn}: {int(wrong.sum())} values off, rows {sorted(set((torch.nonzero(wrong)[:, 0] // 32).tolist()))[:8]} (groups of 32)"
    finally:
        ops.tcgen05_force_tile(0)
    assert int(ops.tcgen05_error_word(torch.device(DEVICE)).item()) == 0


@pytest.mark.parametrize("m, inter, k", [(128, 128, 64), (2048, 9728, 2560), (130, 104, 96), (500, 224, 96)])
def test_tcgen05_gemm_with_swiglu_epilogue(m, inter, k):
    from pylon_b200.kernels import ops

    gate = (torch.randn(inter, k, device=DEVICE) * 0.05).to(torch.bfloat16)
    up = (torch.randn(inter, k, device=DEVICE) * 0.05).to(torch.bfloat16)
    x = torch.randn(m, k, device=DEVICE).to(torch.bfloat16)
    stacked = ops.interleave_gate_up(gate, up)
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    want = g * torch.sigmoid(g) * u
    torch.testing.assert_close(ops.linear_tcgen05(x, stacked, swiglu=True).double(), want, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(ops.linear_swiglu(x, stacked).double(), want, rtol=2e-2, atol=2e-2)   # the dispatch the feed-forward uses
    assert int(ops.tcgen05_error_word(x.device).item()) == 0
    with pytest.raises(ops.KernelError, match="multiples of 8"):
        ops.linear_tcgen05(torch.zeros(128, 20, device=DEVICE, dtype=torch.bfloat16), torch.zeros(64, 20, device=DEVICE, dtype=torch.bfloat16))


@pytest.mark.parametrize("m", [1, 8, 19, 32])
@pytest.mark.parametrize("n, k", [(2560, 4096), (2560, 9728), (96, 2048)])
def test_partial_sums_for_the_residual(m, n, k):
    """Products with few weight rows come back as float32 partial sums over slices of k; the
    add + RMSNorm kernel adds them to the residual in order."""
    from pylon_b200.kernels import ops

    eps = 1e-5
    x = torch.randn(m, k, device=DEVICE).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEVICE) * 0.05).to(torch.bfloat16)
    parts = ops.linear_for_residual(x, w)
    assert parts.dim() == 3 and parts.dtype == torch.float32 and parts.shape[1:] == (m, n)
    product = x.double() @ w.double().T
    torch.testing.assert_close(parts.double().sum(0), product, rtol=1e-3, atol=1e-3)
    residual = torch.randn(m, n, device=DEVICE)
    weight = torch.rand(n, device=DEVICE) + 0.5
    want_residual = residual.double() + product
    want = want_residual / torch.sqrt((want_residual**2).mean(-1, keepdim=True) + eps) * weight.double()
    work = residual.clone()
    normed = ops.add_rmsnorm(work, parts, weight, eps, torch.bfloat16)
    torch.testing.assert_close(work.double(), want_residual, rtol=1e-3, atol=2e-3)
    torch.testing.assert_close(normed.double(), want, rtol=2e-2, atol=2e-2)
    work2 = residual.clone()
    ops.residual_add(work2, parts)
    torch.testing.assert_close(work2.double(), want_residual, rtol=1e-3, atol=2e-3)
    # a row selection (the final norm) takes the sum of the parts as its delta
    rows = torch.tensor([m - 1], device=DEVICE, dtype=torch.int32)
    picked = ops.add_rmsnorm(residual.clone(), parts, weight, eps, torch.bfloat16, rows=rows)
    torch.testing.assert_close(picked.double(), want[m - 1 :], rtol=3e-2, atol=3e-2)
    # many rows, or a matrix with many rows of its own: the plain product
    assert ops.linear_for_residual(torch.zeros(33, k, device=DEVICE, dtype=torch.bfloat16), w).dim() == 2


@pytest.mark.parametrize("m, n, k", [(1, 64, 64), (8, 2560, 4096), (5, 100, 72), (3, 2564, 4104), (8, 130, 1032), (7, 6144, 2560),
                                     (9, 130, 1032), (16, 2560, 4096), (23, 100, 72), (32, 328, 264), (47, 2564, 520), (64, 2560, 1024)])
def test_stream_gemm_partial_sums(m, n, k):
    """The TMA-fed decode product: row, column and k counts that do not fill its 64 x 64 boxes,
    every tile count of the activations, every sensible number of parts, a strided activation
    view; and the same product in its bfloat16 form."""
    from pylon_b200.kernels import ops

    x = torch.randn(m, k + 16, device=DEVICE).to(torch.bfloat16)[:, 8 : 8 + k]
    w = (torch.randn(n, k, device=DEVICE) * 0.05).to(torch.bfloat16)
    want = x.double() @ w.double().T
    k_boxes = -(-k // 64)
    for parts in sorted({None, 1, min(2, k_boxes), min(3, k_boxes), min(k_boxes, 16)}, key=lambda v: -1 if v is None else v):
        y = ops.linear_stream_partial(x, w, parts)
        assert y.dtype == torch.float32 and y.shape[1:] == (m, n) and (parts is None or y.shape[0] == parts)
        torch.testing.assert_close(y.double().sum(0), want, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(ops.linear_stream(x, w).double(), want, rtol=2e-2, atol=2e-2)
    assert int(ops.stream_error_word(torch.device(DEVICE)).item()) == 0
    with pytest.raises(ops.KernelError, match="more than 64 rows"):
        ops.linear_stream_partial(torch.zeros(65, k, device=DEVICE, dtype=torch.bfloat16), w)
    with pytest.raises(ops.KernelError, match="parts"):
        ops.linear_stream_partial(x, w, k_boxes + 1)


def test_stream_gemm_gives_the_same_bits_every_time():
    """The TMA-fed product, 17 rows against the QKV matrix of the 4B shape (its blocks go round their rings), the same call
    8,000 times: every result bit for bit the first one's, which is the plain product.  Its consumers read a ring stage
    with ordinary loads and TMA, another proxy, writes it next; without a proxy fence between the two the next box's first
    rows landed under a warp's last reads about once in 1,500 calls: one weight row off by a box's worth of its sum."""
    from pylon_b200.kernels import ops

    torch.manual_seed(0)
    w = (torch.randn(6_144, 2_560, device=DEVICE) * 0.02).to(torch.bfloat16)
    x = torch.randn(17, 2_560, device=DEVICE).to(torch.bfloat16)
    first = ops.linear_stream_partial(x, w).clone()
    torch.testing.assert_close(first.sum(0).double(), x.double() @ w.double().T, rtol=1e-4, atol=1e-4)
    differing = 0
    for _ in range(80):
        results = [ops.linear_stream_partial(x, w) for _ in range(100)]
        differing += sum(1 for result in results if not torch.equal(result, first))
    assert differing == 0, f"{differing} of 8,000 calls gave other bits than the first"
    assert int(ops.stream_error_word(torch.device(DEVICE)).item()) == 0


def test_kernel_error_words_are_reported_once():
    """A kernel whose bounded wait ran out sets a word on the device; the engine's check turns
    it into an exception and clears it.  (The word is set from the host here: no kernel is made
    to give up.)"""
    from pylon_b200.kernels import ops

    device = torch.device(DEVICE)
    ops.raise_on_kernel_errors(device)            # nothing pending after the tests before this one
    ops.attention_error_word(device).fill_(3)
    with pytest.raises(ops.KernelError, match="attention \\(a bounded wait ran out, code 3\\)"):
        ops.raise_on_kernel_errors(device)
    ops.raise_on_kernel_errors(device)            # cleared
    assert int(ops.tcgen05_error_word(device).item()) == 0 and int(ops.stream_error_word(device).item()) == 0
    # "cuda" and "cuda:0" name the same words
    ops.attention_error_word(torch.device("cuda", torch.cuda.current_device())).fill_(1)
    assert int(ops.attention_error_word(torch.device("cuda")).item()) == 1
    with pytest.raises(ops.KernelError):
        ops.raise_on_kernel_errors(torch.device("cuda"))


def test_after_a_kernel_error_the_decode_attention_counts_from_zero_again():
    """A block of the decode attention that gives up never takes part in the count of the rows it shared, so their
    counters are left above zero.  The check that reports the error puts them back; the next launch is right.
    (Counters and word are written from the host here: no kernel is made to give up.)"""
    from pylon_b200.kernels import ops

    device = torch.device(DEVICE)
    nq, nkv, d = 8, 2, 64
    cache = Paged([700, 640, 90, 513], [1, 1, 1, 1], nkv, d, 64, torch.bfloat16, seed=4)
    fused = torch.randn(cache.tokens, (nq + 2 * nkv) * d, device=DEVICE).to(torch.bfloat16)
    run = lambda: ops.paged_attention(fused, cache.k_pages, cache.v_pages, cache.positions, cache.token_row, cache.q_start, cache.kv_len,
                                      cache.table, nq, 1, max(cache.kv_lens))
    want = attention_reference(fused[:, : nq * d].reshape(cache.tokens, nq, d), cache, nq, nkv, d, None, 1.0 / math.sqrt(d))
    torch.testing.assert_close(run().double(), want, rtol=2e-2, atol=2e-2)
    ops.raise_on_kernel_errors(device)
    counters = ops._zeroed_counters(device, "attention", len(cache.kv_lens) * nkv)
    assert int(counters.abs().sum().item()) == 0           # a launch that runs to its end leaves them at zero
    counters[: len(cache.kv_lens) * nkv] = 1               # what a block that gave up would leave behind
    ops.attention_error_word(device).fill_(1)
    with pytest.raises(ops.KernelError, match="attention"):
        ops.raise_on_kernel_errors(device)
    assert int(counters.abs().sum().item()) == 0
    torch.testing.assert_close(run().double(), want, rtol=2e-2, atol=2e-2)
    ops.raise_on_kernel_errors(device)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_block_table_that_names_a_page_outside_the_pool_is_reported(dtype):
    """The kernels never follow such an entry (they skip the access), and they say so: the cache write sets its
    error word, the attention sets its own; in both cases the check raises and the memory around the pool is untouched."""
    from pylon_b200.kernels import ops

    device = torch.device(DEVICE)
    ops.raise_on_kernel_errors(device)
    nq, nkv, d, page = 4, 2, 64, 64
    cache = Paged([70, 130], [3, 2], nkv, d, page, dtype, seed=9)
    num_pages = cache.k_pages.shape[0]
    qkv = torch.randn(cache.tokens, (nq + 2 * nkv) * d, device=DEVICE).to(dtype)
    broken = cache.table.clone()
    broken[0, 1] = num_pages + 7          # the page the first row's new tokens would be written to
    k_before, v_before = cache.k_pages.clone(), cache.v_pages.clone()
    ops.qk_norm_rope_kv_write(qkv.clone(), None, None, 0.0, None, None, 0, cache.positions, cache.token_row, broken, page,
                              cache.k_pages, cache.v_pages, nq, nkv, d)
    with pytest.raises(ops.KernelError, match="cache write \\(a block table names a page outside the pool, code 5\\)"):
        ops.raise_on_kernel_errors(device)
    written = (cache.k_pages != k_before).flatten(1).any(1) | (cache.v_pages != v_before).flatten(1).any(1)
    assert written.nonzero().flatten().tolist() == [int(cache.table[1, 2])]   # only the second row's page was written
    if dtype == torch.bfloat16:
        ops.paged_attention(qkv, cache.k_pages, cache.v_pages, cache.positions, cache.token_row, cache.q_start, cache.kv_len, broken, nq, 3, 130)
        with pytest.raises(ops.KernelError, match="attention \\(a block table names a page outside the pool, code 5\\)"):
            ops.raise_on_kernel_errors(device)
    ops.raise_on_kernel_errors(device)


def test_skinny_gemm_refuses():
    from pylon_b200.kernels import ops

    w = torch.zeros(16, 20, device=DEVICE, dtype=torch.bfloat16)
    with pytest.raises(ops.KernelError, match="multiples of 8"):
        ops.linear_skinny(torch.zeros(2, 20, device=DEVICE, dtype=torch.bfloat16), w)
    with pytest.raises(ops.KernelError, match="64 rows"):
        ops.linear_skinny(torch.zeros(65, 24, device=DEVICE, dtype=torch.bfloat16), torch.zeros(16, 24, device=DEVICE, dtype=torch.bfloat16))


# ---------------------------------------------------------------------------------------
# a small paged cache for the kernels below
# ---------------------------------------------------------------------------------------
class Paged:
    """Requests with given context lengths and new-token counts over shuffled pages."""

    def __init__(self, kv_lens, q_lens, nkv, d, page_size, dtype, spare_pages=3, seed=0):
        rng = np.random.default_rng(seed)
        self.kv_lens, self.q_lens, self.page_size = list(kv_lens), list(q_lens), page_size
        pages_needed = [-(-n // page_size) for n in kv_lens]
        num_pages = sum(pages_needed) + spare_pages
        order = rng.permutation(num_pages)
        width = max(pages_needed) + 1
        table = np.full((len(kv_lens), width), -1, dtype=np.int32)
        cursor = 0
        for r, need in enumerate(pages_needed):
            table[r, :need] = order[cursor : cursor + need]
            cursor += need
        self.table = torch.tensor(table, device=DEVICE)
        self.k_pages = torch.randn(num_pages, nkv, page_size, d, device=DEVICE).to(dtype)
        self.v_pages = torch.randn(num_pages, nkv, page_size, d, device=DEVICE).to(dtype)
        positions, token_row, q_start = [], [], [0]
        for r, (kv, q) in enumerate(zip(kv_lens, q_lens)):
            positions += list(range(kv - q, kv))
            token_row += [r] * q
            q_start.append(q_start[-1] + q)
        as_int = lambda values: torch.tensor(values, device=DEVICE, dtype=torch.int32)
        self.positions, self.token_row, self.q_start, self.kv_len = as_int(positions), as_int(token_row), as_int(q_start), as_int(kv_lens)
        self.tokens = q_start[-1]

    def gather(self, pages, r):
        """[kv_len, nkv, d] float64 keys or values of request r."""
        kv = self.kv_lens[r]
        rows = [pages[int(self.table[r, j // self.page_size]), :, j % self.page_size] for j in range(kv)]
        return torch.stack(rows).double()


def attention_reference(q, cache: Paged, nq, nkv, d, window, scale):
    out = torch.zeros(cache.tokens, nq, d, dtype=torch.float64, device=DEVICE)
    group = nq // nkv
    cursor = 0
    for r, (kv, ql) in enumerate(zip(cache.kv_lens, cache.q_lens)):
        k, v = cache.gather(cache.k_pages, r), cache.gather(cache.v_pages, r)
        for i in range(ql):
            position = kv - ql + i
            low = 0 if not window else max(0, position - window + 1)
            for h in range(nq):
                scores = (k[low : position + 1, h // group] @ q[cursor + i, h].double()) * scale
                out[cursor + i, h] = torch.softmax(scores, 0) @ v[low : position + 1, h // group]
        cursor += ql
    return out.reshape(cache.tokens, nq * d)


ATTENTION_CASES = [
    # kv_lens, q_lens, nq, nkv, d, page, window
    ([1, 17, 130], [1, 17, 1], 4, 2, 16, 16, None),
    ([300, 64, 65, 7], [1, 64, 2, 7], 6, 3, 32, 8, None),
    ([200, 90], [70, 1], 8, 2, 64, 64, None),
    ([150, 33], [1, 33], 10, 2, 128, 256, None),        # group of 5
    ([97], [97], 2, 2, 256, 24, None),                    # no grouping, page size no power of two
    ([120, 260], [9, 1], 4, 1, 48, 16, None),             # head size 48, one KV head
    ([180, 75, 300], [40, 1, 1], 4, 2, 32, 16, 50),       # window
    ([90], [90], 3, 1, 80, 32, 17),
    # rows long enough for the 128-row blocks, beside short ones
    ([300, 40, 129], [300, 3, 1], 8, 2, 128, 256, None),
    ([260], [260], 4, 1, 64, 16, 33),
    # decoded tokens only (the decode form of the kernel): contiguous pages, gathered pages, groups, windows
    ([300, 64, 65, 7, 1, 129], [1, 1, 1, 1, 1, 1], 8, 2, 128, 64, None),
    ([500, 70], [1, 1], 10, 2, 64, 128, None),
    ([257, 90, 40], [3, 2, 1], 4, 2, 32, 16, None),
    ([400, 33, 64], [1, 1, 1], 4, 2, 64, 64, 100),
    ([1000], [1], 16, 1, 16, 256, None),                  # a group of 16 fills the tile
    # prompt portions for the tcgen05 kernel: several query tiles, tiles that end inside a page, a group of 5, windows
    ([700, 129, 64], [700, 65, 3], 8, 2, 128, 64, None),
    ([1000, 300], [333, 300], 10, 2, 128, 128, None),
    ([520, 77], [200, 77], 4, 4, 64, 64, 150),
    ([900], [900], 6, 1, 64, 192, 70),
    ([100, 257, 64, 31, 90, 400, 300], [1, 1, 1, 2, 1, 200, 300], 8, 2, 128, 64, None),   # decoded rows first, then two prompt portions
    # more rows than a warp scans at once, lengths from 1 to 451, beside a prompt portion in the middle
    ([1 + (37 * i) % 451 for i in range(20)] + [80] + [5 + (53 * i) % 300 for i in range(19)], [1] * 20 + [30] + [1] * 19, 8, 2, 64, 16, None),
]


@pytest.mark.parametrize("case", ATTENTION_CASES, ids=lambda c: f"d{c[4]}_g{c[2] // c[3]}_p{c[5]}_w{c[6]}")
@pytest.mark.parametrize("mode", ["float32", "bfloat16_simple", "bfloat16_mma", "bfloat16_mma_splits", "bfloat16_mma_blocks1", "bfloat16_mma_blocks5", "bfloat16_tcgen05"])
def test_paged_attention(case, mode):
    from pylon_b200.kernels import ops

    kv_lens, q_lens, nq, nkv, d, page, window = case
    if mode == "bfloat16_tcgen05" and not (d in (64, 128) and page % 64 == 0):
        pytest.skip("the tcgen05 kernel takes head sizes 64 and 128 and pages of a multiple of 64 keys")
    dtype = torch.float32 if mode == "float32" else torch.bfloat16
    cache = Paged(kv_lens, q_lens, nkv, d, page, dtype)
    # q sits inside a wider fused buffer, as in the engine
    fused = torch.randn(cache.tokens, (nq + 2 * nkv) * d, device=DEVICE).to(dtype)
    scale = 1.0 / math.sqrt(d)
    expected = attention_reference(fused[:, : nq * d].reshape(cache.tokens, nq, d), cache, nq, nkv, d, window, scale)
    out = ops.paged_attention(
        fused, cache.k_pages, cache.v_pages, cache.positions, cache.token_row, cache.q_start, cache.kv_len, cache.table, nq,
        max(q_lens), max(kv_lens), window=window, force_simple=mode in ("float32", "bfloat16_simple"),
        num_splits=3 if mode == "bfloat16_mma_splits" else (1 if mode == "bfloat16_mma" else None),
        # decoded rows: all their tiles in one block's run, or in five runs that end inside rows
        decode_blocks=int(mode[len("bfloat16_mma_blocks"):]) if mode.startswith("bfloat16_mma_blocks") else None,
        prefill_kernel="tcgen05" if mode == "bfloat16_tcgen05" else ("mma" if mode.startswith("bfloat16_mma") else None),
        row_tokens=q_lens if mode == "bfloat16_tcgen05" else None,   # the hint by which the tcgen05 kernel launches only its rows
    )
    torch.testing.assert_close(out.double(), expected, **(dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)))
    assert int(ops.attention_error_word(torch.device(DEVICE)).item()) == 0   # no wait for a TMA copy ran out


@pytest.mark.parametrize("d, nq, nkv", [(128, 32, 8), (64, 12, 4)])
def test_tcgen05_attention_gives_the_same_bits_every_time(d, nq, nkv):
    """Eight prompt portions of some 500 tokens: several waves of blocks, each with eight key tiles and more in flight.  A
    softmax thread that reads its output before the last weighted sums are added to it (a wait by parity that took the phase
    before last for the one it asked for) gives a result that depends on timing: the same call, many times, must give the same
    bits, and they must be the plain answer."""
    from pylon_b200.kernels import ops

    lengths = [500, 433, 512, 390, 471, 505, 448, 497]
    cache = Paged(lengths, lengths, nkv, d, 64, torch.bfloat16, seed=4)
    fused = torch.randn(cache.tokens, (nq + 2 * nkv) * d, device=DEVICE).to(torch.bfloat16)
    run = lambda: ops.paged_attention(fused, cache.k_pages, cache.v_pages, cache.positions, cache.token_row, cache.q_start, cache.kv_len, cache.table,
                                      nq, max(lengths), max(lengths), prefill_kernel="tcgen05", row_tokens=lengths)
    first = run().clone()
    for turn in range(30):
        assert torch.equal(run(), first), f"call {turn + 1} differs from the first"
    # One portion that ends inside a page, as a prompt of 411 tokens leaves it, many times over: its last tile's values land
    # late now and then, and an issuer that then mistook the softmax threads' next arrival for the one it waited for never
    # came back (a bounded wait ran out: the error word).
    lone = Paged([411], [411], nkv, d, 256, torch.bfloat16, seed=6)
    lone_q = torch.randn(lone.tokens, (nq + 2 * nkv) * d, device=DEVICE).to(torch.bfloat16)
    run_lone = lambda: ops.paged_attention(lone_q, lone.k_pages, lone.v_pages, lone.positions, lone.token_row, lone.q_start, lone.kv_len, lone.table,
                                           nq, 448, 411, prefill_kernel="tcgen05", row_tokens=[411])
    first_lone = run_lone().clone()
    for turn in range(300):
        out = run_lone()
        if turn % 50 == 49:
            assert torch.equal(out, first_lone), f"call {turn + 1} differs from the first"
            assert int(ops.attention_error_word(torch.device(DEVICE)).item()) == 0, f"a wait ran out by call {turn + 1}"
    # against the plain statement, on the two longest rows (the reference is slow)
    longest = sorted(range(len(lengths)), key=lambda r: -lengths[r])[:2]
    for r in longest:
        begin = int(cache.q_start[r])
        q = fused[begin : begin + lengths[r], : nq * d].reshape(lengths[r], nq, d).double()
        k, v = cache.gather(cache.k_pages, r), cache.gather(cache.v_pages, r)
        group = nq // nkv
        scores = torch.einsum("thd,shd->hts", q, k.repeat_interleave(group, dim=1)) / math.sqrt(d)
        scores = scores.masked_fill(torch.triu(torch.ones(lengths[r], lengths[r], dtype=torch.bool, device=DEVICE), 1), -math.inf)
        want = torch.einsum("hts,shd->thd", torch.softmax(scores, -1), v.repeat_interleave(group, dim=1)).reshape(lengths[r], nq * d)
        torch.testing.assert_close(first[begin : begin + lengths[r]].double(), want, rtol=2e-2, atol=2e-2)
    assert int(ops.attention_error_word(torch.device(DEVICE)).item()) == 0


@pytest.mark.parametrize("rows, nkv, group, d, page, window", [
    (1, 8, 4, 128, 256, None),     # one request: clusters of 16
    (3, 2, 4, 128, 64, None),
    (3, 8, 4, 128, 64, None),      # 24 pairs: clusters of 8
    (5, 8, 2, 64, 64, None),       # 40 pairs: clusters of 6
    (8, 8, 4, 128, 256, None),     # 64 pairs: clusters of 4
    (11, 8, 1, 64, 128, 90),       # 88 pairs: clusters of 3, a window
    (30, 4, 2, 128, 64, None),     # 120 pairs: clusters of 2
    (40, 4, 2, 64, 64, None),      # 160 pairs: too many for clusters, the runs
])
@pytest.mark.parametrize("lengths", ["equal", "ragged", "short"])
def test_decode_attention_in_clusters(rows, nkv, group, d, page, window, lengths):
    """Rows of decoded tokens with the hint that they are about equally long: every (row, KV head)
    pair gets a cluster of blocks that combine through distributed shared memory.  The result
    must be right whatever the lengths are: equal, very different (the hint was wrong), and
    shorter than a cluster has blocks (blocks without tiles), with rows of two tokens among them."""
    from pylon_b200.kernels import ops

    nq = nkv * group
    if lengths == "equal":
        kv_lens = [700 + (i % 3) for i in range(rows)]
    elif lengths == "ragged":
        kv_lens = [1 + (211 * i) % 900 for i in range(rows)]
    else:
        kv_lens = [1 + (37 * i) % 130 for i in range(rows)]
    q_lens = [2 if (i % 4 == 1 and kv_lens[i] >= 2 and 2 * group <= 16) else 1 for i in range(rows)]
    cache = Paged(kv_lens, q_lens, nkv, d, page, torch.bfloat16, seed=rows)
    fused = torch.randn(cache.tokens, (nq + 2 * nkv) * d, device=DEVICE).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    expected = attention_reference(fused[:, : nq * d].reshape(cache.tokens, nq, d), cache, nq, nkv, d, window, scale)
    for alike in (True, False):
        out = ops.paged_attention(fused, cache.k_pages, cache.v_pages, cache.positions, cache.token_row, cache.q_start, cache.kv_len, cache.table,
                                  nq, max(q_lens), max(kv_lens), window=window, rows_alike=alike)
        torch.testing.assert_close(out.double(), expected, rtol=2e-2, atol=2e-2)
    assert int(ops.attention_error_word(torch.device(DEVICE)).item()) == 0


@pytest.mark.parametrize("rows, nkv, group, d, page, lengths", [
    (64, 8, 4, 128, 256, "equal"),      # 512 pairs of 6 tiles over 444 blocks: nearly every block shares a pair with its neighbour
    (64, 8, 4, 128, 256, "ragged"),
    (70, 8, 2, 64, 64, "equal"),
    (48, 4, 4, 64, 16, "ragged"),       # pages of 16 keys: the gathering form
    (64, 8, 4, 128, 256, "one_long"),   # one long row among short ones
    (200, 2, 4, 128, 64, "equal"),
])
def test_decode_attention_of_many_short_rows(rows, nkv, group, d, page, lengths):
    """More (row, KV head) pairs than blocks, each a few tiles long (the decode steps of many requests with short
    contexts): runs of a few tiles that nearly all end inside a pair, so that nearly every pair is combined from two
    blocks' partial results; twice in a row, since a call must leave the counters as it found them."""
    from pylon_b200.kernels import ops

    nq = nkv * group
    if lengths == "equal":
        kv_lens = [384 - (i % 2) for i in range(rows)]
    elif lengths == "ragged":
        kv_lens = [1 + (97 * i) % 500 for i in range(rows)]
    else:
        kv_lens = [5_000] + [100 + (53 * i) % 300 for i in range(rows - 1)]
    q_lens = [2 if (i % 5 == 2 and kv_lens[i] >= 2 and 2 * group <= 16) else 1 for i in range(rows)]
    cache = Paged(kv_lens, q_lens, nkv, d, page, torch.bfloat16, seed=rows)
    fused = torch.randn(cache.tokens, (nq + 2 * nkv) * d, device=DEVICE).to(torch.bfloat16)
    expected = attention_reference(fused[:, : nq * d].reshape(cache.tokens, nq, d), cache, nq, nkv, d, None, 1.0 / math.sqrt(d))
    for repeat in range(2):   # the second call finds the counters as the first left them
        out = ops.paged_attention(fused, cache.k_pages, cache.v_pages, cache.positions, cache.token_row, cache.q_start, cache.kv_len, cache.table,
                                  nq, max(q_lens), max(kv_lens))
        torch.testing.assert_close(out.double(), expected, rtol=2e-2, atol=2e-2)
    ops.raise_on_kernel_errors(torch.device(DEVICE))
    assert int(ops._zeroed_counters(torch.device(DEVICE), "attention", rows * nkv).abs().sum().item()) == 0


@pytest.mark.parametrize("mode", ["float32", "bfloat16_mma", "bfloat16_mma_splits"])
def test_attention_finds_one_far_key_among_hundreds(mode):
    """Random keys would hide a wrong page: here one key far back dominates the softmax,
    so the output must be that key's value."""
    from pylon_b200.kernels import ops

    dtype = torch.float32 if mode == "float32" else torch.bfloat16
    nq, nkv, d, page = 4, 2, 64, 16
    cache = Paged([700, 450], [1, 3], nkv, d, page, dtype, seed=5)
    fused = (torch.randn(cache.tokens, (nq + 2 * nkv) * d, device=DEVICE) * 0.1).to(dtype)
    targets = {0: 37, 1: 213}          # row -> position of the dominant key
    cursor = 0
    for r, ql in enumerate(cache.q_lens):
        j = targets[r]
        for kv_head in range(nkv):
            direction = torch.randn(d, device=DEVICE)
            direction = direction / direction.norm()
            cache.k_pages[int(cache.table[r, j // page]), kv_head, j % page] = (direction * 40).to(dtype)
            for i in range(ql):
                for h in range(kv_head * 2, kv_head * 2 + 2):
                    fused[cursor + i, h * d : (h + 1) * d] = (direction * 8).to(dtype)
        cursor += ql
    out = ops.paged_attention(
        fused, cache.k_pages, cache.v_pages, cache.positions, cache.token_row, cache.q_start, cache.kv_len, cache.table, nq,
        max(cache.q_lens), max(cache.kv_lens), force_simple=mode == "float32", num_splits=4 if mode.endswith("splits") else None,
    ).reshape(cache.tokens, nq, d)
    cursor = 0
    for r, ql in enumerate(cache.q_lens):
        j = targets[r]
        for i in range(ql):
            for h in range(nq):
                want = cache.v_pages[int(cache.table[r, j // page]), h // 2, j % page].float()
                torch.testing.assert_close(out[cursor + i, h].float(), want, rtol=2e-2, atol=2e-2)
        cursor += ql


@pytest.mark.parametrize("mode", ["float32", "bfloat16_mma", "bfloat16_mma_splits"])
@pytest.mark.parametrize("q_len", [1, 40])
def test_attention_window_edge(mode, q_len):
    """The key just outside the window is made overwhelming: if the mask were off by one, it
    would take all the weight.  The key just inside must win instead."""
    from pylon_b200.kernels import ops

    dtype = torch.float32 if mode == "float32" else torch.bfloat16
    nq, nkv, d, page, window, kv = 2, 1, 64, 16, 37, 300
    cache = Paged([kv], [q_len], nkv, d, page, dtype, seed=8)
    direction = torch.randn(d, device=DEVICE)
    direction = direction / direction.norm()
    fused = (torch.randn(q_len, (nq + 2) * d, device=DEVICE) * 0.05).to(dtype)
    fused[:, : nq * d] = (direction * 6).to(dtype).repeat(nq)
    last = kv - 1                               # the last token's position; its window is (last - 37, last]
    outside, inside = last - window, last - window + 1

    def set_key(position, scale):
        cache.k_pages[int(cache.table[0, position // page]), 0, position % page] = (direction * scale).to(dtype)

    set_key(outside, 60.0)
    set_key(inside, 30.0)
    out = ops.paged_attention(
        fused, cache.k_pages, cache.v_pages, cache.positions, cache.token_row, cache.q_start, cache.kv_len, cache.table, nq,
        q_len, kv, window=window, force_simple=mode == "float32", num_splits=3 if mode.endswith("splits") else None,
    ).reshape(q_len, nq, d)
    want = cache.v_pages[int(cache.table[0, inside // page]), 0, inside % page].float()
    torch.testing.assert_close(out[-1, 0].float(), want, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out[-1, 1].float(), want, rtol=2e-2, atol=2e-2)
    if q_len > 1:   # the token before still has the big key inside its window
        big = cache.v_pages[int(cache.table[0, outside // page]), 0, outside % page].float()
        torch.testing.assert_close(out[-2, 0].float(), big, rtol=2e-2, atol=2e-2)


def test_attention_refuses_what_it_cannot_do():
    from pylon_b200.kernels import ops

    cache = Paged([5], [5], 2, 16, 8, torch.bfloat16)
    fused = torch.randn(5, 6 * 16, device=DEVICE).to(torch.bfloat16)
    with pytest.raises(ops.KernelError, match="query heads"):
        ops.paged_attention(fused, cache.k_pages, cache.v_pages, cache.positions, cache.token_row, cache.q_start, cache.kv_len, cache.table, 3, 5, 5)
    with pytest.raises(ops.KernelError, match="CUDA"):
        ops.swiglu(torch.zeros(2, 4))


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq, nkv, d, rotary, page, norm", [
    (4, 2, 16, 16, 16, True), (6, 3, 32, 32, 8, True), (32, 8, 128, 128, 256, True), (5, 5, 64, 32, 4, True),
    (2, 1, 80, 80, 24, False), (3, 1, 256, 64, 16, True),
    (4, 2, 64, 64, 16, True), (2, 2, 256, 256, 8, True), (8, 4, 128, 128, 64, False), (7, 1, 128, 128, 16, True),    # the vector forms
])
@pytest.mark.parametrize("kv_lens, q_lens", [([40, 9, 70], [13, 9, 1]), ([100, 9, 70], [77, 9, 1])])   # few tokens, many
def test_qk_norm_rope_kv_write(dtype, nq, nkv, d, rotary, page, norm, kv_lens, q_lens):
    from pylon_b200.kernels import ops

    eps = 1e-5
    cache = Paged(kv_lens, q_lens, nkv, d, page, dtype, seed=2)
    k_before, v_before = cache.k_pages.clone(), cache.v_pages.clone()
    qkv = torch.randn(cache.tokens, (nq + 2 * nkv) * d, device=DEVICE).to(dtype)
    original = qkv.clone()
    qw = torch.rand(d, device=DEVICE) + 0.5 if norm else None
    kw = torch.rand(d, device=DEVICE) + 0.5 if norm else None
    max_pos = 128
    inv_freq = 1.0 / (10_000.0 ** (torch.arange(0, rotary, 2, dtype=torch.float32) / rotary))
    angles = torch.arange(max_pos, dtype=torch.float32).unsqueeze(1) * inv_freq.unsqueeze(0)
    cos, sin = torch.cos(angles).to(DEVICE), torch.sin(angles).to(DEVICE)
    ops.qk_norm_rope_kv_write(qkv, qw, kw, eps, cos, sin, rotary, cache.positions, cache.token_row, cache.table, page,
                              cache.k_pages, cache.v_pages, nq, nkv, d)

    def reference(x, weight, positions):          # x: [T, heads, d] float64
        if weight is not None:
            x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight.double()
        c, s = cos[positions.long()].double().unsqueeze(1), sin[positions.long()].double().unsqueeze(1)
        half = rotary // 2
        first, second, rest = x[..., :half], x[..., half:rotary], x[..., rotary:]
        return torch.cat((first * c - second * s, second * c + first * s, rest), dim=-1)

    heads = original.double().reshape(cache.tokens, nq + 2 * nkv, d)
    want_q = reference(heads[:, :nq], qw, cache.positions)
    want_k = reference(heads[:, nq : nq + nkv], kw, cache.positions)
    want_v = heads[:, nq + nkv :]
    tol = tolerance(dtype)
    torch.testing.assert_close(qkv.double().reshape(cache.tokens, -1, d)[:, :nq], want_q, **tol)
    written = torch.zeros_like(cache.k_pages, dtype=torch.bool)
    for t in range(cache.tokens):
        r, pos = int(cache.token_row[t]), int(cache.positions[t])
        p, slot = int(cache.table[r, pos // page]), pos % page
        torch.testing.assert_close(cache.k_pages[p, :, slot].double(), want_k[t], **tol)
        torch.testing.assert_close(cache.v_pages[p, :, slot].double(), want_v[t], rtol=0, atol=0)
        written[p, :, slot] = True
    # nothing else in the cache was touched
    assert torch.equal(cache.k_pages[~written], k_before[~written]) and torch.equal(cache.v_pages[~written], v_before[~written])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq, nkv, d, tokens", [(4, 2, 16, 5), (5, 1, 80, 33), (32, 8, 128, 70), (3, 3, 272, 9)])
def test_qk_norm_alone(dtype, nq, nkv, d, tokens):
    """RMSNorm of the q and k heads in place; v and, with a missing weight, that kind of head stay as they are."""
    from pylon_b200.kernels import ops

    eps = 1e-5
    torch.manual_seed(tokens)
    original = torch.randn(tokens, (nq + 2 * nkv) * d, device=DEVICE).to(dtype)
    qw, kw = torch.rand(d, device=DEVICE) + 0.5, torch.rand(d, device=DEVICE) + 0.5
    heads = original.double().reshape(tokens, -1, d)
    norm = lambda x, weight: x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight.double()
    for q_weight, k_weight in ((qw, kw), (None, kw)):
        qkv = ops.qk_norm(original.clone(), q_weight, k_weight, eps, nq, nkv, d).double().reshape(tokens, -1, d)
        want_q = norm(heads[:, :nq], q_weight) if q_weight is not None else heads[:, :nq]
        torch.testing.assert_close(qkv[:, :nq], want_q, **(tolerance(dtype) if q_weight is not None else dict(rtol=0, atol=0)))
        torch.testing.assert_close(qkv[:, nq : nq + nkv], norm(heads[:, nq : nq + nkv], k_weight), **tolerance(dtype))
        torch.testing.assert_close(qkv[:, nq + nkv :], heads[:, nq + nkv :], rtol=0, atol=0)


@pytest.mark.parametrize("tokens_each", [(1, 1, 1), (13, 9, 70)])
@pytest.mark.parametrize("nq, nkv, d, norm, parts", [(8, 2, 128, True, 4), (6, 3, 64, True, 3), (4, 1, 256, False, 1)])
def test_qk_norm_rope_kv_write_from_partial_sums(tokens_each, nq, nkv, d, norm, parts):
    """The fused QKV product may arrive as float32 partial sums over slices of k: the kernel adds
    them up, q goes to a tensor of its own, k and v into the pages."""
    from pylon_b200.kernels import ops

    eps, page = 1e-6, 16
    cache = Paged([tokens + 30 for tokens in tokens_each], list(tokens_each), nkv, d, page, torch.bfloat16, seed=4)
    width = (nq + 2 * nkv) * d
    pieces = torch.randn(parts, cache.tokens, width, device=DEVICE)
    total = pieces.double().sum(0).reshape(cache.tokens, nq + 2 * nkv, d)
    qw = torch.rand(d, device=DEVICE) + 0.5 if norm else None
    kw = torch.rand(d, device=DEVICE) + 0.5 if norm else None
    inv_freq = 1.0 / (10_000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    angles = torch.arange(256, dtype=torch.float32).unsqueeze(1) * inv_freq.unsqueeze(0)
    cos, sin = torch.cos(angles).to(DEVICE), torch.sin(angles).to(DEVICE)
    q = ops.qk_norm_rope_kv_write(pieces, qw, kw, eps, cos, sin, d, cache.positions, cache.token_row, cache.table, page,
                                  cache.k_pages, cache.v_pages, nq, nkv, d)
    assert q.shape == (cache.tokens, nq * d) and q.dtype == torch.bfloat16

    def reference(x, weight):
        if weight is not None:
            x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight.double()
        c, s2 = cos[cache.positions.long()].double().unsqueeze(1), sin[cache.positions.long()].double().unsqueeze(1)
        first, second = x[..., : d // 2], x[..., d // 2 :]
        return torch.cat((first * c - second * s2, second * c + first * s2), dim=-1)

    tol = tolerance(torch.bfloat16)
    torch.testing.assert_close(q.double().reshape(cache.tokens, nq, d), reference(total[:, :nq], qw), **tol)
    want_k, want_v = reference(total[:, nq : nq + nkv], kw), total[:, nq + nkv :]
    for t in range(cache.tokens):
        r, pos = int(cache.token_row[t]), int(cache.positions[t])
        p, slot = int(cache.table[r, pos // page]), pos % page
        torch.testing.assert_close(cache.k_pages[p, :, slot].double(), want_k[t], **tol)
        torch.testing.assert_close(cache.v_pages[p, :, slot].double(), want_v[t], **tol)
    with pytest.raises(ops.KernelError, match="partial sums"):
        ops.qk_norm_rope_kv_write(torch.zeros(2, cache.tokens, (nq + 2 * nkv) * 48, device=DEVICE), None, None, eps, None, None, 0, cache.positions,
                                  cache.token_row, cache.table, page, torch.zeros(4, nkv, page, 48, device=DEVICE, dtype=torch.bfloat16),
                                  torch.zeros(4, nkv, page, 48, device=DEVICE, dtype=torch.bfloat16), nq, nkv, 48)


@pytest.mark.parametrize("tokens_each, nq, nkv, d, k, norm, page", [
    ((300, 1, 150), 8, 2, 128, 256, True, 16),      # two whole row tiles and a partly empty one; a row of one token between
    ((1, 130), 6, 3, 64, 200, True, 64),            # heads of 64: four to a tile of 256; k with a remainder
    ((257,), 5, 1, 128, 64, False, 256),            # 7 heads: the last tile is half outside the matrix; no norms; one step of k
    ((64, 64, 64, 64), 4, 4, 64, 72, True, 8),      # rows that end on tile edges
])
def test_qkv_product_with_rotation_in_its_epilogue(tokens_each, nq, nkv, d, k, norm, page):
    """x @ w.T on the tcgen05 kernel with the q/k norms, the rotation and the cache write in its epilogue, against the
    same in float64: q in a tensor of its own, k and v at each token's slot, nothing else in the cache touched, and the
    same bits at the second call; a padding token (row -1) writes nothing, a page that is not there is reported."""
    from pylon_b200.kernels import ops

    eps = 1e-6
    cache = Paged([tokens + 37 for tokens in tokens_each], list(tokens_each), nkv, d, page, torch.bfloat16, seed=11)
    width = (nq + 2 * nkv) * d
    torch.manual_seed(k)
    x = torch.randn(cache.tokens, k, device=DEVICE).to(torch.bfloat16)
    w = (torch.randn(width, k, device=DEVICE) / math.sqrt(k)).to(torch.bfloat16)
    total = (x.double() @ w.double().T).reshape(cache.tokens, nq + 2 * nkv, d)
    qw = torch.rand(d, device=DEVICE) + 0.5 if norm else None
    kw = torch.rand(d, device=DEVICE) + 0.5 if norm else None
    inv_freq = 1.0 / (10_000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    angles = torch.arange(512, dtype=torch.float32).unsqueeze(1) * inv_freq.unsqueeze(0)
    cos, sin = torch.cos(angles).to(DEVICE), torch.sin(angles).to(DEVICE)
    k_before, v_before = cache.k_pages.clone(), cache.v_pages.clone()
    call = lambda: ops.linear_qkv_rotated(x, w, qw, kw, eps, cos, sin, cache.positions, cache.token_row, cache.table, page, cache.k_pages,
                                          cache.v_pages, nq, nkv, d)
    q = call()
    assert q.shape == (cache.tokens, nq * d) and q.dtype == torch.bfloat16

    def reference(heads, weight):
        if weight is not None:
            heads = heads / torch.sqrt((heads * heads).mean(-1, keepdim=True) + eps) * weight.double()
        c, s2 = cos[cache.positions.long()].double().unsqueeze(1), sin[cache.positions.long()].double().unsqueeze(1)
        first, second = heads[..., : d // 2], heads[..., d // 2 :]
        return torch.cat((first * c - second * s2, second * c + first * s2), dim=-1)

    tol = tolerance(torch.bfloat16)
    torch.testing.assert_close(q.double().reshape(cache.tokens, nq, d), reference(total[:, :nq], qw), **tol)
    want_k, want_v = reference(total[:, nq : nq + nkv], kw), total[:, nq + nkv :]
    written = torch.zeros_like(cache.k_pages, dtype=torch.bool)
    for t in range(cache.tokens):
        r, pos = int(cache.token_row[t]), int(cache.positions[t])
        p, slot = int(cache.table[r, pos // page]), pos % page
        torch.testing.assert_close(cache.k_pages[p, :, slot].double(), want_k[t], **tol)
        torch.testing.assert_close(cache.v_pages[p, :, slot].double(), want_v[t], **tol)
        written[p, :, slot] = True
    assert torch.equal(cache.k_pages[~written], k_before[~written]) and torch.equal(cache.v_pages[~written], v_before[~written])
    first_k, first_v = cache.k_pages.clone(), cache.v_pages.clone()
    for _ in range(20):
        assert torch.equal(call(), q) and torch.equal(cache.k_pages, first_k) and torch.equal(cache.v_pages, first_v)
    assert int(ops.tcgen05_error_word(torch.device(DEVICE)).item()) == 0
    # a padding token, and a table that names a page outside the pool
    cache.k_pages.copy_(k_before); cache.v_pages.copy_(v_before)
    rows = cache.token_row.clone()
    rows[cache.tokens - 1] = -1
    ops.linear_qkv_rotated(x, w, qw, kw, eps, cos, sin, cache.positions, rows, cache.table, page, cache.k_pages, cache.v_pages, nq, nkv, d)
    r, pos = int(cache.token_row[-1]), int(cache.positions[cache.tokens - 1])
    p, slot = int(cache.table[r, pos // page]), pos % page
    assert torch.equal(cache.k_pages[p, :, slot], k_before[p, :, slot]) and torch.equal(cache.v_pages[p, :, slot], v_before[p, :, slot])
    ops.raise_on_kernel_errors(torch.device(DEVICE))
    table = cache.table.clone()
    table[0, (cache.kv_lens[0] - 1) // page] = cache.k_pages.shape[0] + 5   # the page of the first row's last token
    ops.linear_qkv_rotated(x, w, qw, kw, eps, cos, sin, cache.positions, cache.token_row, table, page, cache.k_pages, cache.v_pages, nq, nkv, d)
    with pytest.raises(ops.KernelError, match="page"):
        ops.raise_on_kernel_errors(torch.device(DEVICE))


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("vocab", [320, 151_936, 1000, 4099])
def test_sample_argmax(vocab):
    from pylon_b200.kernels import ops

    logits = torch.randn(5, vocab, device=DEVICE)
    logits[2, vocab - 1] = 50.0
    logits[3, 7] = logits[3, 3] = 60.0          # a tie: the lower index wins
    out = ops.sample(logits)
    expected = logits.argmax(-1)
    expected[3] = 3
    assert out.tolist() == expected.tolist()


@pytest.mark.parametrize("vocab, temperature, top_p", [(320, 0.8, 1.0), (151_936, 0.7, 0.9), (1000, 1.5, 0.5), (50, 0.3, 0.95),
                                                       (4099, 0.9, 0.8), (40_003, 1.2, 0.97), (4096, 0.5, 1.0)])
def test_sample_temperature_and_top_p(vocab, temperature, top_p):
    """The kernel's token is the one the plain definition picks for the same uniform number,
    up to float32 rounding of the cumulative sums at a boundary."""
    import plain_qwen3 as plain
    from pylon_b200.kernels import ops

    rows = 64
    logits = torch.randn(rows, vocab, device=DEVICE) * 2
    uniform = torch.rand(rows, device=DEVICE)
    uniform[0], uniform[1] = 0.0, 0.99999
    out = ops.sample(logits, torch.full((rows,), temperature, device=DEVICE), torch.full((rows,), top_p, device=DEVICE), uniform).tolist()
    for r in range(rows):
        probs = plain.sampling_distribution(logits[r].cpu(), temperature, top_p)
        cdf = torch.cumsum(probs, 0)
        token = out[r]
        assert probs[token] > 0, f"row {r}: token {token} is outside the nucleus"
        low = float(cdf[token] - probs[token])
        high = float(cdf[token])
        u = float(uniform[r])
        assert low - 1e-4 <= u <= high + 1e-4, (r, token, low, u, high)


@pytest.mark.parametrize("vocab", [4099, 151_936, 777])
def test_sample_rows_of_every_kind_in_one_call(vocab):
    """Greedy rows, drawn rows, a nucleus so small that one token is left, a row of a wider matrix (a stride that is not the
    vocabulary) and a row without a finite value, in one call; twice, with the same tokens."""
    import plain_qwen3 as plain
    from pylon_b200.kernels import ops

    torch.manual_seed(vocab)
    wide = torch.randn(6, vocab + 37, device=DEVICE) * 3
    logits = wide[:, 5:5 + vocab]
    logits[4, vocab - 2] = 40.0                                                 # the last block's share holds the winner
    logits[5] = float("nan")
    temperature = torch.tensor([0.0, 1.0, 0.7, 1.3, 1.0, 1.0], device=DEVICE)
    top_p = torch.tensor([1.0, 1.0, 0.6, 1e-6, 0.9, 0.9], device=DEVICE)
    uniform = torch.tensor([0.3, 0.999, 0.5, 0.7, 0.2, 0.4], device=DEVICE)
    out = ops.sample(logits, temperature, top_p, uniform).tolist()
    assert out[0] == int(logits[0].argmax())
    assert out[3] == int(logits[3].argmax())                                    # the nucleus keeps the top token alone
    assert out[4] == vocab - 2
    assert 0 <= out[5] < vocab
    for r in (1, 2):
        probs = plain.sampling_distribution(logits[r].cpu(), float(temperature[r]), float(top_p[r]))
        cdf = torch.cumsum(probs, 0)
        assert probs[out[r]] > 0
        assert float(cdf[out[r]] - probs[out[r]]) - 1e-4 <= float(uniform[r]) <= float(cdf[out[r]]) + 1e-4
    for _ in range(50):
        assert ops.sample(logits, temperature, top_p, uniform).tolist() == out


@pytest.mark.parametrize("vocab", [777, 151_936])
def test_sample_reads_and_writes_pinned_host_memory(vocab):
    """The rows' options may lie in pinned host memory, and the kernel leaves the tokens and the kernels' four error words
    in a pinned buffer of the caller: the same tokens as with everything on the device, nothing to copy afterwards."""
    from pylon_b200.kernels import ops

    device = torch.device(DEVICE)
    ops.raise_on_kernel_errors(device)
    rows = 9
    torch.manual_seed(vocab)
    logits = torch.randn(rows, vocab, device=DEVICE) * 2
    options = torch.empty((3, rows), dtype=torch.float32, pin_memory=True)
    options[0] = torch.tensor([0.0, 0.7, 1.0, 0.2, 1.5, 0.0, 0.9, 1.0, 0.4])
    options[1] = torch.tensor([1.0, 0.9, 1.0, 0.95, 0.5, 1.0, 0.3, 1.0, 0.8])
    options[2] = torch.rand(rows)
    on_device = options.to(DEVICE)
    want = ops.sample(logits, on_device[0], on_device[1], on_device[2]).tolist()
    host_copy = torch.full((rows + 4,), -7, dtype=torch.int32, pin_memory=True)
    got = ops.sample(logits, options[0], options[1], options[2], host_copy=host_copy)
    torch.cuda.synchronize()
    assert got.tolist() == want and host_copy[:rows].tolist() == want and host_copy[rows:].tolist() == [0, 0, 0, 0]
    greedy_copy = torch.full((rows + 4,), -7, dtype=torch.int32, pin_memory=True)
    greedy = ops.sample(logits, host_copy=greedy_copy)
    torch.cuda.synchronize()
    assert greedy_copy[:rows].tolist() == greedy.tolist() == logits.argmax(-1).tolist()
    # the words as they stand when the kernel runs (written from the host here: no kernel is made to give up)
    ops.stream_error_word(device).fill_(3)
    ops.sample(logits, host_copy=host_copy)
    torch.cuda.synchronize()
    assert host_copy[rows:].tolist() == [0, 0, 3, 0]
    with pytest.raises(ops.KernelError, match="TMA-fed decode product"):
        ops.raise_on_kernel_errors(device, words=host_copy[rows:])
    ops.raise_on_kernel_errors(device)
    with pytest.raises(ops.KernelError, match="pinned"):
        ops.sample(logits, host_copy=torch.zeros(rows + 4, dtype=torch.int32))


def test_sample_mixed_rows_and_distribution():
    from pylon_b200.kernels import ops

    logits = torch.tensor([[0.0, 1.0, 2.0, 0.5]] * 3, device=DEVICE)
    temperature = torch.tensor([0.0, 1.0, 1.0], device=DEVICE)
    top_p = torch.tensor([1.0, 1.0, 0.5], device=DEVICE)
    counts = torch.zeros(3, 4)
    trials = 2000
    big = logits.repeat(trials, 1)
    out = ops.sample(big, temperature.repeat(trials), top_p.repeat(trials), torch.rand(3 * trials, device=DEVICE)).cpu().reshape(trials, 3)
    for r in range(3):
        counts[r] = torch.bincount(out[:, r].long(), minlength=4).float() / trials
    assert counts[0].tolist() == [0, 0, 1, 0]                                   # temperature 0: arg-max
    torch.testing.assert_close(counts[1], torch.softmax(logits[0].cpu(), 0), atol=0.04, rtol=0)
    assert counts[2].tolist() == [0, 0, 1, 0]                                   # nucleus 0.5 keeps only the top token (p = 0.57)
