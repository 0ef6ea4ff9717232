"""Every hot kernel run many times on two sets of inputs in turn, each result checked against a plain statement.

A kernel that reads something before this launch has produced it (a staging buffer, an accumulator, a partial result in
scratch memory) can pass every single-call test: run twice on the same inputs, what the earlier launch left behind *is*
the right answer.  With two inputs taking turns it never is.  (The tcgen05 product's epilogue had such a fault: a store
loop that let a buffer be overwritten while the store before was still reading it.)"""
from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEVICE = "cuda"
TURNS = 16


def turns(sets, run, tolerance, what):
    for turn in range(TURNS):
        *inputs, want = sets[turn % 2]
        got = run(*inputs)
        wrong = (got.double() - want.double()).abs() > tolerance
        assert not bool(wrong.any()), f"{what}, turn {turn}: {int(wrong.sum())} values off"


@pytest.mark.parametrize("m, n, k", [(1, 2560, 4096), (8, 6144, 2560), (8, 2560, 9728), (32, 2560, 4096), (64, 2560, 4096)])
def test_decode_products_on_alternating_inputs(m, n, k):
    from pylon_b200.kernels import ops

    torch.manual_seed(m + n)
    sets = []
    for _ in range(2):
        x, w = torch.randn(m, k, device=DEVICE).to(torch.bfloat16), (torch.randn(n, k, device=DEVICE) * 0.05).to(torch.bfloat16)
        sets.append((x, w, x.float() @ w.float().T))
    tolerance = 0.3
    turns(sets, lambda x, w: ops.linear_stream(x, w), tolerance, "TMA-fed product")
    turns(sets, lambda x, w: ops.linear_stream_partial(x, w, 4).sum(0), tolerance, "TMA-fed product, partial sums")
    turns(sets, lambda x, w: ops.linear_skinny(x, w, torch.float32), tolerance, "skinny product")
    turns(sets, lambda x, w: ops.linear(x, w), tolerance, "linear")
    folded = lambda y: y.sum(0) if y.dim() == 3 else y
    turns(sets, lambda x, w: folded(ops.linear_for_residual(x, w)), tolerance, "product for the residual stream")
    ops.raise_on_kernel_errors(torch.device(DEVICE))


@pytest.mark.parametrize("m", [8, 32, 300, 2100])
def test_gate_up_products_on_alternating_inputs(m):
    from pylon_b200.kernels import ops

    torch.manual_seed(m)
    inter, k = 9_728, 2_560
    sets = []
    for _ in range(2):
        gate, up = ((torch.randn(inter, k, device=DEVICE) * 0.05).to(torch.bfloat16) for _ in range(2))
        x = torch.randn(m, k, device=DEVICE).to(torch.bfloat16)
        g, u = x.float() @ gate.float().T, x.float() @ up.float().T
        sets.append((x, ops.interleave_gate_up(gate, up), g * torch.sigmoid(g) * u))
    turns(sets, lambda x, w: ops.linear_swiglu(x, w), 0.3, "gate/up with SwiGLU")
    ops.raise_on_kernel_errors(torch.device(DEVICE))


@pytest.mark.parametrize("m, n, k", [(2100, 6144, 2560), (1100, 6144, 2560), (4000, 6144, 320), (2048, 2560, 4096)])
def test_tcgen05_products_on_alternating_inputs(m, n, k):
    from pylon_b200.kernels import ops

    torch.manual_seed(m + k)
    sets = []
    for _ in range(2):
        x, w = torch.randn(m, k, device=DEVICE).to(torch.bfloat16), (torch.randn(n, k, device=DEVICE) * 0.05).to(torch.bfloat16)
        sets.append((x, w, x.float() @ w.float().T))
    turns(sets, lambda x, w: ops.linear_tcgen05(x, w), 0.3, "tcgen05 product")
    ops.raise_on_kernel_errors(torch.device(DEVICE))


@pytest.mark.parametrize("label, kv_lens, q_lens, page", [
    ("eight decoding rows", [700, 900, 650, 1000, 30, 2000, 129, 64], [1] * 8, 256),
    ("one decoding row", [3000], [1], 256),
    ("forty short rows", [100 + 7 * i for i in range(40)], [1] * 40, 64),
    ("portions beside decoded rows", [600, 300, 900, 64], [1, 300, 1, 2], 64),
    ("portions", [700, 500], [700, 200], 256),
])
def test_attention_on_alternating_inputs(label, kv_lens, q_lens, page):
    from pylon_b200.kernels import ops
    from test_kernels_gpu import Paged, attention_reference

    nq, nkv, d = 8, 2, 128
    sets = []
    for seed in range(2):
        cache = Paged(kv_lens, q_lens, nkv, d, page, torch.bfloat16, seed=10 + seed)
        q = torch.randn(cache.tokens, (nq + 2 * nkv) * d, device=DEVICE).to(torch.bfloat16)
        want = attention_reference(q[:, : nq * d].reshape(cache.tokens, nq, d), cache, nq, nkv, d, None, 1 / math.sqrt(d))
        sets.append((cache, q, want))
    for alike in (False, True):
        run = lambda cache, q: ops.paged_attention(q, cache.k_pages, cache.v_pages, cache.positions, cache.token_row, cache.q_start, cache.kv_len,
                                                   cache.table, nq, max(q_lens), max(kv_lens), rows_alike=alike)
        turns(sets, run, 0.03, f"attention, {label}, rows alike {alike}")
    ops.raise_on_kernel_errors(torch.device(DEVICE))


@pytest.mark.parametrize("tokens, width", [(8, 2560), (300, 2560), (2048, 5120)])
def test_norm_over_partial_sums_on_alternating_inputs(tokens, width):
    from pylon_b200.kernels import ops

    torch.manual_seed(tokens)
    sets = []
    for _ in range(2):
        residual, parts, weight = torch.randn(tokens, width, device=DEVICE), torch.randn(4, tokens, width, device=DEVICE), torch.rand(width, device=DEVICE) + 0.5
        total = residual.double() + parts.double().sum(0)
        sets.append((residual, parts, weight, total / torch.sqrt((total**2).mean(-1, keepdim=True) + 1e-6) * weight.double()))
    turns(sets, lambda residual, parts, weight: ops.add_rmsnorm(residual.clone(), parts, weight, 1e-6, torch.bfloat16), 0.05, "add + RMSNorm over partial sums")
