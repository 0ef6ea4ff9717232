"""Each part of a layer alone on the GPU against the plain implementation's function for it,
and models put together in the test from registered parts — among them a toy mixer with a
state of its own and a windowed attention — stepped through the engine without any change
to the framework's files."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from typing import Mapping, Optional, Sequence

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import trace_tools

pytestmark = pytest.mark.gpu

DEVICE = "cuda"


def step_view(q_lens: Sequence[int], starts: Sequence[int], dtype):
    """A StepView for rows that bring ``q_lens`` tokens at positions ``starts``."""
    from pylon_b200.parts.base import StepView

    positions, token_row, q_start = [], [], [0]
    for r, (n, s) in enumerate(zip(q_lens, starts)):
        positions += list(range(s, s + n))
        token_row += [r] * n
        q_start.append(q_start[-1] + n)
    as_int = lambda v: torch.tensor(v, device=DEVICE, dtype=torch.int32)
    step = StepView()
    step.positions, step.token_row, step.q_start = as_int(positions), as_int(token_row), as_int(q_start)
    step.kv_len = as_int([s + n for n, s in zip(q_lens, starts)])
    step.slots = as_int(list(range(len(q_lens))))
    step.token_ids = as_int([0] * q_start[-1])
    step.logit_rows = as_int([])
    step.num_tokens, step.num_rows, step.num_logits = q_start[-1], len(q_lens), 0
    step.max_q, step.max_kv = max(q_lens), max(s + n for n, s in zip(q_lens, starts))
    step.dtype, step.device = dtype, torch.device(DEVICE)
    return step


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part_folds_the_pending_delta(dtype):
    from pylon_b200.parts import NORMS, PartSpec, ResidualStream

    width, eps = 200, 1e-5
    norm = NORMS.build(PartSpec("rmsnorm", {"width": width, "eps": eps}))
    weight = torch.rand(width) + 0.5
    norm.load({"weight": weight.to(DEVICE)}, dtype, torch.device(DEVICE))
    residual = torch.randn(6, width, device=DEVICE)
    delta = torch.randn(6, width, device=DEVICE).to(dtype)
    stream = ResidualStream(residual.clone())
    stream.add(delta)
    out = norm.apply(stream)
    want_sum = residual.double() + delta.double()
    torch.testing.assert_close(stream.residual.double(), want_sum, rtol=1e-6, atol=1e-6)
    assert stream.pending is None
    want = plain.rms_norm(want_sum.cpu(), weight.double(), eps)
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(out.double().cpu(), want, **tol)


def test_rotary_part_builds_the_reference_tables():
    from pylon_b200.parts import POSITION_ENCODINGS, PartSpec

    rope = POSITION_ENCODINGS.build(PartSpec("rope", {"head_dim": 48, "theta": 1_000_000.0, "max_positions": 300}))
    cos, sin, rotary = rope.rotary_table(torch.device(DEVICE))
    want_cos, want_sin = plain.rope_tables(48, 1_000_000.0, torch.arange(300), torch.float32)
    assert rotary == 48 and cos.shape == (300, 24)
    torch.testing.assert_close(cos.cpu(), want_cos[:, :24], rtol=0, atol=1e-6)
    torch.testing.assert_close(sin.cpu(), want_sin[:, :24], rtol=0, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from pylon_b200.parts import FEED_FORWARDS, PartSpec

    width, inter, tokens = 72, 200, 11
    part = FEED_FORWARDS.build(PartSpec("swiglu", {"width": width, "intermediate": inter}))
    weights = {"gate_proj.weight": torch.randn(inter, width) * 0.1, "up_proj.weight": torch.randn(inter, width) * 0.1,
               "down_proj.weight": torch.randn(width, inter) * 0.1}
    weights = {k: v.to(dtype) for k, v in weights.items()}
    part.load({k: v.to(DEVICE) for k, v in weights.items()}, dtype, torch.device(DEVICE))
    h = torch.randn(tokens, width).to(dtype)
    out = part.forward(h.to(DEVICE), None)
    out = out.sum(0) if out.dim() == 3 else out
    want = plain.swiglu_part(h.double(), {"mlp." + k: v.double() for k, v in weights.items()}, "")
    tol = dict(rtol=3e-2, atol=3e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(out.double().cpu(), want, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, dim, window", [(4, 2, 16, None), (6, 3, 32, None), (10, 2, 64, None), (4, 1, 32, 7)])
def test_attention_part_whole_and_in_two_steps(dtype, heads, kv_heads, dim, window):
    """The attention mixer alone with a hand-made cache: a whole sequence in one step, and
    the same sequence in two steps, against the plain attention part."""
    from pylon_b200.parts import MIXERS, LayerCache, PartSpec

    width, tokens, page, eps = 80, 37, 8, 1e-5
    spec = PartSpec("gqa_attention", {
        "width": width, "n_heads": heads, "n_kv_heads": kv_heads, "head_dim": dim, "qk_norm_eps": eps, "window": window,
        "position": PartSpec("rope", {"head_dim": dim, "theta": 10_000.0, "max_positions": 64}),
    })
    torch.manual_seed(3)
    raw = {"q_proj.weight": torch.randn(heads * dim, width) * 0.1, "k_proj.weight": torch.randn(kv_heads * dim, width) * 0.1,
           "v_proj.weight": torch.randn(kv_heads * dim, width) * 0.1, "o_proj.weight": torch.randn(width, heads * dim) * 0.1}
    raw = {k: v.to(dtype) for k, v in raw.items()}
    norms = {"q_norm.weight": torch.rand(dim) + 0.5, "k_norm.weight": torch.rand(dim) + 0.5}
    h = torch.randn(tokens, width).to(dtype)
    cfg = {"num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": dim, "rms_norm_eps": eps}
    cos, sin = plain.rope_tables(dim, 10_000.0, torch.arange(tokens), torch.float64)
    weights64 = {"self_attn." + k: v.double() for k, v in {**raw, **norms}.items()}
    want = plain.attention_part(h.double(), weights64, "", cfg, cos, sin, window)

    def run(cuts):
        part = MIXERS.build(spec)
        part.load({**{k: v.to(DEVICE) for k, v in raw.items()}, **{k: v.to(DEVICE) for k, v in norms.items()}}, dtype, torch.device(DEVICE))
        pages = -(-tokens // page)
        cache = LayerCache(
            k_pages=torch.zeros(pages + 2, kv_heads, page, dim, device=DEVICE, dtype=dtype),
            v_pages=torch.zeros(pages + 2, kv_heads, page, dim, device=DEVICE, dtype=dtype),
            block_table=torch.tensor([[p + 1 for p in range(pages)]], device=DEVICE, dtype=torch.int32), page_size=page,
        )
        outs, start = [], 0
        for count in cuts:
            step = step_view([count], [start], dtype)
            out = part.forward(h[start : start + count].to(DEVICE).contiguous(), step, cache)
            outs.append((out.sum(0) if out.dim() == 3 else out).to(dtype))
            start += count
        return torch.cat(outs).double().cpu()

    tol = dict(rtol=3e-2, atol=3e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(run([tokens]), want, **tol)
    torch.testing.assert_close(run([20, 17]), want, **tol)
    torch.testing.assert_close(run([30, 1, 1, 5]), want, **tol)


# ---------------------------------------------------------------------------------------
# models put together in the test
# ---------------------------------------------------------------------------------------
def register_toy_parts():
    """Two mixers defined here, not in the framework: one with a state of its own (running mean of its
    inputs), one that keeps a single latent row per token in the pages and no value rows."""
    from pylon_b200.parts import MIXERS, CacheNeed, KVNeed, Mixer, StateNeed, TensorDecl
    from pylon_b200.kernels import ops

    if "toy_running_mean" in MIXERS.kinds():
        return

    @MIXERS.register("toy_running_mean")
    class RunningMean(Mixer):
        """delta_t = W mean(h_0..h_t).  State per request: the running sum, float32 [width]."""

        def __init__(self, width: int) -> None:
            self.width = width
            self.w = None

        def tensors(self):
            return (TensorDecl("mix.weight", (self.width, self.width)),)

        def load(self, tensors, dtype, device):
            self.w = tensors["mix.weight"].contiguous()

        def cache_need(self):
            return CacheNeed(state=StateNeed((self.width,), torch.float32))

        def forward(self, h, step, cache):
            # On the device from end to end (no look at the host), so that a decode step can be captured in a CUDA graph.
            rows = step.token_row[: h.shape[0]].long()
            starts, slots = step.q_start.long(), step.slots.long()
            total = torch.cumsum(h.float(), dim=0)
            before_row = torch.where((starts[:-1] > 0).unsqueeze(1), total[(starts[:-1] - 1).clamp(min=0)], torch.zeros_like(total[:1]))
            running = cache.state[slots][rows] + total - before_row[rows]
            cache.state.index_copy_(0, slots, running[starts[1:] - 1])
            means = running / (step.positions[: h.shape[0]].float() + 1.0).unsqueeze(1)
            return ops.linear(means.to(h.dtype), self.w)

    @MIXERS.register("toy_latent")
    class LatentAttention(Mixer):
        """Keeps ONE row per token, a latent c_t = Wc h_t, and no value rows: delta_t = Wo sum_j softmax_j(q_t . c_j / sqrt(L)) c_j
        over j <= t with q_t = Wq h_t.  The rows live in the manager's pages (one head of width L, value width 0)."""

        def __init__(self, width: int, latent: int) -> None:
            self.width, self.latent = width, latent
            self.wc = self.wq = self.wo = None

        def tensors(self):
            return (TensorDecl("c_proj.weight", (self.latent, self.width)), TensorDecl("q_proj.weight", (self.latent, self.width)),
                    TensorDecl("o_proj.weight", (self.width, self.latent)))

        def load(self, tensors, dtype, device):
            self.wc, self.wq, self.wo = (tensors[name].contiguous() for name in ("c_proj.weight", "q_proj.weight", "o_proj.weight"))

        def cache_need(self):
            return CacheNeed(kv=KVNeed(1, self.latent, value_dim=0))

        def forward(self, h, step, cache):
            assert cache.v_pages is None and cache.k_pages.shape[1:] == (1, cache.page_size, self.latent)
            tokens, page = h.shape[0], cache.page_size
            c, q = ops.linear(h, self.wc), ops.linear(h, self.wq)
            positions = step.positions[:tokens].long()
            tables = cache.block_table[step.token_row[:tokens].long()].long()                      # [T, W]
            own_page = tables.gather(1, (positions // page).unsqueeze(1)).squeeze(1)
            cache.k_pages[own_page, 0, positions % page] = c                                       # write first, then read
            rows = cache.k_pages[tables.clamp(min=0)].reshape(tokens, -1, self.latent).float()      # [T, W * page, L]
            scores = torch.einsum("tl,tkl->tk", q.float(), rows) / math.sqrt(self.latent)
            visible = torch.arange(rows.shape[1], device=h.device).unsqueeze(0) <= positions.unsqueeze(1)
            weights = torch.softmax(scores.masked_fill(~visible, float("-inf")), dim=-1)
            context = torch.einsum("tk,tkl->tl", weights, torch.where(visible.unsqueeze(2), rows, torch.zeros_like(rows)))
            return ops.linear(context.to(h.dtype), self.wo)


@dataclass(frozen=True)
class ToyConfig:
    """A made-up architecture for the tests: layer 0 mixes with the running mean, layer 1 with
    windowed attention, layer 2 with full attention, layer 3 with attention over one latent row per
    token; the order runs layer 0 twice.  The embedding is scaled and the logits are soft-capped."""

    architecture = "ToyForCausalLM"
    vocab_size: int = 200
    width: int = 48
    heads: int = 4
    kv_heads: int = 2
    head_dim: int = 16
    intermediate: int = 88
    window: int = 11
    eps: float = 1e-5
    latent: int = 24
    embedding_scale: float = 1.75
    logit_softcap: float = 0.6

    @classmethod
    def from_dict(cls, data):
        return cls(**{k: data[k] for k in ("vocab_size", "width", "heads", "kv_heads", "head_dim", "intermediate", "window", "eps", "latent",
                                           "embedding_scale", "logit_softcap")})

    def to_dict(self):
        return {"architectures": [self.architecture], **self.__dict__}


def toy_spec(config: ToyConfig, max_positions: Optional[int] = None):
    from pylon_b200.parts import LayerSpec, ModelSpec, PartSpec
    from pylon_b200.parts.spec import RunSpec

    positions = max_positions or 512
    norm = PartSpec("rmsnorm", {"width": config.width, "eps": config.eps})
    ffn = PartSpec("swiglu", {"width": config.width, "intermediate": config.intermediate})

    def attention(window):
        return PartSpec("gqa_attention", {
            "width": config.width, "n_heads": config.heads, "n_kv_heads": config.kv_heads, "head_dim": config.head_dim,
            "qk_norm_eps": config.eps, "window": window,
            "position": PartSpec("rope", {"head_dim": config.head_dim, "theta": 10_000.0, "max_positions": positions}),
        })

    def block(mixer):
        return PartSpec("prenorm", {"mixer": mixer, "feed_forward": ffn, "mixer_norm": norm, "ffn_norm": norm})

    layers = (
        LayerSpec("layers.0.", block(PartSpec("toy_running_mean", {"width": config.width}))),
        LayerSpec("layers.1.", block(attention(config.window))),
        LayerSpec("layers.2.", block(attention(None))),
        LayerSpec("layers.3.", block(PartSpec("toy_latent", {"width": config.width, "latent": config.latent}))),
    )
    return ModelSpec(
        width=config.width, vocab_size=config.vocab_size, max_positions=positions, embedding_name="embed.weight", lm_head_name="head.weight",
        final_norm=norm, final_norm_prefix="norm.", layers=layers, order=(RunSpec(0), RunSpec(1), RunSpec(0), RunSpec(2), RunSpec(3)),
        embedding_scale=config.embedding_scale, logit_scale=2.0, logit_softcap=config.logit_softcap,
    )


def toy_plain_forward(config: ToyConfig, w: Mapping[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """The toy model on a whole sequence, from the plain implementation's functions."""
    ids = torch.as_tensor(list(tokens))
    x = w["embed.weight"][ids] * config.embedding_scale
    cos, sin = plain.rope_tables(config.head_dim, 10_000.0, torch.arange(len(ids)), x.dtype)
    cfg = {"num_attention_heads": config.heads, "num_key_value_heads": config.kv_heads, "head_dim": config.head_dim, "rms_norm_eps": config.eps}

    def running_mean(h, prefix):
        means = torch.cumsum(h, dim=0) / torch.arange(1, len(h) + 1, dtype=h.dtype).unsqueeze(1)
        return means @ w[prefix + "self_attn.mix.weight"].T

    def latent_attention(h, prefix):
        c, q = h @ w[prefix + "self_attn.c_proj.weight"].T, h @ w[prefix + "self_attn.q_proj.weight"].T
        scores = q @ c.T / math.sqrt(config.latent)
        causal = torch.tril(torch.ones(len(h), len(h), dtype=torch.bool))
        return torch.softmax(scores.masked_fill(~causal, float("-inf")), dim=-1) @ c @ w[prefix + "self_attn.o_proj.weight"].T

    def run(x, layer, window):
        prefix = f"layers.{layer}."
        h = plain.rms_norm(x, w[prefix + "input_layernorm.weight"], config.eps)
        if layer == 0:
            x = x + running_mean(h, prefix)
        elif layer == 3:
            x = x + latent_attention(h, prefix)
        else:
            x = x + plain.attention_part(h, w, prefix, cfg, cos, sin, window)
        h = plain.rms_norm(x, w[prefix + "post_attention_layernorm.weight"], config.eps)
        return x + plain.swiglu_part(h, w, prefix)

    for layer, window in ((0, None), (1, config.window), (0, None), (2, None), (3, None)):
        x = run(x, layer, window)
    logits = (plain.rms_norm(x, w["norm.weight"], config.eps) @ w["head.weight"].T) * 2.0
    return config.logit_softcap * torch.tanh(logits / config.logit_softcap)


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    from pylon_b200.config import register_architecture
    from pylon_b200.config.registry import ARCHITECTURES
    from pylon_b200.weights import write_random_model

    register_toy_parts()
    register_architecture(ToyConfig.architecture, ToyConfig, toy_spec)
    folder = tmp_path_factory.mktemp("toy")
    write_random_model(ToyConfig(), 11, folder)
    yield folder
    ARCHITECTURES.pop(ToyConfig.architecture, None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "tail_one_by_one", "changing_portions", "mixed"])
def test_toy_model_with_state_window_and_a_layer_run_twice(toy_folder, cutting, dtype):
    """Registered, built from a model folder and stepped through the engine: the state of the
    running-mean mixer lives in the request's slot (one per run of the layer), the windowed
    layers have pages of their own and give back the ones the window has passed."""
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine

    config = ToyConfig()
    _, weights = plain.read_model(toy_folder)
    rng = np.random.default_rng(5)
    requests = {f"t{i}": rng.integers(0, config.vocab_size, size=n).tolist() for i, n in enumerate((61, 9, 44, 90, 25))}
    expected = {rid: plain.as_numpy(toy_plain_forward(config, weights, tokens)) for rid, tokens in requests.items()}
    builders = {"whole": trace_tools.whole, "tail_one_by_one": trace_tools.tail_one_by_one,
                "changing_portions": trace_tools.changing_portions, "mixed": trace_tools.mixed}
    steps = builders[cutting](requests)
    page = 8
    # no portion of these cuttings but a whole prompt is longer than 24 tokens: the pools are sized for steps of that many
    chunk = 24 if cutting in ("changing_portions", "mixed") else 128
    engine = Engine(toy_folder, EngineConfig(dtype=dtype, page_size=page, max_cache_tokens=trace_tools.pool_tokens(steps, page),
                                             max_context=128, max_batch_size=4, prefill_chunk_size=chunk))
    assert len(engine.cache.groups) == 3        # windowed attention, full attention, latent rows: pages of their own
    assert engine.cache.state_bytes_per_request() == 2 * config.width * 4   # one state per run of layer 0
    latent = next(g for g in engine.cache.groups if g.need.value_width == 0)
    assert latent.values is None and latent.keys.shape[2:] == (1, page, config.latent)
    element = 4 if dtype == "float32" else 2
    assert engine.cache.bytes_per_token() == (2 * 2 * config.kv_heads * config.head_dim + config.latent) * element
    got = trace_tools.run_in_process(engine, steps)
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == "float32" else dict(rtol=3e-2, atol=3e-2)
    for rid in requests:
        np.testing.assert_allclose(got[rid], expected[rid], err_msg=rid, **tol)
    windowed = next(g for g in engine.cache.groups if g.need.window is not None)
    full = next(g for g in engine.cache.groups if g.need.window is None and g.need.value_width)
    assert windowed.pool.free_count == windowed.pool.num_pages and full.pool.free_count == full.pool.num_pages
    if cutting != "whole":
        # the windowed group never needed as many pages at once as the full one
        assert windowed.pool.acquired_total >= full.pool.acquired_total > 0
    if chunk == 24:
        # and was given fewer: four requests of window + one step's tokens each, not the whole pool
        assert windowed.pool.num_pages == min(full.pool.num_pages, 4 * (-(-(config.window - 1 + chunk) // page) + 1))
        assert cutting != "mixed" or windowed.pool.num_pages < full.pool.num_pages


@pytest.mark.parametrize("cutting", ["tail_one_by_one", "mixed"])
def test_toy_model_decodes_from_cuda_graphs(toy_folder, cutting):
    """Every mixer of the toy model runs on the device from end to end, so its decode steps are captured.  Capturing a
    step runs it once eagerly first; the running-mean mixer's state must not be advanced by that run as well."""
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine

    config = ToyConfig()
    _, weights = plain.read_model(toy_folder)
    rng = np.random.default_rng(6)
    requests = {f"g{i}": rng.integers(0, config.vocab_size, size=n).tolist() for i, n in enumerate((50, 33, 71, 40))}
    expected = {rid: plain.as_numpy(toy_plain_forward(config, weights, tokens)) for rid, tokens in requests.items()}
    steps = (trace_tools.tail_one_by_one if cutting == "tail_one_by_one" else trace_tools.mixed)(requests)
    engine = Engine(toy_folder, EngineConfig(dtype="float32", page_size=8, max_cache_tokens=trace_tools.pool_tokens(steps, 8),
                                             max_context=128, max_batch_size=4, cuda_graphs=True))
    got = trace_tools.run_in_process(engine, steps)
    for rid in requests:
        np.testing.assert_allclose(got[rid], expected[rid], err_msg=rid, rtol=1e-4, atol=1e-5)
    graphs = engine.step_function.graphs
    assert (graphs.captured or graphs.captured_alike) and not graphs.failed


def test_a_failed_step_leaves_pages_and_state_as_they_were(toy_folder):
    """A step that fails after some of its layers ran (here: the last block raises, once) must leave its requests as
    they were: the pages it acquired go back, and the running-mean state, which its first layers advanced, is restored;
    the same step then gives the logits it should."""
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine, StepEntry

    config = ToyConfig()
    _, weights = plain.read_model(toy_folder)
    rng = np.random.default_rng(7)
    tokens = {"a": rng.integers(0, config.vocab_size, size=40).tolist(), "b": rng.integers(0, config.vocab_size, size=27).tolist()}
    expected = {rid: plain.as_numpy(toy_plain_forward(config, weights, ids)) for rid, ids in tokens.items()}
    engine = Engine(toy_folder, EngineConfig(dtype="float32", page_size=8, max_cache_tokens=256, max_context=128, max_batch_size=4))
    live = {rid: engine.open(rid, 128) for rid in tokens}
    engine.step([StepEntry(live["a"], tokens["a"][:30], ()), StepEntry(live["b"], tokens["b"][:20], ())])
    free_before = engine.cache.free_pages()
    last_block = engine.model.blocks[engine.spec.order[-1].layer]
    healthy = last_block.forward

    def failing(*args, **kwargs):
        last_block.forward = healthy
        raise RuntimeError("injected")

    entries = [StepEntry(live["a"], tokens["a"][30:], tuple(range(10))), StepEntry(live["b"], tokens["b"][20:], tuple(range(7)))]
    last_block.forward = failing
    with pytest.raises(RuntimeError, match="injected"):
        engine.step(entries)
    assert engine.cache.free_pages() == free_before and live["a"].length == 30 and live["b"].length == 20
    engine.cache.check()
    got = engine.step(entries).cpu().numpy()
    np.testing.assert_allclose(got[:10], expected["a"][30:], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(got[10:], expected["b"][20:], rtol=1e-4, atol=1e-5)


# ---------------------------------------------------------------------------------------
# a second made-up architecture: a feed-forward with routing and another position encoding
# ---------------------------------------------------------------------------------------
def register_routed_toy_parts():
    """Defined here, not in the framework: a feed-forward that routes each token to one of a few
    small experts, and a rotary encoding over neighbouring pairs (2j, 2j + 1), which is no
    rotation by the framework's table layout and therefore runs through ``apply``."""
    from pylon_b200.kernels import ops
    from pylon_b200.parts import FEED_FORWARDS, MIXERS, POSITION_ENCODINGS, CacheNeed, FeedForward, Mixer, PositionEncoding, TensorDecl

    if "toy_routed" in FEED_FORWARDS.kinds():
        return

    @MIXERS.register("toy_cache_reader")
    class CacheReader(Mixer):
        """delta = Wo attention(q = Wq h; the keys and values of the run whose cache it is handed).  It keeps nothing
        itself: its run of the order names an earlier run's cache, which holds this step's tokens already."""

        def __init__(self, width: int, n_heads: int, head_dim: int) -> None:
            self.width, self.n_heads, self.head_dim = width, n_heads, head_dim
            self.wq = self.wo = None

        def tensors(self):
            return (TensorDecl("q_proj.weight", (self.n_heads * self.head_dim, self.width)),
                    TensorDecl("o_proj.weight", (self.width, self.n_heads * self.head_dim)))

        def load(self, tensors, dtype, device):
            self.wq, self.wo = tensors["q_proj.weight"].contiguous(), tensors["o_proj.weight"].contiguous()

        def cache_need(self):
            return CacheNeed()

        def forward(self, h, step, cache):
            assert cache.k_pages is not None and cache.v_pages is not None and cache.k_pages.shape[3] == self.head_dim
            q = ops.linear(h, self.wq)
            context = ops.paged_attention(q, cache.k_pages, cache.v_pages, step.positions, step.token_row, step.q_start, step.kv_len,
                                          cache.block_table, self.n_heads, step.max_q, step.max_kv, row_tokens=step.row_tokens,
                                          rows_alike=step.rows_alike)
            return ops.linear(context, self.wo)

    @FEED_FORWARDS.register("toy_routed")
    class Routed(FeedForward):
        """delta = p_e * down_e(gelu(up_e(h))) for the expert e with the largest router logit; p = softmax of
        the logits, which are formed in float32."""

        def __init__(self, width: int, intermediate: int, experts: int) -> None:
            self.width, self.intermediate, self.experts = width, intermediate, experts
            self.router = None
            self.up, self.down = [], []

        def tensors(self):
            decls = [TensorDecl("router.weight", (self.experts, self.width), "vector")]
            for e in range(self.experts):
                decls += [TensorDecl(f"experts.{e}.up.weight", (self.intermediate, self.width)),
                          TensorDecl(f"experts.{e}.down.weight", (self.width, self.intermediate))]
            return decls

        def load(self, tensors, dtype, device):
            self.router = tensors["router.weight"].contiguous()
            self.up = [tensors[f"experts.{e}.up.weight"].contiguous() for e in range(self.experts)]
            self.down = [tensors[f"experts.{e}.down.weight"].contiguous() for e in range(self.experts)]

        def forward(self, h, step):
            logits = h.float() @ self.router.t()
            probabilities = torch.softmax(logits, dim=-1)
            chosen = torch.argmax(logits, dim=-1)
            out = torch.zeros_like(h)
            for e in range(self.experts):
                rows = torch.nonzero(chosen == e).squeeze(1)
                if rows.numel() == 0:
                    continue
                hidden = torch.nn.functional.gelu(ops.linear(h[rows].contiguous(), self.up[e]).float()).to(h.dtype)
                out[rows] = (ops.linear(hidden, self.down[e]).float() * probabilities[rows, e].unsqueeze(1)).to(h.dtype)
            return out

    @POSITION_ENCODINGS.register("toy_neighbour_pairs")
    class NeighbourPairs(PositionEncoding):
        def __init__(self, head_dim: int, theta: float) -> None:
            self.head_dim, self.theta = head_dim, theta

        def apply(self, q, k, step):
            tokens = q.shape[0]
            inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.head_dim, 2, dtype=torch.float32, device=q.device) / self.head_dim))
            angles = step.positions[:tokens].float().unsqueeze(1) * inv_freq.unsqueeze(0)
            cos, sin = torch.cos(angles).unsqueeze(1), torch.sin(angles).unsqueeze(1)     # [T, 1, d/2]
            for x in (q, k):
                pairs = x.unflatten(1, (-1, self.head_dim // 2, 2)).float()                  # [T, heads, d/2, 2]
                even, odd = pairs[..., 0], pairs[..., 1]
                x.copy_(torch.stack((even * cos - odd * sin, odd * cos + even * sin), dim=-1).flatten(1).to(x.dtype))


@dataclass(frozen=True)
class RoutedToyConfig:
    """Layer 0: attention with q/k norms and the neighbour-pair rotation, then the routed feed-forward;
    layer 1: the same attention and a SwiGLU feed-forward; layer 2: a mixer that has queries only and reads the
    keys and values that layer 1 keeps (its run of the order names layer 1's cache), and a SwiGLU feed-forward."""

    architecture = "RoutedToyForCausalLM"
    vocab_size: int = 150
    width: int = 80
    heads: int = 6
    kv_heads: int = 3
    head_dim: int = 16
    intermediate: int = 72
    experts: int = 3
    eps: float = 1e-5

    @classmethod
    def from_dict(cls, data):
        return cls(**{k: data[k] for k in ("vocab_size", "width", "heads", "kv_heads", "head_dim", "intermediate", "experts", "eps")})

    def to_dict(self):
        return {"architectures": [self.architecture], **self.__dict__}


def routed_toy_spec(config: RoutedToyConfig, max_positions: Optional[int] = None):
    from pylon_b200.parts import LayerSpec, ModelSpec, PartSpec
    from pylon_b200.parts.spec import RunSpec

    norm = PartSpec("rmsnorm", {"width": config.width, "eps": config.eps})
    attention = PartSpec("gqa_attention", {
        "width": config.width, "n_heads": config.heads, "n_kv_heads": config.kv_heads, "head_dim": config.head_dim,
        "qk_norm_eps": config.eps, "position": PartSpec("toy_neighbour_pairs", {"head_dim": config.head_dim, "theta": 100.0}),
    })
    routed = PartSpec("toy_routed", {"width": config.width, "intermediate": config.intermediate, "experts": config.experts})
    dense = PartSpec("swiglu", {"width": config.width, "intermediate": config.intermediate})
    reader = PartSpec("toy_cache_reader", {"width": config.width, "n_heads": config.heads, "head_dim": config.head_dim})
    block = lambda ffn, mixer=attention: PartSpec("prenorm", {"mixer": mixer, "feed_forward": ffn, "mixer_norm": norm, "ffn_norm": norm})
    return ModelSpec(
        width=config.width, vocab_size=config.vocab_size, max_positions=max_positions or 512, embedding_name="embed.weight",
        lm_head_name="head.weight", final_norm=norm, final_norm_prefix="norm.",
        layers=(LayerSpec("layers.0.", block(routed)), LayerSpec("layers.1.", block(dense)), LayerSpec("layers.2.", block(dense, reader))),
        order=(RunSpec(0), RunSpec(1), RunSpec(2, cache_of=1)),
    )


def routed_toy_plain_forward(config: RoutedToyConfig, w: Mapping[str, torch.Tensor], tokens: Sequence[int]):
    """Whole sequence, no cache; returns the logits and the smallest gap between the two largest router logits."""
    ids = torch.as_tensor(list(tokens))
    x = w["embed.weight"][ids]
    count, d = len(ids), config.head_dim
    inv_freq = 1.0 / (100.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    angles = (torch.arange(count, dtype=torch.float32).unsqueeze(1) * inv_freq.unsqueeze(0)).to(x.dtype)
    cos, sin = torch.cos(angles), torch.sin(angles)                                        # [T, d/2]

    def rotate(heads):                                                                     # [n, T, d]
        even, odd = heads[..., 0::2], heads[..., 1::2]
        return torch.stack((even * cos - odd * sin, odd * cos + even * sin), dim=-1).flatten(-2)

    def attention(h, prefix):
        project = lambda name, n: (h @ w[prefix + f"self_attn.{name}_proj.weight"].T).reshape(count, n, d).transpose(0, 1)
        q = rotate(plain.rms_norm(project("q", config.heads), w[prefix + "self_attn.q_norm.weight"], config.eps))
        k = rotate(plain.rms_norm(project("k", config.kv_heads), w[prefix + "self_attn.k_norm.weight"], config.eps))
        v = project("v", config.kv_heads)
        kept[prefix] = (k, v)
        context = plain.causal_attention(q, k, v)
        return context.transpose(0, 1).reshape(count, -1) @ w[prefix + "self_attn.o_proj.weight"].T

    kept = {}   # what each attention layer's cache holds: normalised, rotated keys and the values

    def reader(h, prefix, owner):
        q = (h @ w[prefix + "self_attn.q_proj.weight"].T).reshape(count, config.heads, d).transpose(0, 1)
        context = plain.causal_attention(q, *kept[owner])
        return context.transpose(0, 1).reshape(count, -1) @ w[prefix + "self_attn.o_proj.weight"].T

    smallest_gap = float("inf")

    def routed(h, prefix):
        nonlocal smallest_gap
        logits = h @ w[prefix + "mlp.router.weight"].T
        top2 = torch.topk(logits, 2, dim=-1).values
        smallest_gap = min(smallest_gap, float((top2[:, 0] - top2[:, 1]).min()))
        probabilities, chosen = torch.softmax(logits, dim=-1), torch.argmax(logits, dim=-1)
        out = torch.zeros_like(h)
        for t in range(count):
            e = int(chosen[t])
            hidden = torch.nn.functional.gelu(h[t] @ w[prefix + f"mlp.experts.{e}.up.weight"].T)
            out[t] = probabilities[t, e] * (hidden @ w[prefix + f"mlp.experts.{e}.down.weight"].T)
        return out

    for layer in (0, 1, 2):
        prefix = f"layers.{layer}."
        h = plain.rms_norm(x, w[prefix + "input_layernorm.weight"], config.eps)
        x = x + (attention(h, prefix) if layer < 2 else reader(h, prefix, "layers.1."))
        h = plain.rms_norm(x, w[prefix + "post_attention_layernorm.weight"], config.eps)
        x = x + (routed(h, prefix) if layer == 0 else plain.swiglu_part(h, w, prefix))
    return plain.rms_norm(x, w["norm.weight"], config.eps) @ w["head.weight"].T, smallest_gap


@pytest.fixture(scope="module")
def routed_toy_folder(tmp_path_factory):
    """Random weights, except that the routing is made decisive: the embedding of token t carries a strong
    component in coordinate t mod experts, and expert e's router row reads that coordinate.  A token whose two
    largest router logits nearly tie would be routed differently by a rounding error, and one such token spoils
    every later position of its sequence."""
    from safetensors import safe_open
    from safetensors.torch import save_file

    from pylon_b200.config import register_architecture
    from pylon_b200.config.registry import ARCHITECTURES
    from pylon_b200.weights import write_random_model

    register_routed_toy_parts()
    register_architecture(RoutedToyConfig.architecture, RoutedToyConfig, routed_toy_spec)
    config = RoutedToyConfig()
    folder = tmp_path_factory.mktemp("routed_toy")
    write_random_model(config, 23, folder)
    path = str(folder / "model.safetensors")
    with safe_open(path, framework="pt") as handle:
        tensors = {name: handle.get_tensor(name) for name in handle.keys()}
    embedding = tensors["embed.weight"].float()
    embedding[:, : config.experts] = 0.0
    embedding[torch.arange(config.vocab_size), torch.arange(config.vocab_size) % config.experts] = 0.25
    tensors["embed.weight"] = embedding.to(torch.bfloat16)
    router = torch.zeros(config.experts, config.width)
    router[torch.arange(config.experts), torch.arange(config.experts)] = 0.4
    tensors["layers.0.mlp.router.weight"] = router.to(torch.bfloat16)
    save_file(tensors, path, metadata={"format": "pt"})
    yield folder
    ARCHITECTURES.pop(RoutedToyConfig.architecture, None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "tail_one_by_one", "changing_portions", "mixed"])
def test_toy_model_with_routed_feed_forward_and_another_position_encoding(routed_toy_folder, cutting, dtype):
    """Different feed-forwards in different layers, one of them routing tokens to experts, and a
    position encoding that the attention part cannot fuse: it runs between the q/k norms and the
    cache write.  Registered, built from a model folder and stepped through the engine."""
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine

    config = RoutedToyConfig()
    _, weights = plain.read_model(routed_toy_folder)
    rng = np.random.default_rng(9)
    requests = {f"r{i}": rng.integers(0, config.vocab_size, size=n).tolist() for i, n in enumerate((57, 12, 40, 83, 21))}
    expected = {}
    for rid, tokens in requests.items():
        logits, gap = routed_toy_plain_forward(config, weights, tokens)
        assert gap > 0.5, "the routing of the test model is meant to be decisive"
        expected[rid] = plain.as_numpy(logits)
    builders = {"whole": trace_tools.whole, "tail_one_by_one": trace_tools.tail_one_by_one,
                "changing_portions": trace_tools.changing_portions, "mixed": trace_tools.mixed}
    steps = builders[cutting](requests)
    page = 16
    engine = Engine(routed_toy_folder, EngineConfig(dtype=dtype, page_size=page, max_cache_tokens=trace_tools.pool_tokens(steps, page),
                                                    max_context=128, max_batch_size=4))
    # three runs, two caches: the reader's run is handed the pages of the run it names, and they are counted once
    assert len(engine.cache.groups) == 1 and engine.cache.bytes_per_token() == 2 * 2 * config.kv_heads * config.head_dim * (4 if dtype == "float32" else 2)
    got = trace_tools.run_in_process(engine, steps)
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == "float32" else dict(rtol=3e-2, atol=3e-2)
    for rid in requests:
        np.testing.assert_allclose(got[rid], expected[rid], err_msg=rid, **tol)
    # every expert had work: the comparison covered all of them
    used = {int(t) % config.experts for tokens in requests.values() for t in tokens}
    assert used == set(range(config.experts))


# ---------------------------------------------------------------------------------------
# a third made-up architecture: another norm and another arrangement of a block
# ---------------------------------------------------------------------------------------
def register_parallel_toy_parts():
    """Defined here, not in the framework: a norm that subtracts the mean and has a bias, and a block in which
    the mixer and the feed-forward read the same normalised input and both add to the stream."""
    from pylon_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, Norm, TensorDecl

    if "toy_layernorm" in NORMS.kinds():
        return

    @NORMS.register("toy_layernorm")
    class LayerNorm(Norm):
        """y = (x - mean) / sqrt(var + eps) * weight + bias, in float32, on the residual sum with the pending delta folded in."""

        def __init__(self, width: int, eps: float) -> None:
            self.width, self.eps = width, eps
            self.weight = self.bias = self.dtype = None

        def tensors(self):
            return (TensorDecl("weight", (self.width,), "vector"), TensorDecl("bias", (self.width,), "vector"))

        def load(self, tensors, dtype, device):
            self.weight, self.bias, self.dtype = tensors["weight"].float(), tensors["bias"].float() - 1.0, dtype   # vectors are drawn around 1

        def apply(self, stream, rows=None):
            stream.flush()
            x = stream.residual if rows is None else stream.residual[rows.long()]
            centred = x - x.mean(-1, keepdim=True)
            return (centred * torch.rsqrt(centred.square().mean(-1, keepdim=True) + self.eps) * self.weight + self.bias).to(self.dtype)

    @BLOCKS.register("toy_parallel")
    class ParallelBlock(Block):
        """x += mixer(norm(x)) + feed_forward(norm(x)): one norm, two deltas."""

        def __init__(self, mixer, feed_forward, norm) -> None:
            self.mixer, self.feed_forward, self.norm = MIXERS.build(mixer), FEED_FORWARDS.build(feed_forward), NORMS.build(norm)
            self._children = (("self_attn.", self.mixer), ("mlp.", self.feed_forward), ("input_layernorm.", self.norm))

        def tensors(self):
            return [TensorDecl(prefix + d.name, d.shape, d.role) for prefix, part in self._children for d in part.tensors()]

        def load(self, tensors, dtype, device):
            for prefix, part in self._children:
                part.load({name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)}, dtype, device)

        def weight_bytes(self):
            return sum(part.weight_bytes() for _, part in self._children)

        def forward(self, stream, step, cache):
            h = self.norm.apply(stream)
            stream.add(self.mixer.forward(h, step, cache))
            stream.add(self.feed_forward.forward(h, step))   # the delta before it goes into the sum first


@dataclass(frozen=True)
class ParallelToyConfig:
    architecture = "ParallelToyForCausalLM"
    vocab_size: int = 170
    width: int = 56
    heads: int = 3
    kv_heads: int = 1
    head_dim: int = 32
    intermediate: int = 104
    eps: float = 3e-5
    layers: int = 3

    @classmethod
    def from_dict(cls, data):
        return cls(**{k: data[k] for k in ("vocab_size", "width", "heads", "kv_heads", "head_dim", "intermediate", "eps", "layers")})

    def to_dict(self):
        return {"architectures": [self.architecture], **self.__dict__}


def parallel_toy_spec(config: ParallelToyConfig, max_positions: Optional[int] = None):
    from pylon_b200.parts import LayerSpec, ModelSpec, PartSpec

    positions = max_positions or 512
    norm = PartSpec("toy_layernorm", {"width": config.width, "eps": config.eps})
    attention = PartSpec("gqa_attention", {
        "width": config.width, "n_heads": config.heads, "n_kv_heads": config.kv_heads, "head_dim": config.head_dim, "qk_norm_eps": config.eps,
        "window": None, "position": PartSpec("rope", {"head_dim": config.head_dim, "theta": 5_000.0, "max_positions": positions}),
    })
    block = PartSpec("toy_parallel", {"mixer": attention, "feed_forward": PartSpec("swiglu", {"width": config.width, "intermediate": config.intermediate}),
                                      "norm": norm})
    return ModelSpec(
        width=config.width, vocab_size=config.vocab_size, max_positions=positions, embedding_name="embed.weight", lm_head_name=None,
        final_norm=norm, final_norm_prefix="norm.", layers=tuple(LayerSpec(f"layers.{i}.", block) for i in range(config.layers)),
        order=tuple(range(config.layers)),
    )


def parallel_toy_plain_forward(config: ParallelToyConfig, w: Mapping[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    ids = torch.as_tensor(list(tokens))
    x = w["embed.weight"][ids]
    cos, sin = plain.rope_tables(config.head_dim, 5_000.0, torch.arange(len(ids)), x.dtype)
    cfg = {"num_attention_heads": config.heads, "num_key_value_heads": config.kv_heads, "head_dim": config.head_dim, "rms_norm_eps": config.eps}

    def layer_norm(x, prefix):
        centred = x - x.mean(-1, keepdim=True)
        return centred / torch.sqrt(centred.square().mean(-1, keepdim=True) + config.eps) * w[prefix + "weight"] + (w[prefix + "bias"] - 1.0)

    for layer in range(config.layers):
        prefix = f"layers.{layer}."
        h = layer_norm(x, prefix + "input_layernorm.")
        x = x + plain.attention_part(h, w, prefix, cfg, cos, sin, None) + plain.swiglu_part(h, w, prefix)
    return layer_norm(x, "norm.") @ w["embed.weight"].T


@pytest.fixture(scope="module")
def parallel_toy_folder(tmp_path_factory):
    from pylon_b200.config import register_architecture
    from pylon_b200.config.registry import ARCHITECTURES
    from pylon_b200.weights import write_random_model

    register_parallel_toy_parts()
    register_architecture(ParallelToyConfig.architecture, ParallelToyConfig, parallel_toy_spec)
    folder = tmp_path_factory.mktemp("parallel_toy")
    write_random_model(ParallelToyConfig(), 31, folder)
    yield folder
    ARCHITECTURES.pop(ParallelToyConfig.architecture, None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "tail_one_by_one", "changing_portions", "mixed"])
def test_toy_model_with_another_norm_and_another_block_arrangement(parallel_toy_folder, cutting, dtype):
    """A norm with mean and bias and a block whose mixer and feed-forward share one normalised input, both defined
    above; the head shares the embedding table; one KV head of size 32 under three query heads."""
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine

    config = ParallelToyConfig()
    _, weights = plain.read_model(parallel_toy_folder)
    rng = np.random.default_rng(13)
    requests = {f"p{i}": rng.integers(0, config.vocab_size, size=n).tolist() for i, n in enumerate((48, 70, 15, 33, 64))}
    expected = {rid: plain.as_numpy(parallel_toy_plain_forward(config, weights, tokens)) for rid, tokens in requests.items()}
    builders = {"whole": trace_tools.whole, "tail_one_by_one": trace_tools.tail_one_by_one,
                "changing_portions": trace_tools.changing_portions, "mixed": trace_tools.mixed}
    steps = builders[cutting](requests)
    page = 4
    engine = Engine(parallel_toy_folder, EngineConfig(dtype=dtype, page_size=page, max_cache_tokens=trace_tools.pool_tokens(steps, page),
                                                      max_context=128, max_batch_size=4))
    got = trace_tools.run_in_process(engine, steps)
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == "float32" else dict(rtol=3e-2, atol=3e-2)
    for rid in requests:
        np.testing.assert_allclose(got[rid], expected[rid], err_msg=rid, **tol)
