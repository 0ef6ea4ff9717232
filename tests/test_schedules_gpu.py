"""Schedules and sizes that the other engine tests do not reach, each with its logits checked
against the plain implementation: the serving page size (256 tokens) with tables of several
pages and portions that cross page edges; one long request (more than 8,000 tokens) fed in
2,048-token portions and then decoded; decode steps of 64 rows, and 63 decoded rows beside one
prompt portion, at Qwen3-4B widths; and a run whose steps the scheduler makes.

The models here have sharpened attention: the per-head q/k norm weights are scaled up so that a
query's softmax rests on a few keys, and the value and output projections and the head are scaled
up so that what attention returns shows in the logits.  With plain N(0, 0.02) weights a key
that is lost, or read from the wrong page, changes the logits by less than bfloat16 rounding does.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import trace_tools

pytestmark = pytest.mark.gpu


def sharpen(folder, qk_gain: float = 1.6, value_gain: float = 3.0, head_gain: float = 4.0) -> None:
    """Rewrites the model folder's weights as the module's header says."""
    from safetensors import safe_open
    from safetensors.torch import save_file

    path = str(folder / "model.safetensors")
    with safe_open(path, framework="pt") as handle:
        tensors = {name: handle.get_tensor(name) for name in handle.keys()}
    for name in list(tensors):
        gain = None
        if name.endswith(("q_norm.weight", "k_norm.weight")):
            gain = qk_gain
        elif name.endswith(("v_proj.weight", "o_proj.weight")):
            gain = value_gain
        elif name in ("lm_head.weight",):
            gain = head_gain
        if gain is not None:
            tensors[name] = (tensors[name].float() * gain).to(tensors[name].dtype)
    save_file(tensors, path, metadata={"format": "pt"})


def make_model(tmp_path_factory, label: str, fields: dict, seed: int):
    from pylon_b200.config import Qwen3Config
    from pylon_b200.weights import write_random_model

    folder = tmp_path_factory.mktemp(label)
    write_random_model(Qwen3Config(**fields), seed, folder)
    sharpen(folder)
    cfg, weights = plain.read_model(folder, torch.float64)
    return folder, cfg, {name: tensor.cuda() for name, tensor in weights.items()}


def plain_logits(cfg, weights, tokens) -> np.ndarray:
    with torch.no_grad():
        return plain.forward(cfg, weights, tokens).cpu().numpy()


def check(got: np.ndarray, want: np.ndarray, dtype: str, what: str) -> None:
    """float32: close everywhere.  bfloat16: every activation is rounded to 8 bits of mantissa, and a sharp softmax
    multiplies what that does to a score; on these models the error against the plain implementation measures 1 to 1.5 % of
    the logits' spread (root mean square), the same under every cutting, with a largest value near 12 % among hundreds of
    thousands of logits.  The check allows 2.5 % and 25 %, and asks for the plain arg-max wherever its margin is clear.  A
    key tile lost or read from the wrong page for a few positions moves those positions' logits by about the spread itself."""
    assert got.shape == want.shape, (what, got.shape, want.shape)
    spread = float(want.std())
    if dtype == "float32":
        np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-4 * max(1.0, spread), err_msg=what)
        return
    error = got.astype(np.float64) - want
    rms, worst = float(np.sqrt((error**2).mean())), float(np.abs(error).max())
    print(f"bfloat16 {what}: rms {rms / spread:.4f} worst {worst / spread:.3f} of the spread")
    assert rms < 0.025 * spread and worst < 0.25 * spread, (what, rms / spread, worst / spread)
    ordered = np.sort(want, axis=-1)
    clear = (ordered[:, -1] - ordered[:, -2]) > 0.1 * spread
    assert (got.argmax(-1)[clear] == want.argmax(-1)[clear]).all(), what


# ---------------------------------------------------------------------------------------
# (a) the serving page size
# ---------------------------------------------------------------------------------------
PAGE_256_MODEL = dict(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                      intermediate_size=512, max_position_embeddings=2_048, rope_theta=5_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
PAGE_256_LENGTHS = (300, 1_100, 513, 767, 256, 640)


@pytest.fixture(scope="module")
def page_256_model(tmp_path_factory):
    folder, cfg, weights = make_model(tmp_path_factory, "page256", PAGE_256_MODEL, 31)
    rng = np.random.default_rng(41)
    requests = {f"q{i}": rng.integers(0, PAGE_256_MODEL["vocab_size"], size=n).tolist() for i, n in enumerate(PAGE_256_LENGTHS)}
    expected = {rid: plain_logits(cfg, weights, tokens) for rid, tokens in requests.items()}
    return folder, requests, expected


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "tail_one_by_one", "changing_portions", "mixed"])
def test_pages_of_256_tokens_under_every_cutting(page_256_model, cutting, dtype):
    """Requests of 256 to 1,100 tokens over 256-token pages: tables of up to five pages, portions that end on, before and
    after page edges, four 64-key tiles to a page, and a pool so small that pages are used again."""
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine

    folder, requests, expected = page_256_model
    steps = {
        "whole": lambda: trace_tools.whole(requests),
        "tail_one_by_one": lambda: trace_tools.tail_one_by_one(requests),
        "changing_portions": lambda: trace_tools.changing_portions(requests, sizes=(255, 2, 257, 64, 130, 3, 190, 512, 2, 77)),
        "mixed": lambda: trace_tools.mixed(requests, seed=4, decode_tail=10, max_portion=300),
    }[cutting]()
    engine = Engine(folder, EngineConfig(dtype=dtype, page_size=256, max_cache_tokens=trace_tools.pool_tokens(steps, 256), max_context=1_280,
                                         max_batch_size=4, cuda_graphs=dtype == "bfloat16"))
    got = trace_tools.run_in_process(engine, steps)
    for rid in requests:
        check(got[rid], expected[rid], dtype, f"{cutting} {rid}")
    pool = engine.cache.groups[0].pool
    assert pool.free_count == pool.num_pages and pool.acquired_total > pool.num_pages


# ---------------------------------------------------------------------------------------
# (b) one long request
# ---------------------------------------------------------------------------------------
LONG_MODEL = dict(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                  intermediate_size=512, max_position_embeddings=40_960, rope_theta=5_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
LONG_PROMPTS, LONG_TAIL, SHORT_PROMPT = (8_300, 40_000), 32, 45   # 40,000: near the longest request Qwen3-4B takes (40,960)


@pytest.fixture(scope="module", params=LONG_PROMPTS)
def long_model(request, tmp_path_factory):
    folder, cfg, weights = make_model(tmp_path_factory, "long", LONG_MODEL, 32)
    rng = np.random.default_rng(42)
    requests = {"long": rng.integers(0, 512, size=request.param + LONG_TAIL).tolist(), "short": rng.integers(0, 512, size=SHORT_PROMPT + LONG_TAIL // 2).tolist()}
    expected = {rid: plain_logits(cfg, weights, tokens) for rid, tokens in requests.items()}
    del weights
    torch.cuda.empty_cache()
    return folder, requests, expected


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_request_in_portions_of_2048_and_then_token_by_token(long_model, dtype):
    """8,300 tokens (and 40,000) in portions of 2,048 (the second and later portions attend to thousands of cached keys),
    then 32 tokens one by one over more than 128 key tiles: the first 16 beside a short request (rows of very different lengths:
    the decode attention's form of equal runs), the last 16 alone (its cluster form), from CUDA graphs in bfloat16.
    Positions beyond 8,000 with a rotary base of 5,000,000."""
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine

    folder, requests, expected = long_model
    long_tokens, short_tokens = requests["long"], requests["short"]
    LONG_PROMPT = len(long_tokens) - LONG_TAIL
    steps = []

    def add(entries, end=()):
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": tokens, "want": list(range(len(tokens)))} for rid, tokens in entries], "end": list(end)})

    for begin in range(0, LONG_PROMPT, 2_048):
        add([("long", long_tokens[begin : min(begin + 2_048, LONG_PROMPT)])])
    add([("short", short_tokens[:SHORT_PROMPT])])
    half = LONG_TAIL // 2
    for index in range(half):
        add([("long", [long_tokens[LONG_PROMPT + index]]), ("short", [short_tokens[SHORT_PROMPT + index]])], end=["short"] if index == half - 1 else ())
    for index in range(half, LONG_TAIL):
        add([("long", [long_tokens[LONG_PROMPT + index]])], end=["long"] if index == LONG_TAIL - 1 else ())
    engine = Engine(folder, EngineConfig(dtype=dtype, page_size=256, max_cache_tokens=trace_tools.pool_tokens(steps, 256), max_context=-(-len(long_tokens) // 256) * 256,
                                         max_batch_size=2, cuda_graphs=dtype == "bfloat16"))
    got = trace_tools.run_in_process(engine, steps)
    for rid in requests:
        check(got[rid], expected[rid], dtype, rid)
        # the decoded tail by itself, where the attention's other kernels run
        tail = slice(len(requests[rid]) - (LONG_TAIL if rid == "long" else half), None)
        check(got[rid][tail], expected[rid][tail], dtype, f"{rid} tail")
    if dtype == "bfloat16":
        graphs = engine.step_function.graphs
        assert sorted(graphs.captured) == [2] and sorted(graphs.captured_alike) == [1] and not graphs.failed


# ---------------------------------------------------------------------------------------
# (c) steps of 64 rows at Qwen3-4B widths
# ---------------------------------------------------------------------------------------
WIDE_MODEL = dict(vocab_size=151_936, hidden_size=2_560, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                  intermediate_size=9_728, max_position_embeddings=4_096, rope_theta=5_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=True)
WIDE_ROWS, WIDE_PORTION = 64, 200


@pytest.fixture(scope="module")
def wide_model(tmp_path_factory):
    folder, cfg, weights = make_model(tmp_path_factory, "wide", WIDE_MODEL, 33)
    rng = np.random.default_rng(43)
    lengths = rng.integers(20, 90, size=WIDE_ROWS).tolist()
    requests = {f"w{i}": rng.integers(0, WIDE_MODEL["vocab_size"], size=n + 3).tolist() for i, n in enumerate(lengths)}
    requests["portion"] = rng.integers(0, WIDE_MODEL["vocab_size"], size=WIDE_PORTION + 1).tolist()
    # only the last four positions of each request are compared: its decoded tokens (151,936 logits a position)
    expected = {rid: plain_logits(cfg, weights, tokens)[-4:] for rid, tokens in requests.items()}
    del weights
    torch.cuda.empty_cache()
    return folder, requests, expected


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_of_64_rows_at_4b_widths(wide_model, dtype, graphs):
    """64 requests decode together (the library's products, the rotation kernel for many tokens, the decode attention's
    runs over 512 (row, KV head) pairs), eagerly and from the graph of size 64; then 63 of them decode beside one prompt
    portion of 200 tokens (the step function's hint of which rows are portions), then all 64 again."""
    if graphs and dtype == "float32":
        pytest.skip("graphs are checked in bfloat16, the precision that serves")
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine, StepEntry

    folder, requests, expected = wide_model
    names = [f"w{i}" for i in range(WIDE_ROWS)]
    engine = Engine(folder, EngineConfig(dtype=dtype, page_size=256, max_cache_tokens=(WIDE_ROWS + 1) * 256, max_context=256, max_batch_size=WIDE_ROWS,
                                         cuda_graphs=graphs))
    live = {rid: engine.open(rid, 256) for rid in names}
    for start in range(0, WIDE_ROWS, 16):     # prompts, sixteen requests a step
        engine.step([StepEntry(live[rid], requests[rid][:-3], ()) for rid in names[start : start + 16]])
    got = {rid: [] for rid in requests}

    def decode(rows, offset, extra=()):
        entries = [StepEntry(live[rid], [requests[rid][offset]], (0,)) for rid in rows] + list(extra)
        logits = engine.step(entries).float().cpu().numpy()
        for index, rid in enumerate(rows):
            got[rid].append(logits[index])
        return logits[len(rows):]

    decode(names, -3)                                              # 64 rows
    engine.close(live.pop(names[-1]))                              # its slot goes to the request that brings the portion
    live["portion"] = engine.open("portion", 256)
    rest = decode(names[:-1], -2, extra=[StepEntry(live["portion"], requests["portion"][:WIDE_PORTION], (WIDE_PORTION - 3, WIDE_PORTION - 2, WIDE_PORTION - 1))])
    got["portion"] = list(rest)
    rest = decode(names[:-1], -1, extra=[StepEntry(live["portion"], requests["portion"][WIDE_PORTION:], (0,))])   # 64 rows again, from the graph if on
    got["portion"].append(rest[0])
    for rid in names[:-1]:
        check(np.stack(got[rid]), expected[rid][1:], dtype, rid)
    check(np.stack(got[names[-1]]), expected[names[-1]][1:2], dtype, names[-1])
    check(np.stack(got["portion"]), expected["portion"], dtype, "portion")
    if graphs:
        captured = engine.step_function.graphs
        assert 64 in (set(captured.captured) | set(captured.captured_alike)) and not captured.failed
    from pylon_b200.kernels import ops

    ops.raise_on_kernel_errors(engine.device)


WIDE_LONG = 1_300


@pytest.fixture(scope="module")
def wide_long_model(tmp_path_factory):
    folder, cfg, weights = make_model(tmp_path_factory, "wide_long", WIDE_MODEL, 35)
    rng = np.random.default_rng(47)
    requests = {f"s{i}": rng.integers(0, WIDE_MODEL["vocab_size"], size=n + 3).tolist() for i, n in enumerate(rng.integers(20, 200, size=8).tolist())}
    requests["long"] = rng.integers(0, WIDE_MODEL["vocab_size"], size=WIDE_LONG).tolist()
    expected = {rid: plain_logits(cfg, weights, tokens)[-4:] for rid, tokens in requests.items()}
    del weights
    torch.cuda.empty_cache()
    return folder, requests, expected


def test_long_portions_at_4b_widths_finish_their_heads_in_the_product(wide_long_model, monkeypatch):
    """Portions of some 650 tokens at Qwen3-4B widths: their QKV product normalises, rotates and stores its heads in its
    own epilogue.  Eight short prompts run as one such step, the long request's first portion alone, its second beside the eight requests' decoded tokens (rows of one token before
    it in the step, positions that start at 650, pages of 256 that the portion crosses); the last three tokens and the
    decoded rows then go the usual way and read what the epilogues wrote."""
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine, StepEntry
    from pylon_b200.kernels import ops

    folder, requests, expected = wide_long_model
    fused_rows = []
    fused = ops.linear_qkv_rotated
    monkeypatch.setattr(ops, "linear_qkv_rotated", lambda x, *args: (fused_rows.append(x.shape[0]), fused(x, *args))[1])
    monkeypatch.setattr(ops, "QKV_ROTATION_MIN_ROWS", 512)   # the engine fuses from some 3,000 rows on, where it pays; the test makes do with fewer
    short = [f"s{i}" for i in range(8)]
    engine = Engine(folder, EngineConfig(dtype="bfloat16", page_size=256, max_cache_tokens=(8 + 6) * 256, max_context=1_536, max_batch_size=9,
                                         prefill_chunk_size=1_024, cuda_graphs=False))
    live = {rid: engine.open(rid, 256) for rid in short}
    live["long"] = engine.open("long", WIDE_LONG)
    engine.step([StepEntry(live[rid], requests[rid][:-3], ()) for rid in short])
    got = {rid: [] for rid in requests}
    engine.step([StepEntry(live["long"], requests["long"][:650], ())])
    logits = engine.step([StepEntry(live[rid], [requests[rid][-3]], (0,)) for rid in short]
                         + [StepEntry(live["long"], requests["long"][650 : WIDE_LONG - 3], (WIDE_LONG - 3 - 650 - 1,))]).float().cpu().numpy()
    for index, rid in enumerate(short):
        got[rid].append(logits[index])
    got["long"].append(logits[len(short)])
    prompts = sum(len(requests[rid]) - 3 for rid in short)   # the eight short prompts together are long enough as well
    assert fused_rows == [prompts] * 2 + [650] * 2 + [len(short) + WIDE_LONG - 3 - 650] * 2, fused_rows   # two layers a step
    logits = engine.step([StepEntry(live["long"], requests["long"][WIDE_LONG - 3 :], (0, 1, 2))]
                         + [StepEntry(live[rid], [requests[rid][-2]], (0,)) for rid in short]).float().cpu().numpy()
    got["long"] += list(logits[:3])
    for index, rid in enumerate(short):
        got[rid].append(logits[3 + index])
    check(np.stack(got["long"]), expected["long"], "bfloat16", "long")
    for rid in short:
        check(np.stack(got[rid]), expected[rid][1:3], "bfloat16", rid)
    ops.raise_on_kernel_errors(engine.device)


# ---------------------------------------------------------------------------------------
# (d) steps the scheduler makes
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype, graphs", [("float32", False), ("bfloat16", True)])
def test_a_run_the_scheduler_cuts(dtype, graphs, tmp_path_factory):
    """Fourteen requests through ``Engine.generate`` with a prompt budget of 48 tokens a tick, four slots and a pool that
    cannot hold them all: portions of several prompts beside decoded tokens in most ticks, admission that waits for pages.
    Every generated token is checked against the plain implementation's logits on the request's own prefix."""
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine
    from pylon_b200.sampling import SamplingParams

    fields = dict(vocab_size=384, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                  intermediate_size=320, max_position_embeddings=512, rope_theta=1_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
    folder, cfg, weights = make_model(tmp_path_factory, "scheduled", fields, 34)
    rng = np.random.default_rng(44)
    lengths = [130, 7, 64, 201, 33, 90, 150, 12, 75, 48, 180, 5, 111, 66]
    prompts = [rng.integers(0, fields["vocab_size"], size=n).tolist() for n in lengths]
    new_tokens = 12
    engine = Engine(folder, EngineConfig(dtype=dtype, page_size=64, max_cache_tokens=12 * 64, max_context=256, max_batch_size=4, max_queue_size=6,
                                         prefill_chunk_size=48, cuda_graphs=graphs))
    results = engine.generate(prompts, SamplingParams(max_new_tokens=new_tokens, temperature=0.0, ignore_eos=True))
    assert engine.scheduler.ticks > 40
    if graphs:   # the ticks that brought prompt portions were padded to captured sizes and replayed
        replays = engine.step_function.graphs.replays
        assert replays["padded"] > 10 and replays["decode"] > 0 and not engine.step_function.graphs.failed
    spread = None
    for prompt, result in zip(prompts, results):
        assert result.error is None and len(result.output_ids) == new_tokens and result.prompt_tokens == len(prompt)
        logits = plain_logits(cfg, weights, prompt + result.output_ids)
        spread = float(logits.std()) if spread is None else spread
        for offset, token in enumerate(result.output_ids):
            row = logits[len(prompt) - 1 + offset]
            margin = float(row.max() - row[token])
            assert margin <= (1e-4 if dtype == "float32" else 0.06) * spread, (len(prompt), offset, token, int(row.argmax()), margin)
    engine.cache.check()
    pool = engine.cache.groups[0].pool
    assert pool.free_count == pool.num_pages and pool.acquired_total > pool.num_pages


def test_a_trace_of_mixed_steps_gives_the_same_bits_every_time(wide_model):
    """A fixed trace of scheduler-shaped steps at Qwen3-4B widths (portions of up to 700 tokens beside decoded tokens of
    up to eight requests, requests of 100 to 2,400 tokens, pages of 256, graphs on), three times over: the first pass warms
    up and captures, the second and third must agree bit for bit at every step, with no error word set.  The kernels of a
    step overlap one another (dependent launch) and wait for one another through barriers; a result that is read a moment
    too early, or a wait that takes another phase for its own, shows here as a bit that differs from pass to pass or as a
    wait that ran out, whatever the plain logits' tolerance would forgive."""
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine, StepEntry
    from pylon_b200.kernels import ops

    folder, _, _ = wide_model
    rng = np.random.default_rng(12)
    requests = {f"r{index}": rng.integers(0, WIDE_MODEL["vocab_size"], size=int(length)).tolist() for index, length in enumerate(rng.integers(100, 2_400, size=14))}
    steps = trace_tools.mixed(requests, seed=12, max_live=8, decode_tail=16, max_portion=700)
    engine = Engine(folder, EngineConfig(dtype="bfloat16", page_size=256, max_cache_tokens=8 * 2_560, max_context=2_560, max_batch_size=8, cuda_graphs=True))
    engine.step_function.graphs.capture_at_once = True

    def one_pass():
        live, outputs = {}, []
        for step in steps:
            entries = []
            for item in step["entries"]:
                if item["id"] not in live:
                    live[item["id"]] = engine.open(item["id"], 2_560)
                entries.append(StepEntry(live[item["id"]], item["tokens"], (len(item["tokens"]) - 1,)))
            outputs.append(engine.step(entries).clone())
            for name in step["end"]:
                engine.close(live.pop(name))
        torch.cuda.synchronize()
        return outputs

    one_pass()
    second, third = one_pass(), one_pass()
    assert all(bool(torch.isfinite(logits).all()) for logits in second)
    differing = [index for index, (a, b) in enumerate(zip(second, third)) if not torch.equal(a, b)]
    assert not differing, f"steps {differing[:8]} of {len(steps)} differ between two passes over the same trace"
    assert ops._error_words(engine.device).tolist() == [0, 0, 0, 0]
    graphs = engine.step_function.graphs
    assert graphs.replays["padded"] > 50 and graphs.replays["decode"] > 20 and not graphs.failed
    engine.cache.check()


@pytest.mark.parametrize("tokens", [9, 17])
def test_a_short_prompt_portion_gives_the_same_logits_every_time(wide_model, tokens):
    """A prompt portion of a few tokens goes through the kernels of a decode step (the TMA-fed products with their partial
    sums, the rotation that adds them up) and the tcgen05 attention: 200 times over, other steps in between, from graphs.
    (This is where a missing proxy fence in the TMA-fed product showed: 54 different logits in 300 runs.)"""
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine, StepEntry
    from pylon_b200.kernels import ops

    folder, _, _ = wide_model
    rng = np.random.default_rng(5)
    ids = rng.integers(0, WIDE_MODEL["vocab_size"], size=tokens).tolist()
    others = [rng.integers(0, WIDE_MODEL["vocab_size"], size=size).tolist() for size in (600, 33, 1)]
    engine = Engine(folder, EngineConfig(dtype="bfloat16", page_size=256, max_cache_tokens=4 * 1_024, max_context=1_024, max_batch_size=4, cuda_graphs=True))
    engine.step_function.graphs.capture_at_once = True
    seen = {}
    for turn in range(200):
        request = engine.open(("short", turn), 1_024)
        logits = engine.step([StepEntry(request, ids, (tokens - 1,))])
        key = logits.cpu().numpy().tobytes()
        seen[key] = seen.get(key, 0) + 1
        engine.close(request)
        if turn % 3 == 0:
            other = engine.open(("other", turn), 1_024)
            engine.step([StepEntry(other, others[turn // 3 % 3], (len(others[turn // 3 % 3]) - 1,))])
            engine.close(other)
    assert len(seen) == 1, f"{len(seen)} different results: {sorted(seen.values(), reverse=True)[:6]}"
    assert ops._error_words(engine.device).tolist() == [0, 0, 0, 0]
