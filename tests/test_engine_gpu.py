"""Generation through the Python entry point and the command line, long decoding, the first
tokens of a sequence, sampling that does not depend on batching."""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import trace_tools
from conftest import TINY_CONFIGS, TINY_PAGE_SIZES, TINY_SEEDS

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

# the requests of the two tiny benchmark configurations
PROMPT_LENGTHS = {"tinyA": (5, 17, 33), "tinyB": (1, 9, 24, 40)}
NEW_TOKENS = {"tinyA": 8, "tinyB": 6}


def prompts_for(name):
    rng = np.random.default_rng(TINY_SEEDS[name])
    return [rng.integers(0, TINY_CONFIGS[name]["vocab_size"], size=n).tolist() for n in PROMPT_LENGTHS[name]]


def engine_for(folder, name, dtype, **options):
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine

    options.setdefault("max_cache_tokens", 1024)
    options.setdefault("max_batch_size", 4)
    return Engine(folder, EngineConfig(dtype=dtype, page_size=TINY_PAGE_SIZES[name], **options))


@pytest.mark.parametrize("name", ["tinyA", "tinyB"])
def test_greedy_generation_in_float32_equals_the_plain_implementation(name, tiny_folders):
    from pylon_b200.sampling import SamplingParams

    cfg, weights = plain.read_model(tiny_folders[name])
    prompts = prompts_for(name)
    expected = [plain.generate_greedy(cfg, weights, prompt, NEW_TOKENS[name]) for prompt in prompts]
    engine = engine_for(tiny_folders[name], name, "float32")
    results = engine.generate(prompts, SamplingParams(max_new_tokens=NEW_TOKENS[name], temperature=0.0))
    assert [r.output_ids for r in results] == expected
    assert all(r.finish_reason == "length" and r.prompt_tokens == len(p) for r, p in zip(results, prompts))
    engine.cache.check()
    assert engine.cache.free_pages() == [g.pool.num_pages for g in engine.cache.groups]
    # a small prefill budget and a small batch cut the same work differently: same tokens
    tight = engine_for(tiny_folders[name], name, "float32", prefill_chunk_size=7, max_batch_size=2)
    assert [r.output_ids for r in tight.generate(prompts, SamplingParams(max_new_tokens=NEW_TOKENS[name], temperature=0.0))] == expected


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["tinyA", "tinyB"])
def test_greedy_generation_in_bfloat16_follows_the_plain_logits(name, graphs, tiny_folders):
    """bfloat16 may flip a near-tie, so the check is on the plain logits of the engine's own
    prefix: every generated token is the plain arg-max or within rounding of it."""
    from pylon_b200.sampling import SamplingParams

    cfg, weights = plain.read_model(tiny_folders[name])
    prompts = prompts_for(name)
    engine = engine_for(tiny_folders[name], name, "bfloat16", cuda_graphs=graphs)
    results = engine.generate(prompts, SamplingParams(max_new_tokens=NEW_TOKENS[name], temperature=0.0))
    for prompt, result in zip(prompts, results):
        assert len(result.output_ids) == NEW_TOKENS[name]
        logits = plain.forward(cfg, weights, prompt + result.output_ids)
        for offset, token in enumerate(result.output_ids):
            row = logits[len(prompt) - 1 + offset]
            assert float(row.max() - row[token]) < 3e-2, (offset, token, int(row.argmax()))


def test_one_call_generate_and_stop_ids(tiny_folders):
    from pylon_b200 import engine as engine_module
    from pylon_b200.config import EngineConfig
    from pylon_b200.sampling import SamplingParams

    name = "tinyB"
    cfg, weights = plain.read_model(tiny_folders[name])
    prompt = prompts_for(name)[2]
    free_run = plain.generate_greedy(cfg, weights, prompt, 6)
    stop = free_run[3]
    first_stop = free_run.index(stop)
    config = EngineConfig(dtype="float32", page_size=8, max_cache_tokens=256, max_batch_size=2)
    results = engine_module.generate(tiny_folders[name], [prompt], SamplingParams(max_new_tokens=6, temperature=0.0, stop_ids=(stop,)), config)
    assert results[0].finish_reason == "eos" and results[0].output_ids == free_run[:first_stop]
    with pytest.raises(ValueError, match="not a token id"):
        engine_module.generate(tiny_folders[name], [[10_000]], SamplingParams(max_new_tokens=1), config)
    with pytest.raises(ValueError, match="set up for requests of up to"):
        engine_module.generate(tiny_folders[name], [[1] * 300], SamplingParams(max_new_tokens=10), config)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["tinyA", "tinyB"])
def test_running_ahead_generates_the_same_tokens(name, graphs, tiny_folders, dtype="float32"):
    """With ``run_ahead`` (the default) a tick queues its step before the host has the tokens of the step before, and the
    decoding requests' tokens are taken on the device; without it every step waits for its tokens.  Greedy requests with a
    stop id that comes up, and seeded draws, under a small prefill budget: the same outputs either way, and the steps
    did take tokens from the device.  (In float32, where logits do not depend on what else is in a step: the two ways
    batch differently, since the host learns of an ending one tick later.  bfloat16 with tokens taken on the device is
    checked against the plain logits by the test above, which runs ahead by default.)"""
    from pylon_b200.sampling import SamplingParams

    prompts = prompts_for(name) * 2
    free_run = engine_for(tiny_folders[name], name, dtype, run_ahead=False).generate(prompts[:1], SamplingParams(max_new_tokens=8, temperature=0.0, ignore_eos=True))
    stop = free_run[0].output_ids[4]
    params = [SamplingParams(max_new_tokens=9, temperature=0.0, stop_ids=(stop,)) if index % 2 == 0 else
              SamplingParams(max_new_tokens=5 + index, temperature=0.8, top_p=0.9, seed=40 + index, ignore_eos=True) for index in range(len(prompts))]
    outcomes = {}
    for run_ahead in (False, True):
        engine = engine_for(tiny_folders[name], name, dtype, run_ahead=run_ahead, cuda_graphs=graphs, prefill_chunk_size=11, max_batch_size=3)
        healthy_step, taken = engine.step_function, []

        class Step:
            def __call__(self, entries):
                taken.append(sum(1 for entry in entries if entry.source is not None))
                return healthy_step(entries)

            def __getattr__(self, attribute):
                return getattr(healthy_step, attribute)

        engine.step_function = Step()
        results = engine.generate(prompts, params)
        outcomes[run_ahead] = [(r.output_ids, r.finish_reason) for r in results]
        assert (sum(taken) > 20) == run_ahead
        engine.cache.check()
        assert engine.cache.free_pages() == [g.pool.num_pages for g in engine.cache.groups]
    assert outcomes[True] == outcomes[False]
    cut = free_run[0].output_ids.index(stop)
    assert outcomes[True][0] == (free_run[0].output_ids[:cut], "eos")


def test_temperature_sampling_does_not_depend_on_batching(tiny_folders):
    """Seeded requests draw the same tokens alone, together, and under a small prefill budget
    (float32, so the logits themselves agree bit for bit)."""
    from pylon_b200.sampling import SamplingParams

    name = "tinyB"
    prompts = prompts_for(name)
    params = [SamplingParams(max_new_tokens=6, temperature=0.8, top_p=0.95, seed=100 + i) for i in range(len(prompts))]
    together = [r.output_ids for r in engine_for(tiny_folders[name], name, "float32").generate(prompts, params)]
    alone = [engine_for(tiny_folders[name], name, "float32").generate([p], [s])[0].output_ids for p, s in zip(prompts, params)]
    tight = [r.output_ids for r in engine_for(tiny_folders[name], name, "float32", prefill_chunk_size=5, max_batch_size=3).generate(prompts, params)]
    assert together == alone == tight
    other_seed = engine_for(tiny_folders[name], name, "float32").generate(prompts[3:], [SamplingParams(max_new_tokens=6, temperature=0.8, seed=999)])
    assert other_seed[0].output_ids != together[3]
    # and the draws follow the plain distribution: temperature 0.8 over a 320-token vocabulary with
    # near-flat logits cannot give six equal tokens
    assert all(len(set(tokens)) > 1 for tokens in together)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sampled_tokens_lie_in_the_plain_nucleus(dtype, tiny_folders):
    from pylon_b200.sampling import SamplingParams

    name = "tinyA"
    cfg, weights = plain.read_model(tiny_folders[name])
    prompts = prompts_for(name)
    engine = engine_for(tiny_folders[name], name, dtype)
    results = engine.generate(prompts, [SamplingParams(max_new_tokens=8, temperature=0.7, top_p=0.6, seed=i) for i in range(3)])
    for prompt, result in zip(prompts, results):
        logits = plain.forward(cfg, weights, prompt + result.output_ids)
        for offset, token in enumerate(result.output_ids):
            probs = plain.sampling_distribution(logits[len(prompt) - 1 + offset], 0.7, 0.6)
            near_edge = plain.sampling_distribution(logits[len(prompt) - 1 + offset], 0.7, 0.63)   # bfloat16 may move the edge a little
            assert probs[token] > 0 or (dtype == "bfloat16" and near_edge[token] > 0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tinyA", "tinyB"])
def test_long_decoding(name, dtype, tiny_folders):
    """A prompt of 20 tokens, then 330 tokens one by one: many pages, many steps."""
    cfg, weights = plain.read_model(tiny_folders[name])
    rng = np.random.default_rng(9)
    tokens = rng.integers(0, TINY_CONFIGS[name]["vocab_size"], size=350).tolist()
    expected = plain.as_numpy(plain.forward(cfg, weights, tokens))
    steps = trace_tools.tail_one_by_one({"long": tokens}, tail=330)
    engine = engine_for(tiny_folders[name], name, dtype, max_cache_tokens=352, max_context=352, cuda_graphs=dtype == "bfloat16")
    got = trace_tools.run_in_process(engine, steps)["long"]
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == "float32" else dict(rtol=3e-2, atol=3e-2)
    np.testing.assert_allclose(got, expected, **tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tinyA", "tinyB"])
def test_first_tokens_of_a_sequence(name, dtype, tiny_folders):
    """Sequences of one, two and three tokens: whole, and token by token, alone and together."""
    cfg, weights = plain.read_model(tiny_folders[name])
    vocab = TINY_CONFIGS[name]["vocab_size"]
    requests = {"one": [vocab - 1], "two": [0, vocab - 1], "three": [5, 5, 5]}
    expected = {rid: plain.as_numpy(plain.forward(cfg, weights, tokens)) for rid, tokens in requests.items()}
    together = [{"step": 0, "entries": [{"id": rid, "tokens": tokens[:1], "want": [0]} for rid, tokens in requests.items()], "end": ["one"]},
                {"step": 1, "entries": [{"id": rid, "tokens": requests[rid][1:2], "want": [0]} for rid in ("two", "three")], "end": ["two"]},
                {"step": 2, "entries": [{"id": "three", "tokens": requests["three"][2:], "want": [0]}], "end": ["three"]}]
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)
    for steps in (trace_tools.whole(requests), trace_tools.tail_one_by_one(requests), together):
        got = trace_tools.run_in_process(engine_for(tiny_folders[name], name, dtype, max_cache_tokens=64), steps)
        for rid in requests:
            np.testing.assert_allclose(got[rid], expected[rid], err_msg=rid, **tol)


def test_graphs_can_be_captured_ahead_of_use(tiny_folders):
    from pylon_b200.sampling import SamplingParams

    name = "tinyA"
    engine = engine_for(tiny_folders[name], name, "bfloat16", cuda_graphs=True)
    assert engine.capture_decode_graphs([1, 2, 3]) == [1, 2, 3]
    engine.cache.check()
    assert engine.cache.free_slots() == 4 and engine.cache.free_pages() == [g.pool.num_pages for g in engine.cache.groups]
    graphs = engine.step_function.graphs
    # both forms of a step: for requests of about equal length (every size) and for any lengths (from two requests on)
    assert sorted(graphs.captured_alike) == [1, 2, 3] and sorted(graphs.captured) == [2, 3]
    before, before_alike = dict(graphs.captured), dict(graphs.captured_alike)
    results = engine.generate(prompts_for(name), SamplingParams(max_new_tokens=4, temperature=0.0))
    assert all(len(r.output_ids) == 4 for r in results)
    assert all(graphs.captured[size] is graph for size, graph in before.items())               # reused, not recaptured
    assert all(graphs.captured_alike[size] is graph for size, graph in before_alike.items())
    with pytest.raises(RuntimeError, match="cuda_graphs"):
        engine_for(tiny_folders[name], name, "bfloat16").capture_decode_graphs([1])


def test_a_decode_step_replays_the_graph_that_fits_its_lengths(tiny_folders):
    """Two requests of equal length decode from the graph captured for such steps, two of very
    different lengths from the other one; the tokens are those of eager steps either way."""
    from pylon_b200.sampling import SamplingParams

    name = "tinyC"
    rng = np.random.default_rng(3)
    vocab = TINY_CONFIGS[name]["vocab_size"]
    greedy = SamplingParams(max_new_tokens=5, temperature=0.0, ignore_eos=True)
    equal = [rng.integers(0, vocab, size=40).tolist() for _ in range(2)]
    ragged = [rng.integers(0, vocab, size=n).tolist() for n in (150, 9)]
    plain_engine = engine_for(tiny_folders[name], name, "bfloat16")
    engine = engine_for(tiny_folders[name], name, "bfloat16", cuda_graphs=True)
    graphs = engine.step_function.graphs
    got = engine.generate(equal, [greedy] * 2)
    assert sorted(graphs.captured_alike) == [2] and not graphs.captured
    assert [r.output_ids for r in got] == [r.output_ids for r in plain_engine.generate(equal, [greedy] * 2)]
    got = engine.generate(ragged, [greedy] * 2)
    assert sorted(graphs.captured) == [2] and not graphs.failed
    assert [r.output_ids for r in got] == [r.output_ids for r in plain_engine.generate(ragged, [greedy] * 2)]


def test_a_void_step_fails_its_requests_and_the_engine_goes_on(tiny_folders):
    """A kernel that gives up a bounded wait leaves its error word set and its step's result void.  The engine looks at
    the words before it accepts a step's tokens: the requests of that step fail with the kernel error and give back what
    they held; requests that come afterwards run as if nothing had happened.  (The word is set from the host, right after a
    step's kernels are queued: no kernel is made to give up.)"""
    from pylon_b200.kernels import ops
    from pylon_b200.sampling import SamplingParams

    name = "tinyB"
    cfg, weights = plain.read_model(tiny_folders[name])
    prompts = prompts_for(name)[:2]
    engine = engine_for(tiny_folders[name], name, "float32")
    greedy = SamplingParams(max_new_tokens=5, temperature=0.0, ignore_eos=True)
    healthy_step, calls = engine.step_function, []

    class Step:
        """The engine's step function, after whose second sampled step the attention's error word and counters look as
        a kernel that gave up would have left them."""

        def __call__(self, entries):
            logits = healthy_step(entries)
            calls.append(len(entries))
            if len(calls) == 2:
                ops.attention_error_word(engine.device).fill_(1)
                ops._zeroed_counters(engine.device, "attention", 8)[:8] = 3
            return logits

        def __getattr__(self, name):
            return getattr(healthy_step, name)

    engine.step_function = Step()
    for prompt in prompts:
        engine.submit(prompt, greedy)
    results = []
    while engine.scheduler.has_work():
        results += engine.tick()
    assert len(results) == 2 and all(result.finish_reason == "error" and isinstance(result.error, ops.KernelError) for result in results)
    assert all(len(result.output_ids) == 1 for result in results)       # the first step's token was accepted, the void step's was not
    engine.cache.check()
    assert engine.cache.free_pages() == [g.pool.num_pages for g in engine.cache.groups] and engine.cache.free_slots() == 4
    assert int(ops._zeroed_counters(engine.device, "attention", 8).abs().sum().item()) == 0
    engine.step_function = healthy_step
    again = engine.generate(prompts, greedy)
    assert [r.output_ids for r in again] == [plain.generate_greedy(cfg, weights, prompt, 5) for prompt in prompts]


def test_command_line(tiny_folders, tmp_path):
    name = "tinyA"
    cfg, weights = plain.read_model(tiny_folders[name])
    prompts = prompts_for(name)
    (tmp_path / "prompts.json").write_text(json.dumps(prompts))
    command = [sys.executable, str(ROOT / "main.py"), "--model", str(tiny_folders[name]), "--dtype", "float32", "--prompt-ids",
               str(tmp_path / "prompts.json"), "--max-new-tokens", "8", "--temperature", "0", "--page-size", "16",
               "--max-cache-tokens", "512", "--max-batch-size", "2", "--prefill-chunk-size", "16"]
    done = subprocess.run(command, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    lines = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    assert [line["output_ids"] for line in lines] == [plain.generate_greedy(cfg, weights, p, 8) for p in prompts]
    assert all(line["finish_reason"] == "length" for line in lines)
    # random-weights mode from a config file, through the same command
    (tmp_path / "config.json").write_text((tiny_folders[name] / "config.json").read_text())
    done = subprocess.run([sys.executable, str(ROOT / "main.py"), "--random-weights", str(tmp_path / "config.json"), "--seed", "0",
                           "--dtype", "float32", "--prompt-ids", str(tmp_path / "prompts.json"), "--max-new-tokens", "8", "--temperature", "0",
                           "--page-size", "16", "--max-cache-tokens", "512"], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    again = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    assert [line["output_ids"] for line in again] == [line["output_ids"] for line in lines]   # seed 0 is the fixture's seed


def test_smoke_entry():
    import __graft_entry__

    __graft_entry__.smoke()
