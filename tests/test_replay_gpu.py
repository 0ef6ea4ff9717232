"""Replay on the GPU: the same requests cut in every way give the plain implementation's
logits, in true 32-bit and in bfloat16."""
from __future__ import annotations

import numpy as np
import pytest

import plain_qwen3 as plain
import trace_tools
from conftest import TINY_CONFIGS, TINY_PAGE_SIZES

pytestmark = pytest.mark.gpu

REQUEST_LENGTHS = {"tinyA": (70, 45, 133, 8, 96, 33), "tinyB": (40, 131, 64, 9, 77, 24, 1), "tinyC": (150, 70, 201, 9, 64, 130)}
TOLERANCE = {"float32": dict(rtol=1e-4, atol=1e-5), "bfloat16": dict(rtol=2e-2, atol=2e-2)}


def make_requests(name: str) -> dict[str, list[int]]:
    rng = np.random.default_rng(100 + len(name) + TINY_CONFIGS[name]["vocab_size"])
    vocab = TINY_CONFIGS[name]["vocab_size"]
    return {f"r{i}": rng.integers(0, vocab, size=n).tolist() for i, n in enumerate(REQUEST_LENGTHS[name])}


@pytest.fixture(scope="module")
def expected(tiny_folders):
    """name -> request -> float64 logits of the plain implementation at every position."""
    out = {}
    for name, folder in tiny_folders.items():
        cfg, weights = plain.read_model(folder)
        out[name] = {rid: plain.as_numpy(plain.forward(cfg, weights, tokens)) for rid, tokens in make_requests(name).items()}
    return out


def make_engine(folder, name, dtype, steps, max_requests=4, cuda_graphs=False):
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine

    page = TINY_PAGE_SIZES[name]
    tokens = trace_tools.pool_tokens(steps, round_to=page)
    config = EngineConfig(dtype=dtype, page_size=page, max_cache_tokens=tokens, max_context=256, max_batch_size=max_requests,
                          cuda_graphs=cuda_graphs)
    return Engine(folder, config)


def compare(got, want, dtype):
    assert set(got) == set(want)
    for rid in want:
        assert got[rid].shape == want[rid].shape, rid
        np.testing.assert_allclose(got[rid], want[rid], err_msg=f"request {rid}", **TOLERANCE[dtype])


CUTTINGS = {
    "whole": trace_tools.whole,
    "tail_one_by_one": trace_tools.tail_one_by_one,
    "changing_portions": trace_tools.changing_portions,
    "mixed": trace_tools.mixed,
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", list(CUTTINGS))
@pytest.mark.parametrize("name", ["tinyA", "tinyB", "tinyC"])
def test_cuttings_match_plain(name, cutting, dtype, tiny_folders, expected):
    requests = make_requests(name)
    steps = CUTTINGS[cutting](requests)
    engine = make_engine(tiny_folders[name], name, dtype, steps)
    got = trace_tools.run_in_process(engine, steps)
    compare(got, expected[name], dtype)
    pool = engine.cache.groups[0].pool
    assert pool.free_count == pool.num_pages            # everything was given back
    assert pool.acquired_total > pool.num_pages          # and pages were used again


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["tail_one_by_one", "mixed"])
@pytest.mark.parametrize("name", ["tinyA", "tinyB", "tinyC"])
def test_decode_steps_replayed_from_cuda_graphs(name, cutting, dtype, tiny_folders, expected):
    """With graphs on, steps of single tokens come from captured graphs (one per batch size);
    the logits must be the same as without."""
    requests = make_requests(name)
    steps = CUTTINGS[cutting](requests)
    engine = make_engine(tiny_folders[name], name, dtype, steps, cuda_graphs=True)
    got = trace_tools.run_in_process(engine, steps)
    compare(got, expected[name], dtype)
    graphs = engine.step_function.graphs
    assert (graphs.captured or graphs.captured_alike) and not graphs.failed


@pytest.mark.parametrize("dtype, seed", [("float32", 7), ("bfloat16", 7), ("bfloat16", 8), ("bfloat16", 9)])
@pytest.mark.parametrize("name", ["tinyA", "tinyB", "tinyC"])
def test_steps_with_portions_replayed_from_padded_graphs(name, dtype, seed, tiny_folders, expected):
    """Steps as a scheduler makes them (logits wanted at the last token of an entry, or nowhere) that bring prompt
    portions are padded to a captured size and replayed from its graph: rows without tokens, tokens without a row.  The
    logits must be the plain implementation's, and the same sizes must come from the same graph again."""
    from pylon_b200.engine import StepEntry

    requests = make_requests(name)
    steps = trace_tools.mixed(requests, seed=seed, max_portion=40 if seed == 7 else 90)
    engine = make_engine(tiny_folders[name], name, dtype, steps, cuda_graphs=True)
    graphs = engine.step_function.graphs
    at_once = name != "tinyC"
    graphs.capture_at_once = at_once    # a size is captured when it comes up (else: when it comes back), so that more steps are replays
    live, cursor = {}, {rid: 0 for rid in requests}
    for number, step in enumerate(steps):
        entries, places = [], []
        for item in step["entries"]:
            rid, count = item["id"], len(item["tokens"])
            if rid not in live:
                live[rid] = engine.open(rid, engine.max_context)
            wants = number % 3 != 0 or count == 1     # every third step, portions ask for nothing
            entries.append(StepEntry(live[rid], item["tokens"], (count - 1,) if wants else ()))
            if wants:
                places.append((rid, cursor[rid] + count - 1))
            cursor[rid] += count
        logits = engine.step(entries)
        assert (logits is None) == (not places)
        if places:
            got = logits.float().cpu().numpy()
            assert got.shape[0] == len(places)
            for row, (rid, position) in enumerate(places):
                np.testing.assert_allclose(got[row], expected[name][rid][position], err_msg=f"step {number} {rid} position {position}", **TOLERANCE[dtype])
        for rid in step["end"]:
            engine.close(live.pop(rid))
    engine.cache.check()
    assert graphs.replays["padded"] > ((10 if at_once else 3) if seed == 7 else 0) and not graphs.failed
    if seed == 7:
        assert graphs.replays["decode"] > 0
        assert len(graphs.captured_padded) < graphs.replays["padded"]    # sizes came back and were replayed, not captured again
    if not at_once:
        assert all(count >= 2 for key, count in graphs.seen_padded.items() if key in graphs.captured_padded)


@pytest.mark.parametrize("name", ["tinyA", "tinyB"])
def test_cuttings_agree_with_each_other_in_float32(name, tiny_folders):
    """Beyond agreeing with the oracle: in 32-bit the cuttings agree with each other far
    below the oracle tolerance, so a fault that depends on the cut shows even where it is
    smaller than float32-vs-float64 noise."""
    requests = make_requests(name)
    results = {}
    for cutting, build in CUTTINGS.items():
        steps = build(requests)
        results[cutting] = trace_tools.run_in_process(make_engine(tiny_folders[name], name, "float32", steps), steps)
    for cutting, got in results.items():
        for rid in requests:
            np.testing.assert_allclose(got[rid], results["whole"][rid], rtol=0, atol=2e-6, err_msg=f"{cutting} {rid}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, tiny_folders, expected, tmp_path):
    """The bin/trace_run program itself, in a process of its own, on a mixed trace."""
    name = "tinyB"
    requests = make_requests(name)
    steps = trace_tools.mixed(requests, seed=3)
    got = trace_tools.run_program(tiny_folders[name], dtype, steps, tmp_path / "out")
    compare(got, expected[name], dtype)
