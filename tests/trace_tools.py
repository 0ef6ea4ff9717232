"""Builds replay traces (the JSON steps ``bin/trace_run`` reads) and runs them.

A trace is a list of steps ``{"step", "entries": [{"id", "tokens", "want"}], "end"}``.
The builders below cut the same requests in different ways; every builder asks for the
logits of every position, so that the results of all cuttings can be compared position by
position with the plain implementation.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path
from typing import Iterable, Optional, Sequence

import numpy as np

ROOT = Path(__file__).resolve().parent.parent


# ---------------------------------------------------------------------------------------
# cuttings
# ---------------------------------------------------------------------------------------
def whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone, in one step."""
    steps = []
    for name, tokens in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": name, "tokens": tokens, "want": list(range(len(tokens)))}], "end": [name]})
    return steps


def tail_one_by_one(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of each request in one step, its last ``tail`` tokens one step each."""
    steps = []
    for name, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        pieces = [tokens[:head]] + [[t] for t in tokens[head:]]
        for number, piece in enumerate(pieces):
            steps.append({
                "step": len(steps),
                "entries": [{"id": name, "tokens": piece, "want": list(range(len(piece)))}],
                "end": [name] if number == len(pieces) - 1 else [],
            })
    return steps


def changing_portions(requests: dict[str, list[int]], sizes: Sequence[int] = (7, 2, 5, 3, 2, 11, 2, 4, 16, 2, 9)) -> list[dict]:
    """Each request alone in portions of changing size, down to two tokens."""
    steps = []
    for name, tokens in requests.items():
        cursor, turn = 0, 0
        while cursor < len(tokens):
            size = sizes[turn % len(sizes)]
            turn += 1
            if len(tokens) - cursor - size == 1:   # never leave a last portion of one token here
                size += 1
            piece = tokens[cursor : cursor + size]
            cursor += len(piece)
            steps.append({
                "step": len(steps),
                "entries": [{"id": name, "tokens": piece, "want": list(range(len(piece)))}],
                "end": [name] if cursor >= len(tokens) else [],
            })
    return steps


def mixed(requests: dict[str, list[int]], seed: int = 0, max_live: int = 4, decode_tail: int = 12, max_portion: int = 24) -> list[dict]:
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others.

    Each request goes through its first ``len - decode_tail`` tokens in portions of random
    size (2..``max_portion``), then through the rest one token a step; a request is sometimes left out of
    a step; finished requests end and the next one starts, so their pages are used again.
    """
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live: dict[str, dict] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
            name, tokens = waiting.pop(0)
            live[name] = {"tokens": tokens, "cursor": 0}
        entries, ended = [], []
        for name, state in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue   # left out of this step
            tokens, cursor = state["tokens"], state["cursor"]
            remaining = len(tokens) - cursor
            if remaining <= decode_tail:
                size = 1
            else:
                size = int(rng.integers(2, max_portion + 1))
                size = min(size, remaining - decode_tail)
                if size < 2:
                    size = remaining - decode_tail if remaining - decode_tail >= 1 else 1
            piece = tokens[cursor : cursor + size]
            state["cursor"] += len(piece)
            entries.append({"id": name, "tokens": piece, "want": list(range(len(piece)))})
            if state["cursor"] >= len(tokens):
                ended.append(name)
        if not entries:
            continue
        for name in ended:
            del live[name]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def pool_tokens(steps: Iterable[dict], round_to: int = 64) -> int:
    """Most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: dict[str, int] = {}
    most = 0
    for step in steps:
        for entry in step["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        most = max(most, sum(-(-count // round_to) * round_to for count in held.values()))
        for name in step["end"]:
            held.pop(name, None)
    return most


# ---------------------------------------------------------------------------------------
# running
# ---------------------------------------------------------------------------------------
def collect(steps: Sequence[dict], logits_of_step) -> dict[str, np.ndarray]:
    """Per request: float32 ``[tokens, vocab]`` logits put back in position order.
    ``logits_of_step(step)`` returns the ``[wanted, vocab]`` array of one step."""
    rows: dict[str, list[np.ndarray]] = {}
    for step in steps:
        wanted = sum(len(entry["want"]) for entry in step["entries"])
        if not wanted:
            continue
        values = logits_of_step(step)
        assert values.shape[0] == wanted, (values.shape, wanted)
        cursor = 0
        for entry in step["entries"]:
            assert entry["want"] == list(range(len(entry["tokens"]))), "builders here ask for every position"
            rows.setdefault(entry["id"], []).append(values[cursor : cursor + len(entry["want"])])
            cursor += len(entry["want"])
    return {name: np.concatenate(parts, axis=0) for name, parts in rows.items()}


def run_in_process(engine, steps: Sequence[dict]) -> dict[str, np.ndarray]:
    """Replays ``steps`` on an :class:`pylon_b200.engine.Engine` through its step function."""
    import torch

    from pylon_b200.engine import StepEntry

    live = {}

    def one(step):
        entries = []
        for item in step["entries"]:
            if item["id"] not in live:
                live[item["id"]] = engine.open(item["id"], engine.max_context)
            entries.append(StepEntry(live[item["id"]], item["tokens"], item["want"]))
        logits = engine.step(entries)
        for name in step["end"]:
            engine.close(live.pop(name))
        return logits.to(torch.float32).cpu().numpy()

    result = collect(steps, one)
    engine.cache.check()
    return result


def run_program(model_dir: Path, dtype: str, steps: Sequence[dict], out_dir: Path, max_tokens: Optional[int] = None,
                extra_args: Sequence[str] = (), env: Optional[dict] = None) -> dict[str, np.ndarray]:
    """Replays ``steps`` with the ``bin/trace_run`` program in a process of its own."""
    config = json.loads((Path(model_dir) / "config.json").read_text())
    vocab = config["vocab_size"]
    max_tokens = pool_tokens(steps) if max_tokens is None else max_tokens
    command = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
               "--out", str(out_dir), "--max-tokens", str(max_tokens), *extra_args]
    text = "".join(json.dumps(step) + "\n" for step in steps)
    done = subprocess.run(command, input=text, capture_output=True, text=True, env=env, timeout=900)
    assert done.returncode == 0, f"trace_run failed ({done.returncode}):\n{done.stdout[-2000:]}\n{done.stderr[-4000:]}"
    said = [line for line in done.stdout.splitlines() if line.startswith("done ")]
    assert said == [f"done {step['step']}" for step in steps], said[-3:]

    def one(step):
        return np.fromfile(Path(out_dir) / f"{step['step']}.f32", dtype="<f4").reshape(-1, vocab)

    return collect(steps, one)
