"""Decode and prefill throughput of the engine at Qwen3-4B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  A "step" is one decode step of a batch of 8 requests whose caches
hold about 4,096 tokens each (random weights, random token ids; the caches are filled by
real prefill through the engine).  ``value`` is decoded tokens a second timed on the device
over exactly K steps of the step function; ``e2e`` is the same through the public entry
point (``Engine.submit`` / ``Engine.tick``: host token lists in, host token lists out, with
the scheduler, the host-to-device copy of each step's inputs and the device-to-host read of
its tokens inside the timed region; the median of the same R repeats of K ticks, on the host's clock).  ``prefill`` is one 2,048-token prompt in one step;
``roofline`` relates the decode step to HBM bandwidth.  The K timed steps are repeated R times
(``config.repeats``); ``value`` is the median repeat, ``spread`` its lowest and highest, and
``clocks.sm_mhz_per_repeat`` the SM clock sampled during each.  ``points`` holds the other sizes
and workloads: decoding at batch 1 and 64 at the same context; the reference's own decode-heavy
workload (B requests, 128-token prompts, 512 new tokens: B x 511 tokens over the time of the 511
decode steps) at B = 1, 8, 64 with its share of the HBM roofline; the output rate of the two
serving workloads at the 8B and 14B shapes; and a full-depth float32 run at the 14B shape with
its largest logit error against the plain implementation.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for entry in (str(ROOT), str(ROOT / "tests")):   # tests/: the plain implementation, for the float32 check at the 14B shape
    if entry not in sys.path:
        sys.path.insert(0, entry)

QWEN3_4B = dict(
    vocab_size=151_936, hidden_size=2_560, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
    head_dim=128, intermediate_size=9_728, max_position_embeddings=262_144, rope_theta=5_000_000.0,
    rms_norm_eps=1e-6, tie_word_embeddings=True,
)
QWEN3_8B = dict(
    vocab_size=151_936, hidden_size=4_096, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
    head_dim=128, intermediate_size=12_288, max_position_embeddings=40_960, rope_theta=1_000_000.0,
    rms_norm_eps=1e-6, tie_word_embeddings=False,
)
QWEN3_14B = dict(
    vocab_size=151_936, hidden_size=5_120, num_hidden_layers=40, num_attention_heads=40, num_key_value_heads=8,
    head_dim=128, intermediate_size=17_408, max_position_embeddings=40_960, rope_theta=1_000_000.0,
    rms_norm_eps=1e-6, tie_word_embeddings=False,
)
CONTEXT = 4_096
PAGE_SIZE = 256
PREFILL_TOKENS = 2_048
# raun6k/Pylon's published decode_heavy output rate at concurrency 8 (README.md:73): an
# end-to-end HTTP figure on an NVIDIA L4, the only batch-8 number it publishes.
BASELINE_TOKENS_PER_SECOND = 199.8


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            out["hbm_gbs"] = float(data.get("hbm_gbs", out["hbm_gbs"]))
            out["bf16_tflops"] = float(data.get("bf16_tflops", out["bf16_tflops"]))
            out["source"] = "measured"
        except (ValueError, TypeError):
            pass
    return out


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int = 0, interval_ms: int = 100) -> None:
        self.lines: list[str] = []
        self.times: list[float] = []     # time.perf_counter() at which each line arrived
        self.process = None
        self.device_index = device_index
        self.interval_ms = interval_ms

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", str(self.interval_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _read(self) -> None:
        for line in self.process.stdout:
            self.lines.append(line.strip())
            self.times.append(time.perf_counter())

    def __exit__(self, *exc) -> None:
        if self.process is not None:
            time.sleep(0.15)
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()

    def summary(self, begin: float | None = None, end: float | None = None) -> dict:
        """Median SM clock, the highest clock the device offers and the throttle reasons seen, over all samples or over
        those that arrived between two ``time.perf_counter()`` readings."""
        clocks, top, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line, arrived in zip(list(self.lines), list(self.times)):
            if begin is not None and not begin <= arrived <= end:
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(int(float(parts[0])))
                top = max(top, int(float(parts[1])))
            except ValueError:
                continue
            for name, value in zip(names, parts[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": top or None,
                "reasons": sorted(reasons), "samples": len(clocks)}


def fill_caches(engine, torch, batch: int, tokens_each: int, rng, chunk: int):
    """Opens ``batch`` requests and prefills ``tokens_each`` random tokens into each."""
    from pylon_b200.engine import StepEntry

    vocab = engine.spec.vocab_size
    requests = [engine.open(("bench", i, time.time_ns()), CONTEXT) for i in range(batch)]
    for request in requests:
        done = 0
        while done < tokens_each:
            count = min(chunk, tokens_each - done)
            engine.step([StepEntry(request, rng.integers(0, vocab, size=count).tolist(), ())])
            done += count
    torch.cuda.synchronize()
    return requests


class DecodeLoop:
    """Decoding as the engine's scheduler does it when it runs ahead: a step takes its tokens on the device from what the
    sampling kernel chose in the step before, it is queued behind that step, and only then are that step's tokens read
    back to the host.  Every step's tokens do come back, one step late; ``tokens`` are the latest that have."""

    def __init__(self, engine, requests, tokens: list[int]) -> None:
        from pylon_b200.sampling.sampler import Sampler

        self.engine, self.requests, self.tokens = engine, requests, tokens
        self.sampler = Sampler(engine.device)
        self.flying = None
        self.greedy = None

    def step(self) -> None:
        from pylon_b200.engine import StepEntry
        from pylon_b200.sampling import SamplingParams

        if self.greedy is None:
            self.greedy = [SamplingParams(temperature=0.0)] * len(self.requests)
        if self.flying is None or not self.engine.config.run_ahead:
            entries = [StepEntry(request, [token], (0,)) for request, token in zip(self.requests, self.tokens)]
        else:
            entries = [StepEntry(request, [0], (0,), (self.flying.device, row)) for row, request in enumerate(self.requests)]
        launched = self.sampler.launch(self.engine.step(entries), self.greedy, [None] * len(self.requests))
        if self.flying is not None:
            self.tokens = self.flying.result()
        self.flying = launched
        if not self.engine.config.run_ahead:
            self.finish()

    def finish(self) -> list[int]:
        if self.flying is not None:
            self.tokens, self.flying = self.flying.result(), None
        return self.tokens


def time_decode(engine, torch, ops, batch: int, steps: int, warmup: int, rng, repeats: int = 1) -> dict:
    """Decode ``warmup + repeats * steps`` tokens for ``batch`` requests whose contexts end at CONTEXT; each repeat's K
    steps are bracketed by CUDA events on the launching stream.  The figures returned are those of the median repeat."""
    from pylon_b200.engine import StepEntry

    start_length = CONTEXT - (warmup + repeats * steps)
    requests = fill_caches(engine, torch, batch, start_length, rng, PREFILL_TOKENS)
    tokens = rng.integers(0, engine.spec.vocab_size, size=batch).tolist()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(repeats)]
    windows, launches, kv_tokens = [], [], []
    loop = DecodeLoop(engine, requests, tokens)
    for _ in range(warmup):
        loop.step()
    for begin, end in events:
        loop.finish()
        torch.cuda.synchronize()
        before, held = ops.launches[0], 0
        started = time.perf_counter()
        begin.record()
        for _ in range(steps):
            held += sum(request.length + 1 for request in requests)
            loop.step()
        loop.finish()   # the last step's tokens are back on the host inside the timed region
        end.record()
        torch.cuda.synchronize()
        windows.append((started, time.perf_counter()))
        launches.append(ops.launches[0] - before)
        kv_tokens.append(held / steps)
    for request in requests:
        engine.close(request)
    milliseconds = [begin.elapsed_time(end) for begin, end in events]
    middle = sorted(range(repeats), key=lambda index: milliseconds[index])[repeats // 2]
    return {"ms_per_step": milliseconds[middle] / steps, "tokens_per_second": batch * steps / (milliseconds[middle] / 1e3),
            "launches": launches[middle], "kv_tokens_per_step": kv_tokens[middle], "windows": windows,
            "per_repeat": [batch * steps / (ms / 1e3) for ms in milliseconds]}


def time_decode_heavy(engine, torch, ops, batch: int, rng, prompt_tokens: int = 128, new_tokens: int = 512) -> dict:
    """raun6k/Pylon's decode-heavy workload at the step level (README.md:64-74: 128-token prompts, 512 new tokens):
    ``batch`` requests are prefilled, the first token of each comes with the prompt, and the other 511 are decoded in
    511 steps timed as one region with CUDA events: tokens a second = batch x 511 / that time."""
    from pylon_b200.engine import StepEntry

    vocab = engine.spec.vocab_size
    requests = [engine.open(("heavy", batch, index), prompt_tokens + new_tokens) for index in range(batch)]
    logits = None
    for start in range(0, batch, 16):
        group = requests[start : start + 16]
        part = engine.step([StepEntry(request, rng.integers(0, vocab, size=prompt_tokens).tolist(), (prompt_tokens - 1,)) for request in group])
        logits = part if logits is None else torch.cat((logits, part))
    loop = DecodeLoop(engine, requests, ops.sample(logits).cpu().tolist())
    for _ in range(3):    # the first steps of a size capture its graph and warm up; they count as generated tokens all the same
        loop.step()
    loop.finish()
    steps = new_tokens - 1 - 3
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record()
    held = 0
    for _ in range(steps):
        held += sum(request.length + 1 for request in requests)
        loop.step()
    loop.finish()
    end.record()
    torch.cuda.synchronize()
    seconds = begin.elapsed_time(end) / 1e3
    for request in requests:
        engine.close(request)
    bytes_per_step = engine.model.weight_bytes() + held / steps * engine.cache.bytes_per_token()
    return {"tokens_per_second": batch * steps / seconds, "gbs": bytes_per_step / (seconds / steps) / 1e9}


def float32_14b_check(torch) -> dict:
    """The Qwen3-14B shape at its full depth in true 32-bit: 16 requests of 64-token prompts generate 16 tokens each
    through the engine (output tokens a second, prompts included in the time), and the logits of one 64-token request
    at every position are compared with the plain implementation in float64, which draws the same weights tensor by
    tensor (59 GB of float32 weights are on the device; the plain implementation holds one matrix at a time)."""
    import numpy as np

    import plain_qwen3 as plain
    from pylon_b200.config import EngineConfig, Qwen3Config
    from pylon_b200.engine import Engine, StepEntry
    from pylon_b200.sampling import SamplingParams
    from pylon_b200.weights.random_init import device_random_fetch

    fields = QWEN3_14B
    rng = np.random.default_rng(7)
    requests, prompt_tokens, new_tokens = 16, 64, 16
    config = EngineConfig(dtype="float32", page_size=PAGE_SIZE, max_cache_tokens=(requests + 1) * PAGE_SIZE, max_context=PAGE_SIZE,
                          max_batch_size=requests, max_queue_size=requests, prefill_chunk_size=PREFILL_TOKENS)
    engine = Engine(None, config, device="cuda:0", model_config=Qwen3Config(**fields), random_seed=0)
    prompts = [rng.integers(0, fields["vocab_size"], size=prompt_tokens).tolist() for _ in range(requests)]
    engine.generate(prompts[:1], SamplingParams(max_new_tokens=2, temperature=0.0, ignore_eos=True))   # warm up
    torch.cuda.synchronize()
    started = time.perf_counter()
    results = engine.generate(prompts, SamplingParams(max_new_tokens=new_tokens, temperature=0.0, ignore_eos=True))
    torch.cuda.synchronize()
    seconds = time.perf_counter() - started
    assert all(len(result.output_ids) == new_tokens and result.error is None for result in results)
    request = engine.open("check", prompt_tokens)
    logits = engine.step([StepEntry(request, prompts[0], tuple(range(prompt_tokens)))]).double()
    engine.close(request)

    fetch = device_random_fetch(engine.model.tensor_decls(), 0, engine.device, torch.float32)

    class DrawnOnDemand(dict):
        def __missing__(self, name):
            return fetch(name).double()

    cfg = dict(Qwen3Config(**fields).to_dict())
    with torch.no_grad():
        expected = plain.forward(cfg, DrawnOnDemand({"model.embed_tokens.weight": fetch("model.embed_tokens.weight").double()}), prompts[0])
    error = float((logits - expected).abs().max())
    agree = float((logits.argmax(-1) == expected.argmax(-1)).double().mean())
    del engine
    torch.cuda.empty_cache()
    return {"tokens_per_second": requests * new_tokens / seconds, "max_abs_logit_error": error, "argmax_agreement": agree,
            "logit_spread": float(expected.std())}


def time_e2e(engine, torch, batch: int, steps: int, warmup: int, rng, repeats: int = 1) -> dict:
    """The same decode through submit()/tick(): host tokens in, host tokens out.  Prompts are
    sized so that every request is still decoding when the timed ticks end (requests finish
    their prompts at different ticks), and the value counts the tokens the ticks returned.  The K
    timed ticks are repeated ``repeats`` times, each between synchronisations and on the host's clock;
    the value is that of the median repeat (56 ms of ticks by themselves gave figures 2 % apart)."""
    from pylon_b200.engine.step import StepLayout
    from pylon_b200.sampling import SamplingParams

    vocab = engine.spec.vocab_size
    prompt_ticks = batch * -(-CONTEXT // PREFILL_TOKENS)          # ticks until the last prompt is in
    new_tokens = warmup + repeats * steps + prompt_ticks + 8
    prompt_length = CONTEXT - new_tokens
    params = SamplingParams(max_new_tokens=new_tokens, temperature=0.0, ignore_eos=True)
    for _ in range(batch):
        engine.submit(rng.integers(0, vocab, size=prompt_length).tolist(), params)
    scheduler = engine.scheduler
    while any(r.prefilling for r in scheduler.active) or scheduler.waiting or len(scheduler.active) < batch:
        engine.tick()
    for _ in range(warmup):
        engine.tick()
    rates = []
    for _ in range(repeats):
        torch.cuda.synchronize()
        before = sum(len(r.output_ids) for r in scheduler.active)
        started = time.perf_counter()
        finished = []
        for _ in range(steps):
            finished += engine.tick()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - started
        produced = sum(len(r.output_ids) for r in scheduler.active) + sum(len(f.output_ids) for f in finished) - before
        assert not finished and produced == batch * steps, (len(finished), produced)
        rates.append(produced / seconds)
    while scheduler.has_work():
        engine.tick()
    # per step: the packed int32 metadata buffer goes up; one int32 token per request and the kernels' four error words come back
    layout = StepLayout(tokens=batch, rows=batch, logits=batch, table_widths=(CONTEXT // PAGE_SIZE,))
    return {"value": sorted(rates)[len(rates) // 2], "unit": "tokens/s", "h2d_bytes_per_step": layout.total * 4, "d2h_bytes_per_step": batch * 4 + 16,
            "spread": [round(min(rates), 1), round(max(rates), 1)]}


def time_prefill(engine, torch, repeats: int, rng) -> dict:
    from pylon_b200.engine import StepEntry

    vocab = engine.spec.vocab_size
    best = None
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for index in range(repeats):
        request = engine.open(("prefill", index), PREFILL_TOKENS)
        tokens = rng.integers(0, vocab, size=PREFILL_TOKENS).tolist()
        torch.cuda.synchronize()
        begin.record()
        engine.step([StepEntry(request, tokens, (PREFILL_TOKENS - 1,))])
        end.record()
        torch.cuda.synchronize()
        engine.close(request)
        elapsed = begin.elapsed_time(end)
        if index >= 2:   # the first runs warm up
            best = elapsed if best is None else min(best, elapsed)
    return {"ms": best}


def profile_steps(engine, torch, ops, kind: str, batch: int, rng, prompt_tokens: int = PREFILL_TOKENS, context: int = CONTEXT) -> None:
    """Warm up, then run two steps of ``kind`` inside the profiler's range (eagerly, so that a
    profiler sees every kernel as its own launch)."""
    from pylon_b200.engine import StepEntry

    vocab = engine.spec.vocab_size
    if kind == "decode":
        requests = fill_caches(engine, torch, batch, context - 8, rng, PREFILL_TOKENS)
        tokens = [1] * batch

        def step():
            nonlocal tokens
            logits = engine.step([StepEntry(request, [token], (0,)) for request, token in zip(requests, tokens)])
            tokens = ops.sample(logits).cpu().tolist()
    else:
        counter = [0]

        def step():
            request = engine.open(("profile", counter[0]), prompt_tokens)
            counter[0] += 1
            engine.step([StepEntry(request, rng.integers(0, vocab, size=prompt_tokens).tolist(), (prompt_tokens - 1,))])
            torch.cuda.synchronize()
            engine.close(request)
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    for _ in range(2):
        step()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    print(f"profiled 2 {kind} steps: {engine.spec.order.__len__()} layers, batch {batch}, context {context}, prompt of {prompt_tokens} tokens")


def run_serving_workload(name: str, torch) -> dict:
    """The two serving workloads beside the headline one, through submit()/tick() from the first
    request to the last token:

    ``mixed8b``     Qwen3-8B shape, 64 requests with 2,048-token prompts and 128 new tokens each, greedy, batch 64,
                    prefill portions of 2,048 tokens beside the decoding requests (continuous batching)
    ``sampled14b``  Qwen3-14B shape, 16 requests with prompt lengths uniform in [64, 4096] and 256 new tokens each,
                    temperature 0.7 with a fixed seed
    """
    import numpy as np

    from pylon_b200.config import EngineConfig, Qwen3Config
    from pylon_b200.engine import Engine
    from pylon_b200.sampling import SamplingParams

    rng = np.random.default_rng(0)
    if name == "mixed8b":
        fields, requests, new_tokens = QWEN3_8B, 64, 128
        lengths = [2_048] * requests
        params = [SamplingParams(max_new_tokens=new_tokens, temperature=0.0, ignore_eos=True)] * requests
    else:
        fields, requests, new_tokens = QWEN3_14B, 16, 256
        lengths = rng.integers(64, 4_097, size=requests).tolist()
        params = [SamplingParams(max_new_tokens=new_tokens, temperature=0.7, top_p=1.0, seed=1_000 + i, ignore_eos=True) for i in range(requests)]
    longest = max(lengths) + new_tokens
    config = EngineConfig(
        dtype="bfloat16", page_size=PAGE_SIZE, max_cache_tokens=requests * (-(-longest // PAGE_SIZE) * PAGE_SIZE), max_context=longest,
        max_batch_size=requests, max_queue_size=requests, prefill_chunk_size=PREFILL_TOKENS, cuda_graphs=True,
    )
    engine = Engine(None, config, device="cuda:0", model_config=Qwen3Config(**fields), random_seed=0)
    prompts = [rng.integers(0, fields["vocab_size"], size=n).tolist() for n in lengths]
    engine.generate(prompts[:2], [SamplingParams(max_new_tokens=4, temperature=0.0, ignore_eos=True)] * 2)   # warm up: libraries, allocator
    # The decode graph of every batch size is captured before the first request, as raun6k/Pylon does when it starts
    # (src/pylon/engine.py:823-836); otherwise each size's first step pays for its capture (about 20 ms).
    captured = engine.capture_decode_graphs()
    # ... and the graphs of the ticks that bring a prompt portion beside 0 to 63 decoding requests
    engine.capture_padded_graphs([(ones, 1, min(PREFILL_TOKENS, max(lengths))) for ones in (0, 1, 2, 4, 8, 16, 32, 64)[: 1 + requests.bit_length()]])
    torch.cuda.synchronize()
    started = time.perf_counter()
    for prompt, sampling in zip(prompts, params):
        engine.submit(prompt, sampling)
    ticks = mixed_ticks = 0
    results = []
    scheduler = engine.scheduler
    while scheduler.has_work():
        results += engine.tick()
        ticks += 1
        mixed_ticks += any(count > 1 for _, count in scheduler.last_step)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - started
    produced = sum(len(r.output_ids) for r in results)
    assert len(results) == requests and produced == requests * new_tokens and all(r.error is None for r in results)
    first_token = sorted(r.first_token_seconds for r in results)
    return {
        "metric": f"output tokens/s, {name}", "value": round(produced / seconds, 1), "unit": "tokens/s", "n_gpus": 1,
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "seconds": round(seconds, 3), "prompt_tokens": int(sum(lengths)), "output_tokens": produced,
        "all_tokens_per_second": round((sum(lengths) + produced) / seconds, 1), "ticks": ticks, "ticks_with_prompt_portions": mixed_ticks,
        "first_token_seconds_median": round(first_token[len(first_token) // 2], 4),
        "config": {"model": "Qwen3-8B shape" if name == "mixed8b" else "Qwen3-14B shape", "layers": fields["num_hidden_layers"],
                   "hidden": fields["hidden_size"], "q_heads": fields["num_attention_heads"], "kv_heads": fields["num_key_value_heads"],
                   "head_dim": fields["head_dim"], "intermediate": fields["intermediate_size"], "vocab": fields["vocab_size"],
                   "requests": requests, "new_tokens": new_tokens, "page_size": PAGE_SIZE, "prefill_chunk": PREFILL_TOKENS,
                   "temperature": params[0].temperature, "cuda_graphs": True, "graphs_captured_at_start": len(captured)},
    }


def prefill_flops(cfg: dict, tokens: int) -> float:
    h, q, kv, inter = cfg["hidden_size"], cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"], cfg["intermediate_size"]
    per_layer = 2 * tokens * (h * (q + 2 * kv) + q * h + 3 * h * inter)
    attention = 2 * 2 * cfg["num_attention_heads"] * cfg["head_dim"] * tokens * (tokens + 1) / 2   # causal half of QK^T and PV
    head = 2 * cfg["vocab_size"] * h   # one row
    return cfg["num_hidden_layers"] * (per_layer + attention) + head


METRIC = "decode tokens/s, Qwen3-4B shape, batch 8, context 4096"


REPEATS = 5


def headline_config(layers: int, batch: int, cuda_graphs: bool, peak_source: str, run_ahead: bool = True) -> dict:
    fields = QWEN3_4B
    return {
        "model": "Qwen3-4B shape", "layers": layers, "layers_of_model": fields["num_hidden_layers"],
        "hidden": fields["hidden_size"], "q_heads": fields["num_attention_heads"], "kv_heads": fields["num_key_value_heads"],
        "head_dim": fields["head_dim"], "intermediate": fields["intermediate_size"], "vocab": fields["vocab_size"],
        "global_batch": batch, "seq_len": CONTEXT, "page_size": PAGE_SIZE, "prefill_tokens": PREFILL_TOKENS,
        "parallelism": "single GPU", "cuda_graphs": cuda_graphs, "run_ahead": run_ahead, "repeats": REPEATS, "l2": "inputs larger than L2 (8 GB of weights per step)",
        "peaks": peak_source, "baseline": "Pylon README decode_heavy c=8 on L4 (HTTP end to end)",
    }


def run_reference_arm(args) -> int:
    """raun6k/Pylon itself on the same workload: see baseline/reference_arm.py."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("reference_arm", ROOT / "baseline" / "reference_arm.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    peak = peaks()
    shared = {
        "context": CONTEXT, "page_size": PAGE_SIZE, "prefill_tokens": PREFILL_TOKENS, "clock_sampler": ClockSampler, "peaks": peak,
        "prefill_flops": lambda tokens: prefill_flops(QWEN3_4B, tokens), "metric": METRIC,
        "baseline_tokens_per_second": BASELINE_TOKENS_PER_SECOND,
        "config": headline_config(QWEN3_4B["num_hidden_layers"], args.batch, True, peak["source"], run_ahead=False),   # the reference waits for every step's tokens
    }
    return module.run(args, shared)


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="pylon_b200", choices=["pylon_b200", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=QWEN3_4B["num_hidden_layers"],
                        help="run fewer layers than the configuration has (named in the output)")
    parser.add_argument("--skip-points", action="store_true", help="leave out the batch 1 and 64 points")
    parser.add_argument("--workload", choices=["decode4b", "mixed8b", "sampled14b"], default="decode4b",
                        help="decode4b: the headline measurement (default); the others are the serving workloads of the 8B and 14B shapes")
    parser.add_argument("--profile", choices=["decode", "prefill"],
                        help="no measurement: run a few steps of this kind between cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    parser.add_argument("--profile-tokens", type=int, default=PREFILL_TOKENS, help="with --profile prefill: tokens of the prompt")
    parser.add_argument("--profile-context", type=int, default=CONTEXT, help="with --profile decode: tokens each request holds")
    args = parser.parse_args()

    if args.impl == "reference":
        return run_reference_arm(args)
    if args.gpus != 1:
        print("bench.py measures a single-GPU engine; --gpus must be 1")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch

    from pylon_b200.config import EngineConfig, Qwen3Config
    from pylon_b200.engine import Engine
    from pylon_b200.kernels import ops

    if args.workload != "decode4b":
        print(json.dumps(run_serving_workload(args.workload, torch)))
        return 0
    fields = dict(QWEN3_4B, num_hidden_layers=args.layers)
    model_config = Qwen3Config(**fields)
    rng = np.random.default_rng(0)
    largest = args.batch if args.skip_points else max(args.batch, 64)
    engine_config = EngineConfig(
        dtype="bfloat16", page_size=PAGE_SIZE, max_cache_tokens=largest * CONTEXT, max_context=CONTEXT,
        max_batch_size=largest, max_queue_size=largest, prefill_chunk_size=PREFILL_TOKENS,
        cuda_graphs=os.environ.get("PYLON_CUDA_GRAPHS", "true").lower() in ("1", "true"),
    )
    if args.profile:
        engine_config = EngineConfig(
            dtype="bfloat16", page_size=PAGE_SIZE, max_cache_tokens=max(args.batch, 2) * CONTEXT, max_context=CONTEXT,
            max_batch_size=max(args.batch, 2), prefill_chunk_size=max(PREFILL_TOKENS, args.profile_tokens), cuda_graphs=False,
        )
    engine = Engine(None, engine_config, device="cuda:0", model_config=model_config, random_seed=0)
    if args.profile:
        profile_steps(engine, torch, ops, args.profile, args.batch, rng, args.profile_tokens, args.profile_context)
        return 0
    peak = peaks()

    prefill = time_prefill(engine, torch, 5, rng)
    with ClockSampler(interval_ms=25) as sampler:
        decode = time_decode(engine, torch, ops, args.batch, args.steps, args.warmup, rng, repeats=REPEATS)
    clocks = sampler.summary(decode["windows"][0][0], decode["windows"][-1][1])
    clocks["sm_mhz_per_repeat"] = [sampler.summary(begin, end)["sm_mhz"] for begin, end in decode["windows"]]
    e2e = time_e2e(engine, torch, args.batch, args.steps, args.warmup, rng, repeats=REPEATS)
    points = {}
    if not args.skip_points:
        for batch in (1, 64):
            points[f"decode_b{batch}"] = round(time_decode(engine, torch, ops, batch, max(16, args.steps // 2), args.warmup, rng, repeats=3)["tokens_per_second"], 1)   # the median of three
        for batch in (1, 8, 64):
            heavy = time_decode_heavy(engine, torch, ops, batch, rng)
            points[f"decode_heavy_b{batch}"] = round(heavy["tokens_per_second"], 1)
            points[f"decode_heavy_b{batch}_hbm_frac"] = round(heavy["gbs"] / peak["hbm_gbs"], 4)
    weight_bytes = engine.model.weight_bytes()
    kv_bytes = decode["kv_tokens_per_step"] * engine.cache.bytes_per_token()
    achieved = (weight_bytes + kv_bytes) / (decode["ms_per_step"] / 1e3) / 1e9
    flops = prefill_flops(fields, PREFILL_TOKENS)
    record = {
        "metric": METRIC,
        "value": round(decode["tokens_per_second"], 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(decode["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": round(decode["tokens_per_second"] / BASELINE_TOKENS_PER_SECOND, 2),
        "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids, caches filled by real prefill",
        "config": headline_config(args.layers, args.batch, engine_config.cuda_graphs, peak["source"], engine_config.run_ahead),
        "clocks": clocks,
        "e2e": {k: (round(v, 1) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": decode["launches"],
        "prefill": {"value": round(PREFILL_TOKENS / (prefill["ms"] / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(prefill["ms"], 3),
                    "frac": round(flops / (prefill["ms"] / 1e3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": points,
        "spread": {"min": round(min(decode["per_repeat"]), 1), "max": round(max(decode["per_repeat"]), 1), "repeats": REPEATS},
    }
    if not args.skip_points:
        # the other shapes need the memory: the 4B engine goes first
        del engine
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        for name in ("mixed8b", "sampled14b"):
            points[f"{name}_output_tokens_per_second"] = run_serving_workload(name, torch)["value"]
            gc.collect()
            torch.cuda.empty_cache()
        check = float32_14b_check(torch)
        points["float32_14b_tokens_per_second"] = round(check["tokens_per_second"], 1)
        points["float32_14b_max_abs_logit_error"] = float(f"{check['max_abs_logit_error']:.3g}")
        points["float32_14b_argmax_agreement"] = round(check["argmax_agreement"], 4)
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
