"""The reference arm of ``bench.py``: raun6k/Pylon itself, unmodified, on the headline workload.

``baseline/_ref/pylon`` is a byte-for-byte copy of the reference's package (``src/pylon`` of its
repository), laid out as a wheel install would lay it out.  This module imports it from there
and drives its own classes on its own code path; nothing of ``pylon_b200`` is imported, and no
kernel or library of this repository is loaded into the process.

What runs, in the order it is tried:

1. **The serving path** (paged cache, CUDA graphs), as the reference's engine uses it:
   ``Qwen3Config`` at its stock 4B sizes (src/pylon/model/config.py:20-32), ``Qwen3Model`` on the
   GPU with its weights overwritten by N(0, 0.02) (src/pylon/model/model.py:18-35), ``KVPagePool``
   with 256-token pages (src/pylon/kv/pool.py:19-45), ``Decoder`` (src/pylon/decode/runner.py:58-64),
   the prompts through ``Decoder.packed_caches`` in 2,048-token portions (runner.py:271-302),
   ``capture_decode_graphs`` (src/pylon/decode/warmup.py:140-167), then K timed
   ``Decoder.decode_caches`` steps (runner.py:227-269) with the arg-max and the read-back of the
   tokens inside the timed region, as its engine does after every step (src/pylon/engine.py:454-471).
   ``e2e`` goes through ``Engine(config, decoder=..., capacity=...)`` and ``Engine.enqueue``
   (src/pylon/engine.py:113-162, 241-253): host token lists in, futures with host token lists out.
2. If the paged attention call refuses to run on the installed PyTorch (the reference asks for
   torch >= 2.13 and passes ``varlen_attn`` arguments that older versions do not take,
   src/pylon/kv/cache.py:250-263), the refusal's text is kept in the record and the same model runs
   the reference's **other stock cache**, the dense per-request ``KVCache`` that ``Decoder`` uses when
   it has no page pool (src/pylon/kv/dense.py, runner.py:117-146 and 265-269, 341-367): whole prompts
   through ``Decoder.prefill``, decoding through ``Decoder.decode_caches``.  That path has no graphs
   and no engine above it; the record says which path its numbers come from.

The line printed has the keys of ``bench.py``'s own line plus ``"impl": "reference"``.
"""
from __future__ import annotations

import json
import shutil
import sys
import time
import traceback
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_ROOT = HERE / "_ref"
UPSTREAM = Path("/root/reference/src/pylon")   # where the reference is mounted on the build machine


def _place_reference() -> str | None:
    """Makes sure ``baseline/_ref/pylon`` exists; returns a reason if it cannot."""
    package = REF_ROOT / "pylon"
    if (package / "engine.py").is_file():
        return None
    if (UPSTREAM / "engine.py").is_file():
        REF_ROOT.mkdir(parents=True, exist_ok=True)
        shutil.copytree(UPSTREAM, package, ignore=shutil.ignore_patterns("__pycache__"))
        return None
    return f"no copy of raun6k/Pylon's package at {package} and none to copy from"


def _short(error: BaseException) -> str:
    text = f"{type(error).__name__}: {error}".replace("\n", " ")
    return text[:300]


class _Arm:
    def __init__(self, args, shared) -> None:
        import torch

        self.torch = torch
        self.args = args
        self.context = shared["context"]
        self.page_size = shared["page_size"]
        self.prefill_tokens = shared["prefill_tokens"]
        self.device = torch.device("cuda", 0)
        from pylon.model.config import Qwen3Config
        from pylon.model.model import Qwen3Model

        self.config = Qwen3Config()   # the stock Qwen3-4B sizes
        torch.manual_seed(0)
        with torch.device(self.device):
            self.model = Qwen3Model(self.config)
        with torch.no_grad():
            for name, parameter in self.model.named_parameters():
                if parameter.dim() == 1:   # norm scales
                    parameter.copy_(1.0 + 0.02 * torch.randn_like(parameter))
                else:
                    parameter.normal_(0.0, 0.02)
        self.model.eval()
        self.generator = torch.Generator().manual_seed(0)

    def tokens(self, count: int) -> list[int]:
        return self.torch.randint(0, self.config.vocab_size, (count,), generator=self.generator).tolist()

    # -- the serving path: pages and graphs --------------------------------------------------
    def timed_repeats(self, step, steps: int, warmup: int, repeats: int) -> list[float]:
        """``warmup`` untimed calls of ``step``, then ``repeats`` times K calls between CUDA events; milliseconds of each repeat."""
        torch = self.torch
        for _ in range(warmup):
            step()
        spans = []
        for _ in range(repeats):
            begin_event, end_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            begin_event.record()
            for _ in range(steps):
                step()
            end_event.record()
            torch.cuda.synchronize()
            spans.append(begin_event.elapsed_time(end_event))
        return spans

    @staticmethod
    def middle(spans: list[float]) -> float:
        return sorted(spans)[len(spans) // 2]

    def paged_decode(self, batch: int, steps: int, warmup: int, graphs: bool, repeats: int = 1) -> dict:
        torch = self.torch
        from pylon.decode.runner import Decoder
        from pylon.decode.warmup import capture_decode_graphs
        from pylon.kv.cache import PagedKVCache
        from pylon.kv.pool import KVPagePool

        pages_each = -(-self.context // self.page_size)
        pool = KVPagePool(self.config, batch * pages_each + batch + 1, device=self.device, page_size=self.page_size)
        decoder = Decoder(self.model)
        decoder.page_pool = pool
        try:
            start_length = self.context - (warmup + repeats * steps)
            caches = [PagedKVCache(pool, self.context) for _ in range(batch)]
            for cache in caches:
                prompt = self.tokens(start_length)
                for begin in range(0, start_length, self.prefill_tokens):
                    decoder.packed_caches([cache], [prompt[begin : begin + self.prefill_tokens]], logit_rows=[])
            torch.cuda.synchronize()
            captured = ()
            if graphs:
                captured = capture_decode_graphs(decoder, token_id=1, max_batch_size=batch, max_tokens=self.context)
            state = {"tokens": self.tokens(batch)}

            def step():
                logits = decoder.decode_caches(caches, state["tokens"])
                state["tokens"] = logits.argmax(dim=-1).cpu().tolist()

            spans = self.timed_repeats(step, steps, warmup, repeats)
            milliseconds = self.middle(spans)
            for cache in caches:
                decoder.release_cache(cache)
            return {"ms_per_step": milliseconds / steps, "tokens_per_second": batch * steps / (milliseconds / 1e3),
                    "graphs": batch in captured, "per_repeat": [batch * steps / (ms / 1e3) for ms in spans]}
        finally:
            decoder.graphs = None
            decoder.release_page_pool()
            del pool
            torch.cuda.empty_cache()

    def paged_prefill(self, repeats: int = 5) -> float:
        torch = self.torch
        from pylon.decode.runner import Decoder
        from pylon.kv.cache import PagedKVCache
        from pylon.kv.pool import KVPagePool

        pool = KVPagePool(self.config, 2 * (-(-self.prefill_tokens // self.page_size)), device=self.device, page_size=self.page_size)
        decoder = Decoder(self.model)
        decoder.page_pool = pool
        best = None
        begin_event, end_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        try:
            for index in range(repeats):
                cache = PagedKVCache(pool, self.prefill_tokens)
                prompt = self.tokens(self.prefill_tokens)
                torch.cuda.synchronize()
                begin_event.record()
                decoder.packed_caches([cache], [prompt], logit_rows=[0])
                end_event.record()
                torch.cuda.synchronize()
                decoder.release_cache(cache)
                if index >= 2:
                    elapsed = begin_event.elapsed_time(end_event)
                    best = elapsed if best is None else min(best, elapsed)
        finally:
            decoder.release_page_pool()
            del pool
            torch.cuda.empty_cache()
        return best

    def engine_e2e(self, batch: int, steps: int, warmup: int) -> dict:
        """Through ``Engine.enqueue``: the requests' own records of when each token came back say how long the
        ticks took while all ``batch`` requests were decoding."""
        torch = self.torch
        from pylon.api.types import Sampling
        from pylon.config import PylonConfig
        from pylon.decode.runner import Decoder
        from pylon.engine import Engine
        from pylon.kv.budget import CacheCapacity

        bytes_per_token = self.config.n_layers * 2 * self.config.n_kv_heads * self.config.head_dim * 2
        pages = batch * (-(-self.context // self.page_size)) + batch + 1
        budget = pages * self.page_size * bytes_per_token
        capacity = CacheCapacity(free_bytes=budget, device_occupied_bytes=0, activation_headroom_bytes=0, bytes_per_token=bytes_per_token,
                                 max_tokens=self.context, kv_budget_bytes=budget, model_occupied_bytes=0)
        config = PylonConfig(prefix_cache=False, cuda_graphs=True, max_batch_size=batch, max_queue_size=max(batch, 32),
                             prefill_chunk_size=self.prefill_tokens)
        engine = Engine(config, decoder=Decoder(self.model), capacity=capacity)
        try:
            engine.capture_decode_graphs([1])
            new_tokens = warmup + steps + 3 * batch + 8
            prompt_length = self.context - new_tokens
            sampling = Sampling(temperature=0, top_p=1, max_new_tokens=new_tokens)
            futures = [engine.enqueue(self.tokens(prompt_length), (), sampling, request_id=f"bench-{index}") for index in range(batch)]
            results = [future.result(timeout=600) for future in futures]
        finally:
            engine.close()
            torch.cuda.empty_cache()
        last = max(results, key=lambda result: result.first_token_at)          # the request that began to decode last
        first_done = min(result.first_token_at + sum(result.token_intervals) for result in results)
        window = last.token_intervals[warmup : warmup + steps]
        window_end = last.first_token_at + sum(last.token_intervals[: warmup + steps])
        if len(window) != steps or window_end > first_done or any(len(result.output_ids) != new_tokens for result in results):
            raise RuntimeError("the timed ticks were not all ticks of the full batch")
        seconds = sum(window)
        return {"value": batch * steps / seconds, "unit": "tokens/s", "h2d_bytes_per_step": batch * (8 + 8 + 8 + 4 * (self.context // self.page_size) + 12) + 8,
                "d2h_bytes_per_step": batch * 8}

    # -- the dense cache: no pages, no graphs ------------------------------------------------
    def dense_decode(self, batch: int, steps: int, warmup: int, host_timed: bool = False, repeats: int = 1) -> dict:
        torch = self.torch
        from pylon.api.types import Sampling
        from pylon.decode.runner import Decoder

        decoder = Decoder(self.model)
        new_tokens = warmup + repeats * steps
        start_length = self.context - new_tokens
        sampling = Sampling(temperature=0, top_p=1, max_new_tokens=new_tokens)
        caches = [decoder.prefill(self.tokens(start_length), sampling, max_total_tokens=self.context).cache for _ in range(batch)]
        state = {"tokens": self.tokens(batch)}

        def step():
            logits = decoder.decode_caches(caches, state["tokens"])
            state["tokens"] = logits.argmax(dim=-1).cpu().tolist()

        if host_timed:
            for _ in range(warmup):
                step()
            torch.cuda.synchronize()
            started = time.perf_counter()
            for _ in range(steps):
                step()
            torch.cuda.synchronize()
            seconds = time.perf_counter() - started
        else:
            spans = self.timed_repeats(step, steps, warmup, repeats)
            milliseconds = self.middle(spans)
        for cache in caches:
            decoder.release_cache(cache)
        del caches
        torch.cuda.empty_cache()
        if host_timed:
            return {"value": batch * steps / seconds, "unit": "tokens/s", "h2d_bytes_per_step": batch * 16, "d2h_bytes_per_step": batch * 8}
        return {"ms_per_step": milliseconds / steps, "tokens_per_second": batch * steps / (milliseconds / 1e3), "graphs": False,
                "per_repeat": [batch * steps / (ms / 1e3) for ms in spans]}

    def dense_prefill(self, repeats: int = 5) -> float:
        torch = self.torch
        from pylon.api.types import Sampling
        from pylon.decode.runner import Decoder

        decoder = Decoder(self.model)
        sampling = Sampling(temperature=0, top_p=1, max_new_tokens=1)
        best = None
        begin_event, end_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for index in range(repeats):
            prompt = self.tokens(self.prefill_tokens)
            torch.cuda.synchronize()
            begin_event.record()
            result = decoder.prefill(prompt, sampling, max_total_tokens=self.prefill_tokens + 1)
            end_event.record()
            torch.cuda.synchronize()
            decoder.release_cache(result.cache)
            if index >= 2:
                elapsed = begin_event.elapsed_time(end_event)
                best = elapsed if best is None else min(best, elapsed)
        return best


def run(args, shared: dict) -> int:
    """``shared``: bench.py's constants, its clock sampler class, its peaks and its flop count, so that both arms
    describe the same work in the same words."""
    def unavailable(reason: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": reason}))
        return 0

    if args.gpus != 1:
        return unavailable("raun6k/Pylon is a single-GPU engine; --gpus must be 1")
    reason = _place_reference()
    if reason:
        return unavailable(reason)
    sys.path.insert(0, str(REF_ROOT))
    try:
        import torch

        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        import pylon.decode.runner   # noqa: F401  (the imports the arm needs, before any GPU work)
        import pylon.engine          # noqa: F401
    except Exception as error:   # a missing dependency of the reference
        return unavailable(f"raun6k/Pylon does not import here: {_short(error)}")
    if args.warmup < 3:
        args.warmup = 3
    try:
        arm = _Arm(args, shared)
    except Exception as error:
        return unavailable(f"raun6k/Pylon's model could not be built: {_short(error)}")

    batch, steps, warmup, repeats = args.batch, args.steps, args.warmup, int(shared["config"].get("repeats", 1))
    sampler_class = shared["clock_sampler"]
    notes = {}
    path = "paged cache + CUDA graphs (the engine's serving path)"
    try:
        with sampler_class() as sampler:
            decode = arm.paged_decode(batch, steps, warmup, graphs=True, repeats=repeats)
        prefill_ms = arm.paged_prefill()
        paged = True
    except Exception as error:
        notes["paged_path_refused"] = _short(error)
        sys.stderr.write("reference arm: the paged path did not run:\n" + traceback.format_exc())
        paged = False
    if paged:
        try:
            e2e = arm.engine_e2e(batch, steps, warmup)
        except Exception as error:
            notes["engine_e2e_failed"] = _short(error)
            e2e = None
        points = {}
        if not args.skip_points:
            for size in (1, 64):
                try:
                    points[f"decode_b{size}"] = round(arm.paged_decode(size, max(16, steps // 2), warmup, graphs=True)["tokens_per_second"], 1)
                except Exception as error:
                    notes[f"decode_b{size}_failed"] = _short(error)
    else:
        path = "dense per-request KVCache through Decoder (no pages, no graphs, no Engine): the paged path was refused"
        try:
            with sampler_class() as sampler:
                decode = arm.dense_decode(batch, steps, warmup, repeats=repeats)
            prefill_ms = arm.dense_prefill()
            e2e = arm.dense_decode(batch, steps, warmup, host_timed=True)
        except Exception as error:
            sys.stderr.write("reference arm: the dense path did not run either:\n" + traceback.format_exc())
            return unavailable(f"raun6k/Pylon's paged path: {notes['paged_path_refused']}; its dense path: {_short(error)}")
        points = {}
        if not args.skip_points:
            for size in (1, 64):
                try:
                    points[f"decode_b{size}"] = round(arm.dense_decode(size, max(16, steps // 2), warmup)["tokens_per_second"], 1)
                except Exception as error:
                    notes[f"decode_b{size}_failed"] = _short(error)

    peak = shared["peaks"]
    config = arm.config
    flops = shared["prefill_flops"](arm.prefill_tokens)
    record = {
        "impl": "reference",
        "metric": shared["metric"],
        "value": round(decode["tokens_per_second"], 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": round(decode["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": round(decode["tokens_per_second"] / shared["baseline_tokens_per_second"], 2),
        "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids, caches filled by real prefill",
        "config": dict(shared["config"], cuda_graphs=bool(decode["graphs"])),
        "reference_path": path,
        "clocks": sampler.summary(),
        "prefill": {"value": round(arm.prefill_tokens / (prefill_ms / 1e3), 1), "tokens": arm.prefill_tokens, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)},
        "points": points,
        "spread": {"min": round(min(decode["per_repeat"]), 1), "max": round(max(decode["per_repeat"]), 1), "repeats": repeats},
    }
    if e2e is not None:
        record["e2e"] = {key: (round(value, 1) if isinstance(value, float) else value) for key, value in e2e.items()}
    record.update(notes)
    assert config.n_layers == 36 and config.hidden_size == 2_560   # the stock sizes are the headline's
    print(json.dumps(record))
    return 0
