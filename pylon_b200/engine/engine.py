"""The engine: a model folder in, generated tokens out, on one GPU.

:class:`Engine` loads the model the folder's ``config.json`` names, sets up the cache
manager, the step function, the sampler and the scheduler, and offers two levels of use:

* ``generate(prompts, sampling)`` — the Python entry point: runs the scheduler until every
  prompt has its tokens (raun6k/Pylon's counterpart is ``Engine.enqueue`` plus its
  scheduler thread, src/pylon/engine.py:241-267; here the caller's thread drives the ticks).
* ``open`` / ``step`` / ``close`` — the step function itself, for callers that decide the
  batches themselves (trace replay, benchmarks, tests).
"""
from __future__ import annotations

import math
from pathlib import Path
from typing import Optional, Sequence

import torch

from pylon_b200.cache.manager import CacheManager, RequestCache, group_page_counts
from pylon_b200.config.engine_config import EngineConfig
from pylon_b200.config.registry import ARCHITECTURES, read_config
from pylon_b200.engine.scheduler import GenerationResult, Scheduler
from pylon_b200.engine.step import StepEntry, StepFunction
from pylon_b200.kernels import ops
from pylon_b200.models.decoder import DecoderModel
from pylon_b200.sampling.params import SamplingParams
from pylon_b200.sampling.sampler import Sampler
from pylon_b200.weights.loader import Checkpoint
from pylon_b200.weights.random_init import device_random_fetch


def require_gpu(device: Optional[str | torch.device] = None) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("pylon_b200 needs a CUDA device (NVIDIA B200, sm_100a); there is no CPU path")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    major, minor = torch.cuda.get_device_capability(device)
    if major != 10:
        raise RuntimeError(f"pylon_b200's kernels are built for sm_100a; this device is sm_{major}{minor}")
    return device


class Engine:
    def __init__(
        self,
        model_dir: Optional[str | Path],
        config: Optional[EngineConfig] = None,
        device: Optional[str | torch.device] = None,
        *,
        model_config: Optional[object] = None,
        random_seed: Optional[int] = None,
    ) -> None:
        """``model_dir``: a folder with ``config.json`` and safetensors.  Alternatively
        ``model_dir=None`` with a typed ``model_config`` and a ``random_seed`` draws the
        weights on the device (same distributions as the random-weights mode that writes a
        folder; no file is touched), for benchmarks of shapes too large to write out."""
        self.config = config or EngineConfig()
        self.device = require_gpu(device)
        dtype = self.config.torch_dtype
        if model_dir is not None:
            self.model_dir = Path(model_dir)
            self.architecture, self.model_config = read_config(self.model_dir)
            checkpoint = Checkpoint(self.model_dir)
        else:
            if model_config is None or random_seed is None:
                raise ValueError("without a model folder, a model configuration and a random seed are needed")
            self.model_dir = None
            self.architecture, self.model_config = ARCHITECTURES[model_config.architecture], model_config
            checkpoint = None
        limit = self.config.max_context
        if limit is None and self.config.max_cache_tokens is not None:
            limit = self.config.max_cache_tokens
        self.spec = self.architecture.build_spec(self.model_config, limit)
        self.model = DecoderModel(self.spec)
        if checkpoint is not None:
            checkpoint.verify(self.model.tensor_decls(), self.spec.ignored_tensors)
            fetch = checkpoint.fetch
        else:
            fetch = device_random_fetch(self.model.tensor_decls(), random_seed, self.device, dtype)
        with torch.cuda.device(self.device):
            self.model.load(fetch, dtype, self.device)
            needs = self.model.cache_needs()
            cache_of = [run.cache_of for run in self.spec.order]
            page_size = self.config.page_size
            page_counts = self._pool_pages(needs, dtype, page_size)
            self.cache = CacheManager(
                needs, cache_of, page_size=page_size, num_pages=page_counts,
                max_requests=self.config.max_batch_size, dtype=dtype, device=self.device,
            )
        # a request can be as long as the groups that keep every key have room for
        keeps_all = [group.pool.num_pages * page_size for group in self.cache.groups if group.need.window is None]
        self.max_context = min([self.spec.max_positions] + keeps_all)
        self.step_function = StepFunction(self.model, self.cache)
        if self.config.cuda_graphs:
            self.step_function.enable_graphs()
        self.sampler = Sampler(self.device)
        self.scheduler = Scheduler(
            self.cache, self._checked_step, _CheckedSampler(self.sampler),
            max_batch_size=self.config.max_batch_size, prefill_chunk_size=self.config.prefill_chunk_size,
            max_queue_size=self.config.max_queue_size, admit_skip=self.config.admit_skip, seed=self.config.seed,
            run_ahead=self.config.run_ahead,
        )
        self._next_id = 0

    # -- sizing ----------------------------------------------------------------------------
    def _pool_pages(self, needs, dtype: torch.dtype, page_size: int) -> dict:
        """Pages for every cache group (by its :class:`~pylon_b200.parts.base.KVNeed`).  With ``max_cache_tokens`` the
        pool holds that many tokens; else it takes what is left of the allowed share of the device after the weights,
        less room for the activations of one full step (raun6k/Pylon sizes its pool the same way,
        src/pylon/kv/budget.py:70-113).  A windowed group is given only what ``max_batch_size`` requests can hold of it
        at once, and the groups that keep everything share the rest."""
        slots, chunk, longest = self.config.max_batch_size, self.config.prefill_chunk_size, self.spec.max_positions
        if self.config.max_cache_tokens is not None:
            return group_page_counts(needs, page_size, self.config.max_cache_tokens, slots, longest, chunk)
        element = torch.empty((), dtype=dtype).element_size()
        most = group_page_counts(needs, page_size, longest * slots, slots, longest, chunk)   # what could ever be used
        page_bytes: dict = {}
        for need in needs:
            if need is not None and need.kv is not None:
                row_bytes = need.kv.n_kv_heads * (need.kv.head_dim + need.kv.value_width) * element
                page_bytes[need.kv] = page_bytes.get(need.kv, 0) + row_bytes * page_size
        if not page_bytes:
            return {}
        free, total = torch.cuda.mem_get_info(self.device)
        activation_room = chunk * self.spec.width * 64
        budget = int(total * self.config.max_gpu_utilization) - (total - free) - activation_room
        windowed = {kv: pages for kv, pages in most.items() if kv.window is not None}
        budget -= sum(pages * page_bytes[kv] for kv, pages in windowed.items())
        shared = sum(size for kv, size in page_bytes.items() if kv.window is None)
        pages = budget // shared if shared else 0
        if budget < 0 or (shared and pages < 1):
            raise RuntimeError("no memory is left for the cache after loading the weights")
        return {kv: (count if kv.window is not None else int(min(pages, count))) for kv, count in most.items()}

    # -- the step function, for callers that batch themselves --------------------------------
    def open(self, request_id: object, capacity: int) -> RequestCache:
        return self.cache.open(request_id, capacity)

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        with torch.cuda.device(self.device):
            return self.step_function(entries)

    def close(self, request: RequestCache) -> None:
        self.cache.close(request)

    def capture_decode_graphs(self, batch_sizes: Optional[Sequence[int]] = None) -> list[int]:
        """Captures the decode graphs of the given batch sizes (default: every size up to
        ``max_batch_size``) now instead of at their first use, as raun6k/Pylon does at start-up
        (src/pylon/engine.py:823-836).  Needs ``cuda_graphs``; returns the sizes that have a graph."""
        if self.step_function.graphs is None:
            raise RuntimeError("cuda_graphs is off")
        sizes = list(batch_sizes) if batch_sizes is not None else list(range(1, self.config.max_batch_size + 1))
        graphs = self.step_function.graphs
        with torch.cuda.device(self.device):
            try:
                for size in sizes:
                    if size > min(self.cache.free_slots(), min(self.cache.free_pages(), default=size)):
                        continue
                    # both forms of the step: for requests of about equal length, and (from two requests on) for any
                    for alike in ((True,) if size == 1 else (True, False)):
                        if size in (graphs.captured_alike if alike else graphs.captured):
                            continue
                        graphs.force_alike = alike
                        requests = [self.cache.open(("capture", size, i), 1) for i in range(size)]
                        try:
                            self.step_function([StepEntry(request, [0], (0,)) for request in requests])
                        finally:
                            for request in requests:
                                self.cache.close(request)
            finally:
                graphs.force_alike = None
            torch.cuda.synchronize(self.device)
        return sorted(set(graphs.captured) | set(graphs.captured_alike))

    def capture_padded_graphs(self, sizes: Sequence[tuple[int, int, int]]) -> list[tuple[int, int, int]]:
        """Captures now, instead of at their first use, the graphs of steps that bring prompt portions: each size is
        (rows of one token, portion rows, portion tokens), rounded up to the sizes steps are padded to.  Returns the sizes
        that have a graph.  Needs ``cuda_graphs`` and a model whose parts take padded steps."""
        from pylon_b200.engine.graphs import bucket_rows, bucket_tokens

        graphs = self.step_function.graphs
        if graphs is None:
            raise RuntimeError("cuda_graphs is off")
        if not graphs.pad_steps:
            return []
        graphs.capture_at_once = True
        try:
            with torch.cuda.device(self.device):
                for ones, portions, tokens in sizes:
                    key = (bucket_rows(ones), bucket_rows(portions), bucket_tokens(tokens))
                    if key in graphs.captured_padded or key in graphs.failed or key[1] < 1:
                        continue
                    # as few real rows as give this size, so that the example step fits beside nothing else
                    real_ones = key[0] // 2 + 1 if key[0] >= 2 else key[0]
                    real_portions = key[1] // 2 + 1 if key[1] >= 2 else key[1]
                    each = max(2, min(key[2] // real_portions, self.max_context))
                    counts = [each] * real_portions
                    counts[0] = max(2, min(self.max_context, key[2] - each * (real_portions - 1)))
                    if real_ones + real_portions > self.cache.free_slots() or bucket_tokens(sum(counts)) != key[2]:
                        continue
                    requests = [self.cache.open(("capture", key, index), count) for index, count in enumerate([1] * real_ones + counts)]
                    try:
                        self.step_function([StepEntry(request, [0] * request.capacity, (request.capacity - 1,)) for request in requests])
                    finally:
                        for request in requests:
                            self.cache.close(request)
                torch.cuda.synchronize(self.device)
        finally:
            graphs.capture_at_once = False
        return sorted(graphs.captured_padded)

    # -- generation --------------------------------------------------------------------------
    def submit(self, prompt: Sequence[int], sampling: Optional[SamplingParams] = None, request_id: Optional[object] = None) -> object:
        """Queues one request (raun6k/Pylon's ``Engine.enqueue``, src/pylon/engine.py:241-253);
        returns its id.  :meth:`tick` makes progress; finished requests come back from it."""
        sampling = sampling or SamplingParams()
        self._validate(prompt, sampling)
        if request_id is None:
            request_id = ("request", self._next_id)
            self._next_id += 1
        stop = sampling.stop_ids if sampling.stop_ids is not None else self.default_stop_ids()
        self.scheduler.add(request_id, prompt, sampling, stop)
        return request_id

    def tick(self) -> list[GenerationResult]:
        """One scheduler tick: admit, run one step, accept its tokens."""
        with torch.cuda.device(self.device):
            return self._tick()

    def _tick(self) -> list[GenerationResult]:
        return self.scheduler.tick()

    # What the scheduler calls (with _CheckedSampler below).  A kernel that gave up one of its bounded waits leaves a void
    # result and an error word; the words are looked at (a 16-byte read) where the device is waited for anyway, and inside
    # the scheduler's own error handling, so that the requests of a void step fail instead of going on with its tokens.
    def _checked_step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        logits = self.step_function(entries)
        if logits is None:   # nothing will be sampled from this step: look now
            ops.raise_on_kernel_errors(self.device)
        return logits

    def default_stop_ids(self) -> tuple[int, ...]:
        return tuple(self.spec.eos_token_ids)

    def generate(
        self,
        prompts: Sequence[Sequence[int]],
        sampling: Optional[SamplingParams | Sequence[SamplingParams]] = None,
    ) -> list[GenerationResult]:
        """Generates a continuation for every prompt (lists of token ids); results come back
        in the order of the prompts."""
        if sampling is None:
            sampling = SamplingParams()
        per_prompt = [sampling] * len(prompts) if isinstance(sampling, SamplingParams) else list(sampling)
        if len(per_prompt) != len(prompts):
            raise ValueError("one SamplingParams for all prompts, or one per prompt")
        for prompt, params in zip(prompts, per_prompt):
            self._validate(prompt, params)
        ids = []
        waiting = list(zip(prompts, per_prompt))
        results: dict[object, GenerationResult] = {}
        with torch.cuda.device(self.device):
            while waiting or self.scheduler.has_work():
                while waiting and len(self.scheduler.waiting) < self.scheduler.max_queue_size:
                    prompt, params = waiting.pop(0)
                    request_id = ("generate", self._next_id)
                    self._next_id += 1
                    stop = params.stop_ids if params.stop_ids is not None else self.default_stop_ids()
                    self.scheduler.add(request_id, prompt, params, stop)
                    ids.append(request_id)
                for result in self._tick():
                    results[result.request_id] = result
        ordered = [results[request_id] for request_id in ids]
        for result in ordered:
            if result.error is not None:
                raise result.error
        return ordered

    def _validate(self, prompt: Sequence[int], params: SamplingParams) -> None:
        vocab = self.spec.vocab_size
        if len(prompt) < 1:
            raise ValueError("an empty prompt: a request needs at least one token to start from")
        for token in prompt:
            if isinstance(token, bool) or not isinstance(token, int) or not 0 <= token < vocab:
                raise ValueError(f"{token!r} is not a token id of this model: ids are whole numbers from 0 to {vocab - 1}")
        needed = len(prompt) + params.max_new_tokens
        if needed > self.max_context:
            raise ValueError(f"prompt plus max_new_tokens is {needed} tokens; this engine was set up for requests of up to {self.max_context}")


class _CheckedSampler:
    """The sampler as the scheduler uses it: a copy of the kernels' error words is queued behind the step and travels with
    its tokens; whoever waits for the tokens (at once, or a step later when the scheduler runs ahead) gets the error
    instead, if the step's result is void."""

    def __init__(self, sampler: Sampler) -> None:
        self.sampler = sampler

    def launch(self, logits, params, randoms):
        return self.sampler.launch(logits, params, randoms, check_errors=True)

    def __call__(self, logits, params, randoms) -> list[int]:
        return self.launch(logits, params, randoms).result()


def generate(
    model_dir: str | Path,
    prompts: Sequence[Sequence[int]],
    sampling: Optional[SamplingParams | Sequence[SamplingParams]] = None,
    config: Optional[EngineConfig] = None,
) -> list[GenerationResult]:
    """One-call form: load the model folder, generate, return the results."""
    return Engine(model_dir, config).generate(prompts, sampling)
