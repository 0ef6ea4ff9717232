"""Continuous batching above the step function.

Each tick: admit waiting requests, build one step (a token for every decoding request plus
portions of waiting prompts under a token budget), run it, choose tokens, finish requests
and free what they held.  The scheduler is plain host code around two callables — the step
function and the sampler — so its decisions can be tested without a GPU.

Policies follow raun6k/Pylon:

* admission (src/pylon/scheduler/admit.py:11-95): first come first served while request
  slots are free; a request reserves the pages of its whole life (prompt + max_new_tokens)
  and is admitted only if all reservations fit the pool and the pages left over are at
  least the number of decoding requests; if the head does not fit, up to ``admit_skip``
  younger requests may go first unless one of them has waited 100 ms; a request that could
  never fit fails at once.
* portions (src/pylon/scheduler/batch.py:6-54): up to ``prefill_chunk_size`` prompt tokens
  per tick over as many prompts as fit, cut anywhere; a prompt that has waited 100 ms goes
  first, else one that ends inside the budget, else the oldest.  Decoded tokens do not
  count against the budget.  With every slot decoding and the oldest prompt younger than
  100 ms the tick decodes only (src/pylon/engine.py:30-35,277-281).
* tokens (src/pylon/engine.py:598-618): a stop id ends the request (``"eos"``, the stop
  token is not returned); ``max_new_tokens`` outputs end it (``"length"``); the first
  token comes from the step that brings the prompt's last portion.
* pages: reservations make running out impossible for admitted requests; waiting requests
  wait.  If a step fails all the same (out of pages or any other error), the requests of
  that step fail with the error and give back what they held, the others go on.  (The
  reference fails every active request, src/pylon/engine.py:262-264,716-722.)
"""
from __future__ import annotations

import logging
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

from pylon_b200.cache.manager import CacheManager, RequestCache
from pylon_b200.engine.step import StepEntry
from pylon_b200.sampling.params import SamplingParams
from pylon_b200.sampling.sampler import RequestRandom

logger = logging.getLogger("pylon_b200")   # key=value lines, as raun6k/Pylon logs its scheduler (src/pylon/scheduler/admit.py:16-57)

PREFILL_MAX_WAIT_SECONDS = 0.1
ADMIT_SKIP_WAIT_SECONDS = 0.1
FULL_BATCH_PREFILL_WAIT_SECONDS = 0.1


class QueueFullError(RuntimeError):
    pass


@dataclass
class GenerationResult:
    request_id: object
    output_ids: list[int]
    finish_reason: str                       # "eos" | "length" | "error"
    prompt_tokens: int
    queue_seconds: float = 0.0
    prefill_seconds: float = 0.0
    first_token_seconds: Optional[float] = None
    inter_token_seconds: list[float] = field(default_factory=list)
    elapsed_seconds: float = 0.0
    error: Optional[BaseException] = None


@dataclass
class Request:
    request_id: object
    prompt: list[int]
    sampling: SamplingParams
    stop_ids: frozenset[int]
    enqueued_at: float
    random: Optional[RequestRandom] = None
    # while active
    cache: Optional[RequestCache] = None
    reservation: list[int] = field(default_factory=list)
    prompt_offset: int = 0
    pending_token: Optional[int] = None
    output_ids: list[int] = field(default_factory=list)
    prefill_wait_started: float = 0.0
    admitted_at: float = 0.0
    first_token_at: Optional[float] = None
    last_token_at: Optional[float] = None
    prefill_seconds: float = 0.0
    inter_token_seconds: list[float] = field(default_factory=list)

    @property
    def capacity(self) -> int:
        return len(self.prompt) + self.sampling.max_new_tokens

    @property
    def prefilling(self) -> bool:
        return self.pending_token is None and self.prompt_offset < len(self.prompt)


class Scheduler:
    def __init__(
        self,
        cache: CacheManager,
        run_step: Callable[[Sequence[StepEntry]], object],
        sample: Callable[[object, Sequence[SamplingParams], Sequence[Optional[RequestRandom]]], list[int]],
        *,
        max_batch_size: int = 32,
        prefill_chunk_size: int = 2048,
        max_queue_size: int = 32,
        admit_skip: int = 4,
        free_page_floor: bool = True,
        clock: Callable[[], float] = time.perf_counter,
        seed: int = 0,
    ) -> None:
        if max_batch_size < 1 or max_batch_size > cache.max_requests:
            raise ValueError(f"max_batch_size must be between 1 and the cache's {cache.max_requests} request slots")
        if prefill_chunk_size < 1:
            raise ValueError("prefill_chunk_size must be a positive integer")
        if max_queue_size < 1:
            raise ValueError("max_queue_size must be at least 1")
        if admit_skip < 0:
            raise ValueError("admit_skip must be an integer of at least 0")
        self.cache = cache
        self.run_step = run_step
        self.sample = sample
        self.max_batch_size = max_batch_size
        self.prefill_chunk_size = prefill_chunk_size
        self.max_queue_size = max_queue_size
        self.admit_skip = admit_skip
        self.free_page_floor = free_page_floor
        self.clock = clock
        self.seed = seed
        self.waiting: deque[Request] = deque()
        self.active: list[Request] = []
        self.finished: list[GenerationResult] = []
        self.head_skips = 0
        self.ticks = 0
        self._submitted = 0
        self.last_step: list[tuple[object, int]] = []   # (request id, tokens) of the last step, for tests and logs

    # -- intake ------------------------------------------------------------------------
    def add(self, request_id: object, prompt: Sequence[int], sampling: SamplingParams, stop_ids: Sequence[int] = ()) -> Request:
        if len(self.waiting) >= self.max_queue_size:
            raise QueueFullError("The generation waiting queue is full.")
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("A request prompt must contain at least one token.")
        capacity = len(prompt) + sampling.max_new_tokens
        needed = self.cache.lifetime_pages(capacity, self.prefill_chunk_size)
        for g, group in enumerate(self.cache.groups):
            if needed[g] > group.pool.num_pages:
                raise ValueError(
                    f"Request needs {needed[g]} cache pages in group {g}, but the pool has {group.pool.num_pages}."
                )
        seed = sampling.seed if sampling.seed is not None else self.seed * 1_000_003 + self._submitted
        self._submitted += 1
        request = Request(
            request_id, prompt, sampling, frozenset(() if sampling.ignore_eos else stop_ids), self.clock(),
            random=None if sampling.greedy else RequestRandom(seed),
        )
        self.waiting.append(request)
        return request

    def abort(self, request_id: object) -> bool:
        """Drops a waiting or active request; what it held goes back at once."""
        for request in list(self.waiting):
            if request.request_id == request_id:
                self.waiting.remove(request)
                return True
        for request in self.active:
            if request.request_id == request_id:
                self._release(request)
                self.active.remove(request)
                return True
        return False

    def has_work(self) -> bool:
        return bool(self.waiting or self.active)

    # -- admission -----------------------------------------------------------------------
    def _reserved(self) -> list[int]:
        totals = [0] * len(self.cache.groups)
        for request in self.active:
            for g, pages in enumerate(request.reservation):
                totals[g] += pages
        return totals

    def _fits(self, request: Request) -> bool:
        reserved = self._reserved()
        needed = self.cache.lifetime_pages(request.capacity, self.prefill_chunk_size)
        decoding = sum(1 for active in self.active if active.pending_token is not None)
        for g, group in enumerate(self.cache.groups):
            left = group.pool.num_pages - reserved[g] - needed[g]
            if left < 0 or (self.free_page_floor and left < decoding):
                return False
        return True

    def _select_waiting(self, now: float) -> Optional[tuple[Request, bool]]:
        head = self.waiting[0]
        if self._fits(head):
            return head, False
        if now - head.enqueued_at >= ADMIT_SKIP_WAIT_SECONDS or self.admit_skip <= 0:
            return None
        skips = 0
        for request in list(self.waiting)[1:]:
            if self._fits(request):
                return request, True
            if now - request.enqueued_at >= ADMIT_SKIP_WAIT_SECONDS or skips >= self.admit_skip:
                return None
            skips += 1
        return None

    def admit(self) -> None:
        if self.waiting and len(self.active) >= self.max_batch_size:
            logger.debug("admission_blocked request_id=%s reason=slots", self.waiting[0].request_id)
        while self.waiting and len(self.active) < self.max_batch_size:
            now = self.clock()
            selected = self._select_waiting(now)
            if selected is None:
                logger.debug("admission_blocked request_id=%s reason=memory", self.waiting[0].request_id)
                return
            request, skipped_head = selected
            self.waiting.remove(request)
            request.cache = self.cache.open(request.request_id, request.capacity)
            request.reservation = self.cache.lifetime_pages(request.capacity, self.prefill_chunk_size)
            request.admitted_at = now
            request.prefill_wait_started = request.enqueued_at
            self.active.append(request)
            if skipped_head:
                self.head_skips += 1
                logger.info("admission_skipped_head request_id=%s admitted=%s head_skips=%s", self.waiting[0].request_id, request.request_id, self.head_skips)

    # -- building a step -------------------------------------------------------------------
    def _choose_prefill(self, pending: list[Request], budget: int, now: float) -> Request:
        aged = [r for r in pending if now - r.prefill_wait_started >= PREFILL_MAX_WAIT_SECONDS]
        if aged:
            return min(aged, key=lambda r: r.prefill_wait_started)
        fitting = [r for r in pending if len(r.prompt) - r.prompt_offset <= budget]
        return (fitting or pending)[0]

    def _prefill_portions(self, now: float) -> list[tuple[Request, list[int]]]:
        pending = [r for r in self.active if r.prefilling]
        chosen = []
        budget = self.prefill_chunk_size
        while pending and budget > 0:
            request = self._choose_prefill(pending, budget, now)
            pending.remove(request)
            count = min(budget, len(request.prompt) - request.prompt_offset)
            chosen.append((request, request.prompt[request.prompt_offset : request.prompt_offset + count]))
            budget -= count
        return chosen

    def build_step(self) -> tuple[list[Request], list[list[int]]]:
        now = self.clock()
        decoding = [r for r in self.active if r.pending_token is not None]
        waiting_prompts = [r.prefill_wait_started for r in self.active if r.prefilling]
        hold_off = (
            len(decoding) == self.max_batch_size
            and waiting_prompts
            and now - min(waiting_prompts) < FULL_BATCH_PREFILL_WAIT_SECONDS
        )
        portions = [] if hold_off else self._prefill_portions(now)
        selected = decoding + [request for request, _ in portions]
        chunks = [[r.pending_token] for r in decoding] + [tokens for _, tokens in portions]
        return selected, chunks

    # -- one tick --------------------------------------------------------------------------
    def tick(self) -> list[GenerationResult]:
        """Admit, run one step, accept its tokens.  Returns the requests that finished."""
        self.ticks += 1
        done_before = len(self.finished)
        self.admit()
        if self.active:
            selected, chunks = self.build_step()
            if selected:
                self._execute(selected, chunks)
        self.admit()
        return self.finished[done_before:]

    def run(self) -> list[GenerationResult]:
        """Ticks until nothing is waiting or active; returns everything that finished."""
        start = len(self.finished)
        while self.has_work():
            before = (len(self.waiting), len(self.active), len(self.finished))
            self.tick()
            if not self.active and self.waiting and before == (len(self.waiting), 0, len(self.finished)):
                raise RuntimeError("a waiting request can never be admitted")   # guarded by add(); defensive
        return self.finished[start:]

    def _execute(self, selected: list[Request], chunks: list[list[int]]) -> None:
        entries, ready = [], []
        for request, chunk in zip(selected, chunks):
            samples = request.pending_token is not None or request.prompt_offset + len(chunk) >= len(request.prompt)
            entries.append(StepEntry(request.cache, chunk, (len(chunk) - 1,) if samples else ()))
            if samples:
                ready.append(request)
        self.last_step = [(request.request_id, len(chunk)) for request, chunk in zip(selected, chunks)]
        started = self.clock()
        try:
            logits = self.run_step(entries)
            tokens = self.sample(logits, [r.sampling for r in ready], [r.random for r in ready]) if ready else []
        except Exception as error:   # the step's requests fail; the others go on
            logger.exception("model_batch_failed requests=%s", [request.request_id for request in selected])
            for request in selected:
                self._finish(request, "error", error)
            return
        now = self.clock()
        elapsed = now - started
        for request, chunk in zip(selected, chunks):
            if request.pending_token is None:
                request.prompt_offset += len(chunk)
                request.prefill_wait_started = now
                request.prefill_seconds += elapsed
            else:
                request.inter_token_seconds.append(elapsed)
        for request, token in zip(ready, tokens):
            self._accept(request, int(token), now)

    def _accept(self, request: Request, token: int, now: float) -> None:
        if request.first_token_at is None:
            request.first_token_at = now
        if token in request.stop_ids:
            self._finish(request, "eos")
            return
        request.last_token_at = now
        request.output_ids.append(token)
        if len(request.output_ids) >= request.sampling.max_new_tokens:
            self._finish(request, "length")
            return
        request.pending_token = token

    # -- ending ----------------------------------------------------------------------------
    def _release(self, request: Request) -> None:
        if request.cache is not None and not request.cache.closed:
            if request.cache.pending:
                self.cache.rollback(request.cache)
            self.cache.close(request.cache)
        request.reservation = []

    def _finish(self, request: Request, reason: str, error: Optional[BaseException] = None) -> None:
        self._release(request)
        if request in self.active:
            self.active.remove(request)
        now = self.clock()
        self.finished.append(
            GenerationResult(
                request_id=request.request_id,
                output_ids=request.output_ids,
                finish_reason=reason,
                prompt_tokens=len(request.prompt),
                queue_seconds=request.admitted_at - request.enqueued_at,
                prefill_seconds=request.prefill_seconds,
                first_token_seconds=None if request.first_token_at is None else request.first_token_at - request.enqueued_at,
                inter_token_seconds=request.inter_token_seconds,
                elapsed_seconds=now - request.enqueued_at,
                error=error,
            )
        )
