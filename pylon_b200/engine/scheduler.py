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

# How long a request is made to wait by the three policies below before it goes first, in seconds
# (raun6k/Pylon uses 100 ms for each: src/pylon/scheduler/admit.py:8, src/pylon/scheduler/batch.py:3, src/pylon/engine.py:27).
ADMISSION_PATIENCE = 0.1     # a waiting request this old is not overtaken at admission
PROMPT_PATIENCE = 0.1        # a prompt that made no progress for this long gets the next portion
FULL_BATCH_PATIENCE = 0.1    # with every slot decoding, prompts are held back this long at most


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
    prompt_progress_at: float = 0.0     # when the prompt last got a portion (or was queued)
    admitted_at: float = 0.0
    first_token_at: Optional[float] = None
    last_token_at: Optional[float] = None
    prefill_seconds: float = 0.0
    inter_token_seconds: list[float] = field(default_factory=list)

    @property
    def capacity(self) -> int:
        return len(self.prompt) + self.sampling.max_new_tokens

    @property
    def prompt_left(self) -> int:
        return len(self.prompt) - self.prompt_offset

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
        self.overtakes = 0    # admissions that passed the oldest waiting request
        self.ticks = 0
        self._submitted = 0
        self.last_step: list[tuple[object, int]] = []   # (request id, tokens) of the last step, for tests and logs

    # -- intake ------------------------------------------------------------------------
    def add(self, request_id: object, prompt: Sequence[int], sampling: SamplingParams, stop_ids: Sequence[int] = ()) -> Request:
        if len(self.waiting) >= self.max_queue_size:
            raise QueueFullError(f"{len(self.waiting)} requests are waiting already, which is max_queue_size; try again when one has started")
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("an empty prompt: a request needs at least one token to start from")
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

    def _next_admission(self, now: float) -> Optional[tuple[Request, bool]]:
        """The waiting request that may start now and whether it overtakes the oldest one, or ``None``.

        The queue is walked from its oldest request: the first that fits goes.  The walk ends at a
        request that does not fit and has run out of patience (nobody overtakes it), and after
        ``admit_skip`` younger requests that did not fit either."""
        passed_over = 0
        for place, request in enumerate(self.waiting):
            if self._fits(request):
                return request, place > 0
            if now - request.enqueued_at >= ADMISSION_PATIENCE:
                return None
            if place > 0:
                passed_over += 1
            if passed_over > self.admit_skip or self.admit_skip == 0:
                return None
        return None

    def admit(self) -> None:
        if self.waiting and len(self.active) >= self.max_batch_size:
            logger.debug("admission_blocked request_id=%s reason=slots", self.waiting[0].request_id)
        while self.waiting and len(self.active) < self.max_batch_size:
            now = self.clock()
            selected = self._next_admission(now)
            if selected is None:
                logger.debug("admission_blocked request_id=%s reason=memory", self.waiting[0].request_id)
                return
            request, overtakes = selected
            self.waiting.remove(request)
            request.cache = self.cache.open(request.request_id, request.capacity)
            request.reservation = self.cache.lifetime_pages(request.capacity, self.prefill_chunk_size)
            request.admitted_at = now
            request.prompt_progress_at = request.enqueued_at
            self.active.append(request)
            if overtakes:
                self.overtakes += 1
                logger.info("admission_overtook request_id=%s admitted=%s overtakes=%s", self.waiting[0].request_id, request.request_id, self.overtakes)

    # -- building a step -------------------------------------------------------------------
    def _portion_rank(self, request: Request, budget: int, now: float) -> tuple[int, float]:
        """Sort key of a prompt that waits for its next portion (the smallest goes first): prompts out of
        patience before all others, the longest wait first; then those whose rest fits the budget, so that
        they begin to decode; then the rest.  Equal keys keep the order of admission."""
        stalled = now - request.prompt_progress_at
        if stalled >= PROMPT_PATIENCE:
            return (0, -stalled)
        return (1, 0.0) if request.prompt_left <= budget else (2, 0.0)

    def _cut_portions(self, now: float) -> list[tuple[Request, list[int]]]:
        """Portions of the waiting prompts for this tick: at most ``prefill_chunk_size`` tokens in all, cut anywhere."""
        candidates = [request for request in self.active if request.prefilling]
        portions = []
        budget = self.prefill_chunk_size
        while candidates and budget > 0:
            request = min(candidates, key=lambda candidate: self._portion_rank(candidate, budget, now))
            candidates.remove(request)
            begin = request.prompt_offset
            size = min(budget, request.prompt_left)
            portions.append((request, request.prompt[begin : begin + size]))
            budget -= size
        return portions

    def build_step(self) -> tuple[list[Request], list[list[int]]]:
        now = self.clock()
        decoding = [r for r in self.active if r.pending_token is not None]
        stalled_since = [r.prompt_progress_at for r in self.active if r.prefilling]
        # every slot decodes: prompts wait, so that the step stays a graph replay, until the oldest runs out of patience
        hold_off = len(decoding) == self.max_batch_size and stalled_since and now - min(stalled_since) < FULL_BATCH_PATIENCE
        portions = [] if hold_off else self._cut_portions(now)
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
                request.prompt_progress_at = now
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
