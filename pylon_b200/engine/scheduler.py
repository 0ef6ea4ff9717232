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
* running ahead (this engine's own; the reference waits for every step's tokens before it builds the next,
  src/pylon/engine.py:454-471): with ``run_ahead`` a tick queues its step behind the one before and only then waits
  for that one's tokens, so the device never waits for the host.  A decoding request's token for the new step is taken on
  the device from what the sampling kernel chose in the step before.  The host is one step behind: a request that met a
  stop id has been given one more step already, whose token is dropped; ``max_new_tokens`` is known beforehand and never
  overrun, and a request gives back its slot and pages when its last token by count is launched, not when it arrives.
  What a request generates is the same either way.
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
    prompt_offset: int = 0              # prompt tokens handed to steps so far
    pending_token: Optional[int] = None     # the last token chosen, known here and not yet fed to a step
    in_flight: Optional[tuple[object, int]] = None   # (sampled tokens of a step not read back yet, row): the same, still on the device
    launched: int = 0                   # tokens being chosen by steps whose results are not read back yet
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
        return self.pending_token is None and self.in_flight is None and self.prompt_offset < len(self.prompt)

    @property
    def decoding(self) -> bool:
        """Has a last token (here or on the device) and room for one more."""
        return (self.pending_token is not None or self.in_flight is not None) and len(self.output_ids) + self.launched < self.sampling.max_new_tokens


class _Known:
    """Tokens that are there already, in the form of a sampler's ``launch`` result."""

    device = None

    def __init__(self, tokens: Sequence[int]) -> None:
        self._tokens = list(tokens)

    def result(self) -> list[int]:
        return self._tokens


@dataclass
class _Launched:
    """A step that is queued and whose tokens are not accepted yet."""

    selected: list[Request]
    chunks: list[list[int]]
    prompt_rows: list[bool]          # by selected request: it brought a portion of its prompt
    ready: list[Request]             # the requests a token is chosen for, in the order of the tokens
    tokens: object                   # result() gives them; .device holds them before that
    started: float


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
        run_ahead: bool = False,
    ) -> None:
        if max_batch_size < 1 or max_batch_size > cache.max_requests:
            raise ValueError(f"max_batch_size must be between 1 and the cache's {cache.max_requests} request slots")
        if prefill_chunk_size < 1:
            raise ValueError("prefill_chunk_size must be a positive integer")
        if max_queue_size < 1:
            raise ValueError("max_queue_size must be at least 1")
        if admit_skip < 0:
            raise ValueError("admit_skip must be an integer of at least 0")
        if run_ahead and not hasattr(sample, "launch"):
            raise ValueError("run_ahead needs a sampler with launch(): one that hands out its tokens on the device before the host has them")
        self.cache = cache
        self.run_step = run_step
        self.sample = sample
        self.run_ahead = run_ahead
        self._flying: Optional[_Launched] = None    # the step whose tokens are not read back yet
        self._collected_at = 0.0
        self.max_batch_size = max_batch_size
        self.prefill_chunk_size = prefill_chunk_size
        self.max_queue_size = max_queue_size
        self.admit_skip = admit_skip
        self.free_page_floor = free_page_floor
        self.clock = clock
        self.seed = seed
        self.waiting: deque[Request] = deque()
        self.active: list[Request] = []
        self.leaving: list[Request] = []    # running ahead: their last token is being chosen; slot and pages are given back already
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
        for holding in (self.active, self.leaving):
            for request in holding:
                if request.request_id == request_id:
                    self._release(request)
                    holding.remove(request)
                    return True
        return False

    def has_work(self) -> bool:
        return bool(self.waiting or self.active or self.leaving or self._flying is not None)

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
        decoding = sum(1 for active in self.active if active.pending_token is not None or active.in_flight is not None)
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
        decoding = [r for r in self.active if r.decoding]
        stalled_since = [r.prompt_progress_at for r in self.active if r.prefilling]
        # every slot decodes: prompts wait, so that the step stays a graph replay, until the oldest runs out of patience
        hold_off = len(decoding) == self.max_batch_size and stalled_since and now - min(stalled_since) < FULL_BATCH_PATIENCE
        portions = [] if hold_off else self._cut_portions(now)
        selected = decoding + [request for request, _ in portions]
        chunks = [[r.pending_token if r.in_flight is None else 0] for r in decoding] + [tokens for _, tokens in portions]   # 0: taken on the device
        return selected, chunks

    # -- one tick --------------------------------------------------------------------------
    def tick(self) -> list[GenerationResult]:
        """Admit, queue one step, accept tokens: this step's, or with ``run_ahead`` those of the step before.  Returns the
        requests that finished."""
        self.ticks += 1
        done_before = len(self.finished)
        self.admit()
        launched = None
        if self.active:
            selected, chunks = self.build_step()
            if selected:
                launched = self._launch(selected, chunks)
        if self._flying is not None:   # the step before: the new one is queued behind it, now its tokens are waited for
            flying, self._flying = self._flying, None
            self._collect(flying)
        if launched is not None:
            if self.run_ahead:
                self._flying = launched
            else:
                self._collect(launched)
        self.admit()
        return self.finished[done_before:]

    def run(self) -> list[GenerationResult]:
        """Ticks until nothing is waiting, active or in flight; returns everything that finished."""
        start = len(self.finished)
        while self.has_work():
            before = (len(self.waiting), len(self.active), len(self.finished))
            self.tick()
            if not self.active and self._flying is None and self.waiting and before == (len(self.waiting), 0, len(self.finished)):
                raise RuntimeError("a waiting request can never be admitted")   # guarded by add(); defensive
        return self.finished[start:]

    def _fail_step(self, selected: Sequence[Request], error: BaseException) -> None:
        """The step's requests fail; the others go on."""
        logger.error("model_batch_failed requests=%s error=%r", [request.request_id for request in selected], error)
        for request in selected:
            if request in self.active or request in self.leaving:
                self._finish(request, "error", error)

    def _launch(self, selected: list[Request], chunks: list[list[int]]) -> Optional["_Launched"]:
        """Queues the step and the choice of its tokens; waits for nothing."""
        entries, ready, prompt_rows = [], [], []
        for request, chunk in zip(selected, chunks):
            decodes = not request.prefilling
            samples = decodes or request.prompt_offset + len(chunk) >= len(request.prompt)
            source = None if request.in_flight is None else (request.in_flight[0].device, request.in_flight[1])
            entries.append(StepEntry(request.cache, chunk, (len(chunk) - 1,) if samples else (), source))
            prompt_rows.append(not decodes)
            if samples:
                ready.append(request)
        self.last_step = [(request.request_id, len(chunk)) for request, chunk in zip(selected, chunks)]
        started = self.clock()
        try:
            logits = self.run_step(entries)
            if not ready:
                tokens = _Known([])
            elif hasattr(self.sample, "launch"):
                tokens = self.sample.launch(logits, [r.sampling for r in ready], [r.random for r in ready])
            else:
                tokens = _Known(self.sample(logits, [r.sampling for r in ready], [r.random for r in ready]))
        except Exception as error:
            self._fail_step(selected, error)
            return None
        for request, chunk, prompt_row in zip(selected, chunks, prompt_rows):
            if prompt_row:
                request.prompt_offset += len(chunk)
        for row, request in enumerate(ready):
            request.pending_token = None
            request.in_flight = (tokens, row)
            request.launched += 1
            if self.run_ahead and len(request.output_ids) + request.launched >= request.sampling.max_new_tokens:
                # The token being chosen is the request's last whatever it is, and no later step will read its cache: slot
                # and pages go back now, a tick before the token is here, so that a waiting request can have them (the
                # device runs its steps in the order they were queued: whoever gets the pages writes them after this step).
                self._release(request)
                self.active.remove(request)
                self.leaving.append(request)
        return _Launched(selected, chunks, prompt_rows, ready, tokens, started)

    def _collect(self, step: "_Launched") -> None:
        """Waits for a queued step's tokens and accepts them."""
        try:
            tokens = step.tokens.result()
        except Exception as error:
            self._fail_step(step.selected, error)
            return
        now = self.clock()
        elapsed = now - max(step.started, self._collected_at)
        self._collected_at = now
        for request, chunk, prompt_row in zip(step.selected, step.chunks, step.prompt_rows):
            if request not in self.active and request not in self.leaving:
                continue   # finished (a stop id in the step before, an error, an abort) while this step was in flight
            if prompt_row:
                request.prompt_progress_at = now
                request.prefill_seconds += elapsed
            else:
                request.inter_token_seconds.append(elapsed)
        for request, token in zip(step.ready, tokens):
            if request not in self.active and request not in self.leaving:
                continue   # likewise: the token is dropped
            request.launched -= 1
            if request.in_flight is not None and request.in_flight[0] is step.tokens:
                request.in_flight = None   # no later step has taken it on the device: it is fed from here
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
        if request.in_flight is None:
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
        for holding in (self.active, self.leaving):
            if request in holding:
                holding.remove(request)
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
