"""The cache manager: pages of keys and values with a block table per request, in groups,
and slots of fixed-size state per request.

* Runs of the model whose mixers need the same kind of key/value cache (same KV heads, row
  widths and window) form a **group**.  Each group has pages of its own: one pool of page
  numbers - as many pages as that group needs, which for a windowed group is far fewer than
  for one that keeps everything -, a device tensor of key rows ``[runs, pages, kv_heads,
  page_size, head_dim]``, one of value rows of the width the group's mixers ask for (or none,
  for a mixer that keeps one row per token), and for every request one table *logical page ->
  physical page*.
* Pages are acquired just before the step that writes them (all of a step or none), given
  back when the request is closed, and — in a windowed group — as soon as every position
  on them lies behind the window of every token still to come.  Free pages are reused
  last-in first-out.
* Every open request also holds a **slot**; mixers that keep a state of fixed size find
  theirs at ``state[slot]``.  States are zeroed when the slot is taken.  Qwen3 has none.

Host bookkeeping is plain Python and needs no GPU; device tensors are only allocated when a
device is given.  Compared with raun6k/Pylon (src/pylon/kv/pool.py:19-75,
src/pylon/kv/cache.py:20-135, 380-455): same lazy all-or-nothing acquisition and LIFO
reuse; ownership is explicit (a page is held by exactly one request) instead of resting on
garbage-collector finalizers, and there are groups, windows and state slots.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, Mapping, Optional, Sequence, Union

import numpy as np
import torch

from pylon_b200.parts.base import CacheNeed, KVNeed, LayerCache, StateNeed


class OutOfPages(RuntimeError):
    """A step needs more pages than a group has free.  Nothing was acquired."""


class CacheError(RuntimeError):
    """The manager was used against its rules (a page freed twice, a closed request...)."""


# ---------------------------------------------------------------------------------------
class PagePool:
    """Page numbers of one group: who is free, who is held."""

    def __init__(self, num_pages: int) -> None:
        if num_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free = list(range(self.num_pages - 1, -1, -1))  # page 0 is handed out first
        self._held = [False] * self.num_pages
        self.acquired_total = 0   # pages handed out over the pool's life (shows reuse)

    @property
    def free_count(self) -> int:
        return len(self._free)

    def acquire(self, count: int) -> list[int]:
        if count < 0:
            raise ValueError("page count must not be negative")
        if count > len(self._free):
            raise OutOfPages(f"{count} pages wanted, {len(self._free)} free")
        pages = [self._free.pop() for _ in range(count)]
        for page in pages:
            if self._held[page]:
                raise CacheError(f"page {page} was on the free list while held")
            self._held[page] = True
        self.acquired_total += count
        return pages

    def release(self, pages: Iterable[int]) -> None:
        for page in pages:
            if not 0 <= page < self.num_pages:
                raise CacheError(f"page {page} does not exist")
            if not self._held[page]:
                raise CacheError(f"page {page} is freed twice")
            self._held[page] = False
            self._free.append(page)

    def held_pages(self) -> set[int]:
        return {page for page, held in enumerate(self._held) if held}


# ---------------------------------------------------------------------------------------
@dataclass
class CacheGroup:
    need: KVNeed
    runs: list[int]                      # positions in the model's run order
    pool: PagePool
    page_size: int
    keys: Optional[torch.Tensor] = None      # [runs, pages, kv_heads, page_size, head_dim]
    values: Optional[torch.Tensor] = None    # [runs, pages, kv_heads, page_size, value width]; None if the need has no value rows

    def pages_for(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size

    def lifetime_pages(self, capacity: int, max_step_tokens: int) -> int:
        """Most pages a request of ``capacity`` tokens holds at any time in this group, when
        no step brings it more than ``max_step_tokens`` tokens."""
        full = self.pages_for(capacity)
        if self.need.window is None:
            return full
        # A step's tokens plus the window before its first token, not page aligned.
        span = min(capacity, self.need.window - 1 + max(1, max_step_tokens))
        return min(full, self.pages_for(span) + 1)

    def bytes_per_token(self, element_size: Optional[int] = None) -> int:
        if element_size is None:
            element_size = 0 if self.keys is None else self.keys.element_size()
        return len(self.runs) * self.need.n_kv_heads * (self.need.head_dim + self.need.value_width) * element_size


@dataclass
class RequestCache:
    """What one open request holds."""

    request_id: object
    slot: int
    capacity: int
    length: int = 0
    pending: int = 0                                  # tokens prepared but not committed
    tables: list[list[int]] = field(default_factory=list)   # per group: logical -> physical, -1 = none
    closed: bool = False

    def held(self, group: int) -> list[int]:
        return [page for page in self.tables[group] if page >= 0]


def group_page_counts(needs: Sequence[Optional[CacheNeed]], page_size: int, pool_tokens: int, max_requests: int,
                      longest_request: int, max_step_tokens: int) -> dict[KVNeed, int]:
    """Pages per group for a pool that holds ``pool_tokens`` tokens: a group that keeps every key gets
    ``pool_tokens / page_size`` pages; a windowed group gets what ``max_requests`` requests of
    ``longest_request`` tokens can hold at once (window plus one step's tokens each), if that is fewer."""
    counts: dict[KVNeed, int] = {}
    full = max(1, -(-int(pool_tokens) // page_size))
    for need in needs:
        if need is None or need.kv is None or need.kv in counts:
            continue
        pages = full
        if need.kv.window is not None:
            probe = CacheGroup(need.kv, [], PagePool(1), page_size)
            pages = min(full, max_requests * probe.lifetime_pages(longest_request, max_step_tokens))
        counts[need.kv] = max(1, pages)
    return counts


# ---------------------------------------------------------------------------------------
class CacheManager:
    def __init__(
        self,
        needs: Sequence[Optional[CacheNeed]],
        cache_of: Sequence[Optional[int]],
        *,
        page_size: int,
        num_pages: Union[int, Mapping[KVNeed, int]],
        max_requests: int,
        dtype: torch.dtype = torch.bfloat16,
        device: Optional[torch.device] = None,
    ) -> None:
        """``needs[i]`` / ``cache_of[i]`` describe run ``i`` of the model's order: what its
        mixer keeps, or which earlier run's cache it reads.  ``num_pages``: how many pages of
        ``page_size`` tokens each group gets - one number for all, or a number per
        :class:`KVNeed` (see :func:`group_page_counts`).  ``device=None`` keeps the books only."""
        if page_size < 1:
            raise ValueError("page size must be positive")
        if max_requests < 1:
            raise ValueError("at least one request slot is needed")
        if len(needs) != len(cache_of):
            raise ValueError("needs and cache_of describe different numbers of runs")
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.dtype = dtype
        self.device = None if device is None else torch.device(device)
        self.groups: list[CacheGroup] = []
        self._group_of_run: list[Optional[int]] = [None] * len(needs)
        self._index_in_group: list[int] = [0] * len(needs)
        self._state_needs: list[Optional[StateNeed]] = [None] * len(needs)
        self._states: list[Optional[torch.Tensor]] = [None] * len(needs)
        self._cache_of = list(cache_of)
        by_need: dict[KVNeed, int] = {}
        for run, need in enumerate(needs):
            if need is None:
                continue
            if need.kv is not None:
                if need.kv not in by_need:
                    by_need[need.kv] = len(self.groups)
                    pages = num_pages if isinstance(num_pages, int) else num_pages[need.kv]
                    self.groups.append(CacheGroup(need.kv, [], PagePool(pages), self.page_size))
                group = by_need[need.kv]
                self._group_of_run[run] = group
                self._index_in_group[run] = len(self.groups[group].runs)
                self.groups[group].runs.append(run)
            if need.state is not None:
                self._state_needs[run] = need.state
        if self.device is not None:
            for group in self.groups:
                kv = group.need
                rows = (len(group.runs), group.pool.num_pages, kv.n_kv_heads, self.page_size)
                group.keys = torch.zeros((*rows, kv.head_dim), dtype=dtype, device=self.device)
                if kv.value_width:
                    group.values = torch.zeros((*rows, kv.value_width), dtype=dtype, device=self.device)
            for run, state in enumerate(self._state_needs):
                if state is not None:
                    self._states[run] = torch.zeros((self.max_requests, *state.shape), dtype=state.dtype, device=self.device)
        self._free_slots = list(range(self.max_requests - 1, -1, -1))
        self._open: dict[object, RequestCache] = {}

    # -- sizes ---------------------------------------------------------------------------
    def bytes_per_token(self) -> int:
        return sum(group.bytes_per_token() for group in self.groups)

    def state_bytes_per_request(self) -> int:
        total = 0
        for state in self._state_needs:
            if state is not None:
                total += int(np.prod(state.shape, dtype=np.int64)) * torch.empty((), dtype=state.dtype).element_size()
        return total

    def free_pages(self) -> list[int]:
        return [group.pool.free_count for group in self.groups]

    def free_slots(self) -> int:
        return len(self._free_slots)

    def lifetime_pages(self, capacity: int, max_step_tokens: int) -> list[int]:
        return [group.lifetime_pages(capacity, max_step_tokens) for group in self.groups]

    def open_requests(self) -> list[RequestCache]:
        return list(self._open.values())

    # -- life of a request ---------------------------------------------------------------
    def open(self, request_id: object, capacity: int) -> RequestCache:
        if request_id in self._open:
            raise CacheError(f"request {request_id!r} is open already")
        if capacity < 1:
            raise ValueError("a request needs room for at least one token")
        if not self._free_slots:
            raise CacheError("no request slot is free")
        slot = self._free_slots.pop()
        request = RequestCache(request_id, slot, int(capacity), tables=[[] for _ in self.groups])
        self._open[request_id] = request
        for state in self._states:
            if state is not None:
                state[slot].zero_()
        return request

    def pages_missing(self, request: RequestCache, new_tokens: int) -> list[int]:
        """Pages each group would have to acquire to hold ``new_tokens`` more tokens."""
        end = request.length + request.pending + new_tokens
        return [max(0, group.pages_for(end) - len(request.tables[g])) for g, group in enumerate(self.groups)]

    def prepare(self, batch: Sequence[tuple[RequestCache, int]]) -> None:
        """Acquire the pages that the step ``[(request, new tokens), ...]`` writes: all of
        them or, if any group is short, none (:class:`OutOfPages`)."""
        seen = set()
        for request, count in batch:
            if request.closed or self._open.get(request.request_id) is not request:
                raise CacheError(f"request {request.request_id!r} is not open")
            if id(request) in seen:
                raise CacheError(f"request {request.request_id!r} appears twice in one step")
            seen.add(id(request))
            if count < 1:
                raise ValueError("a step brings each of its requests at least one token")
            if request.pending:
                raise CacheError(f"request {request.request_id!r} has an uncommitted step")
            if request.length + count > request.capacity:
                raise CacheError(
                    f"request {request.request_id!r} would hold {request.length + count} tokens, more than its capacity {request.capacity}"
                )
        wanted = [0] * len(self.groups)
        for request, count in batch:
            for g, missing in enumerate(self.pages_missing(request, count)):
                wanted[g] += missing
        for g, group in enumerate(self.groups):
            if wanted[g] > group.pool.free_count:
                raise OutOfPages(
                    f"the step needs {wanted[g]} new pages in cache group {g}, but only {group.pool.free_count} are free"
                )
        for request, count in batch:
            for g, missing in enumerate(self.pages_missing(request, count)):
                request.tables[g].extend(self.groups[g].pool.acquire(missing))
            request.pending = count

    def commit(self, request: RequestCache) -> None:
        """The prepared tokens are in the cache now; pages a window has passed go back."""
        request.length += request.pending
        request.pending = 0
        for g, group in enumerate(self.groups):
            window = group.need.window
            if window is None:
                continue
            first_needed = request.length - window + 1          # oldest key a later token reads
            dead_pages = max(0, first_needed) // self.page_size  # logical pages wholly before it
            table = request.tables[g]
            freed = [table[i] for i in range(min(dead_pages, len(table))) if table[i] >= 0]
            for i in range(min(dead_pages, len(table))):
                table[i] = -1
            group.pool.release(freed)

    def rollback(self, request: RequestCache) -> None:
        """Undo a prepare whose step did not run: pages beyond the committed length go back."""
        request.pending = 0
        for g, group in enumerate(self.groups):
            keep = group.pages_for(request.length)
            table = request.tables[g]
            group.pool.release([page for page in table[keep:] if page >= 0])
            del table[keep:]

    def close(self, request: RequestCache) -> None:
        if request.closed or self._open.get(request.request_id) is not request:
            raise CacheError(f"request {request.request_id!r} is closed twice")
        for g, group in enumerate(self.groups):
            group.pool.release(request.held(g))
            request.tables[g] = []
        request.closed = True
        request.length = request.pending = 0
        del self._open[request.request_id]
        self._free_slots.append(request.slot)

    # -- fixed-size state across a step that may fail ------------------------------------------
    def has_state(self) -> bool:
        return any(state is not None for state in self._states)

    def save_state(self, requests: Sequence[RequestCache]) -> Optional[list]:
        """Copies of the state slots of ``requests`` (``None`` if no run keeps a state): what
        :meth:`restore_state` puts back when the step that was to advance them did not happen."""
        if not self.has_state() or self.device is None:
            return None
        slots = torch.tensor([request.slot for request in requests], dtype=torch.long, device=self.device)
        return [slots] + [None if state is None else state.index_select(0, slots) for state in self._states]

    def restore_state(self, saved: Optional[list]) -> None:
        if saved is None:
            return
        slots = saved[0]
        for state, copy in zip(self._states, saved[1:]):
            if state is not None:
                state.index_copy_(0, slots, copy)

    # -- what a step hands the kernels -----------------------------------------------------
    def block_table(self, requests: Sequence[RequestCache], group: int, width: Optional[int] = None) -> np.ndarray:
        """int32 ``[rows, width]`` tables of ``requests`` in ``group`` (-1 where no page)."""
        needed = max((len(request.tables[group]) for request in requests), default=1)
        width = max(1, needed) if width is None else width
        if needed > width:
            raise CacheError(f"a block table of width {width} cannot hold {needed} pages")
        table = np.full((len(requests), width), -1, dtype=np.int32)
        for row, request in enumerate(requests):
            pages = request.tables[group]
            table[row, : len(pages)] = pages
        return table

    def layer_caches(self, block_tables: Sequence[torch.Tensor]) -> list[LayerCache]:
        """One :class:`LayerCache` per run; ``block_tables[g]`` is group ``g``'s device table."""
        caches: list[LayerCache] = []
        for run in range(len(self._group_of_run)):
            source = self._cache_of[run]
            if source is not None:
                caches.append(caches[source])
                continue
            cache = LayerCache(page_size=self.page_size, state=self._states[run])
            group = self._group_of_run[run]
            if group is not None:
                index = self._index_in_group[run]
                cache.k_pages = self.groups[group].keys[index]
                cache.v_pages = None if self.groups[group].values is None else self.groups[group].values[index]
                cache.block_table = block_tables[group]
            caches.append(cache)
        return caches

    # -- invariants (tests and debugging) ------------------------------------------------
    def check(self) -> None:
        """No page lost, none held twice; slots likewise."""
        for g, group in enumerate(self.groups):
            owners: dict[int, object] = {}
            for request in self._open.values():
                for page in request.held(g):
                    if page in owners:
                        raise CacheError(f"page {page} of group {g} is held by {owners[page]!r} and {request.request_id!r}")
                    owners[page] = request.request_id
            if set(owners) != group.pool.held_pages():
                raise CacheError(f"group {g}: pages held by requests and pages marked held differ")
            if len(owners) + group.pool.free_count != group.pool.num_pages:
                raise CacheError(f"group {g}: {len(owners)} held + {group.pool.free_count} free != {group.pool.num_pages}")
        slots = [request.slot for request in self._open.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a request slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("a request slot is lost")
