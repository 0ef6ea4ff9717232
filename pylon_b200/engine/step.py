"""The step function: one batch of (request, its next tokens) through the model.

A step may hold portions of prompts beside single decoded tokens, cut anywhere.  It runs
only the tokens it is given, as one batch, against what earlier steps left in the cache,
and returns float32 logits at the wanted places.  Nothing else in the engine runs the
model: generation, the scheduler and trace replay all come through here.

Counterpart in raun6k/Pylon: ``Decoder.packed_caches`` with
``PackedBatchCache.prepare_packed`` (src/pylon/decode/runner.py:271-302,
src/pylon/kv/cache.py:380-455).  Differences: logits may be asked at any token of a row,
not only its last; all metadata of a step travels in one pinned int32 buffer and one copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from pylon_b200.cache.manager import CacheManager, RequestCache
from pylon_b200.models.decoder import DecoderModel
from pylon_b200.parts.base import StepView


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and which of them want logits
    (indices into ``tokens``)."""

    request: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)
    # (int32 tokens on the device, row): the entry's one token is that one - what the sampling kernel chose for the request
    # in the step before, not read back yet - and ``tokens`` holds any valid id in its place.  All such entries of a step
    # name the same tensor.
    source: Optional[tuple[torch.Tensor, int]] = None


def _aligned(count: int) -> int:
    return (count + 3) & ~3   # sections start on 16-byte boundaries


@dataclass
class StepLayout:
    """Where each array of a step lies in the step's one int32 buffer."""

    tokens: int
    rows: int
    logits: int
    table_widths: tuple[int, ...]
    offsets: dict[str, int] = field(default_factory=dict)
    total: int = 0

    def __post_init__(self) -> None:
        cursor = 0
        sections = [
            ("token_ids", self.tokens), ("positions", self.tokens), ("token_row", self.tokens), ("token_source", self.tokens),
            ("q_start", self.rows + 1), ("kv_len", self.rows), ("slots", self.rows), ("logit_rows", max(1, self.logits)),
        ] + [(f"block_table_{g}", self.rows * width) for g, width in enumerate(self.table_widths)]
        for name, size in sections:
            self.offsets[name] = cursor
            cursor += _aligned(size)
        self.total = cursor


class StepFunction:
    def __init__(self, model: DecoderModel, cache: CacheManager) -> None:
        if model.device is None:
            raise RuntimeError("the model has no weights yet")
        self.model = model
        self.cache = cache
        self.device = model.device
        self.dtype = model.dtype
        self.vocab_size = model.spec.vocab_size
        self.max_positions = model.spec.max_positions
        self.graphs = None

    def enable_graphs(self) -> None:
        """Steps of the shapes a scheduler makes are replayed from CUDA graphs from now on: decode-only steps (one token
        per request, logits wanted for each) from a graph of their exact batch size, steps that bring prompt portions from a
        graph of the next larger captured size, padded.  The logits tensor such a step returns is reused by the next step
        that replays the same graph."""
        from pylon_b200.engine.graphs import StepGraphs

        self.graphs = StepGraphs(self)

    # -- host side ---------------------------------------------------------------------
    def fill(self, entries: Sequence[StepEntry], layout: StepLayout, buffer: np.ndarray) -> tuple[int, int]:
        """Writes the step's arrays into ``buffer`` (int32, ``layout.total`` long) and returns
        (longest row, longest context)."""
        off = layout.offsets
        cursor = 0
        wanted = 0
        max_q = max_kv = 0
        buffer[off["q_start"]] = 0
        for row, entry in enumerate(entries):
            count = len(entry.tokens)
            start = entry.request.length
            buffer[off["token_ids"] + cursor : off["token_ids"] + cursor + count] = entry.tokens
            buffer[off["positions"] + cursor : off["positions"] + cursor + count] = np.arange(start, start + count, dtype=np.int32)
            buffer[off["token_row"] + cursor : off["token_row"] + cursor + count] = row
            buffer[off["token_source"] + cursor : off["token_source"] + cursor + count] = -1 if entry.source is None else entry.source[1]
            for index in entry.want:
                buffer[off["logit_rows"] + wanted] = cursor + index
                wanted += 1
            cursor += count
            buffer[off["q_start"] + row + 1] = cursor
            buffer[off["kv_len"] + row] = start + count
            buffer[off["slots"] + row] = entry.request.slot
            max_q, max_kv = max(max_q, count), max(max_kv, start + count)
        requests = [entry.request for entry in entries]
        for g, width in enumerate(layout.table_widths):
            table = self.cache.block_table(requests, g, width)
            base = off[f"block_table_{g}"]
            buffer[base : base + table.size] = table.reshape(-1)
        return max_q, max_kv

    def fill_padded(self, ones: Sequence[StepEntry], portions: Sequence[StepEntry], order: Sequence[StepEntry], layout: StepLayout,
                    buffer: np.ndarray, one_rows: int) -> None:
        """The arrays of a step padded to a captured size (see ``StepView.padded``): rows ``[0, one_rows)`` are for the
        entries that bring one token (``ones``; the rows beyond them have no tokens), rows ``[one_rows, layout.rows)`` for
        the others (``portions``; likewise); the tokens of all of them lie side by side and padding tokens follow.  Logits
        are asked for in the order of ``order`` (the caller's entries), at the last token of each entry that wants any."""
        off = layout.offsets
        for name in ("token_ids", "positions"):
            buffer[off[name] : off[name] + layout.tokens] = 0
        buffer[off["token_row"] : off["token_row"] + layout.tokens] = -1
        buffer[off["token_source"] : off["token_source"] + layout.tokens] = -1
        for name in ("kv_len", "slots"):
            buffer[off[name] : off[name] + layout.rows] = 0
        buffer[off["logit_rows"] : off["logit_rows"] + max(1, layout.logits)] = 0
        last_token: dict[int, int] = {}
        cursor = 0
        starts = np.zeros(layout.rows + 1, dtype=np.int32)
        placed: list[Optional[StepEntry]] = [None] * layout.rows
        for row, entry in list(enumerate(ones)) + [(one_rows + index, entry) for index, entry in enumerate(portions)]:
            placed[row] = entry
        for row in range(layout.rows):
            starts[row] = cursor
            entry = placed[row]
            if entry is None:
                continue
            count, start = len(entry.tokens), entry.request.length
            buffer[off["token_ids"] + cursor : off["token_ids"] + cursor + count] = entry.tokens
            buffer[off["positions"] + cursor : off["positions"] + cursor + count] = np.arange(start, start + count, dtype=np.int32)
            buffer[off["token_row"] + cursor : off["token_row"] + cursor + count] = row
            if entry.source is not None:
                buffer[off["token_source"] + cursor] = entry.source[1]
            buffer[off["kv_len"] + row] = start + count
            buffer[off["slots"] + row] = entry.request.slot
            cursor += count
            last_token[id(entry)] = cursor - 1
        starts[layout.rows] = cursor
        buffer[off["q_start"] : off["q_start"] + layout.rows + 1] = starts
        wanted = 0
        for entry in order:
            if entry.want:
                buffer[off["logit_rows"] + wanted] = last_token[id(entry)]
                wanted += 1
        for g, width in enumerate(layout.table_widths):
            table = np.full((layout.rows, width), -1, dtype=np.int32)
            for row, entry in enumerate(placed):
                if entry is not None:
                    pages = entry.request.tables[g]
                    table[row, : len(pages)] = pages
            base = off[f"block_table_{g}"]
            buffer[base : base + table.size] = table.reshape(-1)

    @staticmethod
    def rows_alike(entries: Sequence[StepEntry]) -> bool:
        """Whether the requests of the step hold about equally many tokens after it: the longest
        at most an eighth above the mean (see :class:`~pylon_b200.parts.base.StepView`)."""
        lengths = [entry.request.length + len(entry.tokens) for entry in entries]
        return max(lengths) * len(lengths) * 8 <= sum(lengths) * 9

    @staticmethod
    def sampled_source(entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """The tensor of sampled tokens that entries of the step take their token from, or ``None``."""
        for entry in entries:
            if entry.source is not None:
                return entry.source[0]
        return None

    def take_sampled(self, device_buffer: torch.Tensor, layout: StepLayout, sampled: Optional[torch.Tensor]) -> None:
        """After the step's arrays are on the device: the tokens that come from ``sampled`` are put in their places."""
        if sampled is None:
            return
        from pylon_b200.kernels import ops

        off = layout.offsets
        ops.take_tokens(device_buffer[off["token_ids"] : off["token_ids"] + layout.tokens],
                        device_buffer[off["token_source"] : off["token_source"] + layout.tokens], sampled)

    def validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise ValueError("a step needs at least one entry")
        sampled = self.sampled_source(entries)
        for entry in entries:
            count = len(entry.tokens)
            if count < 1:
                raise ValueError(f"request {entry.request.request_id!r} brings no tokens")
            if entry.source is not None:
                tensor, row = entry.source
                if count != 1 or tensor is not sampled or not 0 <= int(row) < tensor.shape[0]:
                    raise ValueError(f"request {entry.request.request_id!r}: a token taken from the device is one token, a row of the one tensor "
                                     "of sampled tokens that the step names")
            for token in entry.tokens:
                if not 0 <= int(token) < self.vocab_size:
                    raise ValueError(f"token id {token} is outside the vocabulary [0, {self.vocab_size})")
            for index in entry.want:
                if not 0 <= int(index) < count:
                    raise ValueError(f"request {entry.request.request_id!r} wants logits at place {index} of {count} tokens")
            if entry.request.length + count > self.max_positions:
                raise ValueError(
                    f"request {entry.request.request_id!r} would reach {entry.request.length + count} tokens; "
                    f"the engine was set up for at most {self.max_positions}"
                )

    def view(self, device_buffer: torch.Tensor, layout: StepLayout, max_q: int, max_kv: int) -> tuple[StepView, list[torch.Tensor]]:
        off = layout.offsets
        step = StepView()
        step.token_ids = device_buffer[off["token_ids"] : off["token_ids"] + layout.tokens]
        step.positions = device_buffer[off["positions"] : off["positions"] + layout.tokens]
        step.token_row = device_buffer[off["token_row"] : off["token_row"] + layout.tokens]
        step.q_start = device_buffer[off["q_start"] : off["q_start"] + layout.rows + 1]
        step.kv_len = device_buffer[off["kv_len"] : off["kv_len"] + layout.rows]
        step.slots = device_buffer[off["slots"] : off["slots"] + layout.rows]
        step.logit_rows = device_buffer[off["logit_rows"] : off["logit_rows"] + layout.logits]
        step.num_tokens, step.num_rows, step.num_logits = layout.tokens, layout.rows, layout.logits
        step.max_q, step.max_kv = max_q, max_kv
        step.dtype, step.device = self.dtype, self.device
        tables = [
            device_buffer[off[f"block_table_{g}"] : off[f"block_table_{g}"] + layout.rows * width].view(layout.rows, width)
            for g, width in enumerate(layout.table_widths)
        ]
        return step, tables

    # -- the step ----------------------------------------------------------------------
    def __call__(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs the step; returns logits ``[wanted, vocab]`` in the order of the entries and of
        their ``want`` lists, or ``None`` if nothing is wanted.  The cache is advanced only
        after every launch was enqueued; if preparing or launching fails, the requests hold
        what they held before: their pages, and (where a mixer keeps a state of fixed size) a
        copy of their state slots taken before the first launch."""
        self.validate(entries)
        batch = [(entry.request, len(entry.tokens)) for entry in entries]
        self.cache.prepare(batch)          # all pages of the step, or OutOfPages and nothing
        saved_state = None
        try:
            saved_state = self.cache.save_state([request for request, _ in batch])   # None for models without state
            logits = None
            if self.graphs is not None:
                logits = self.graphs.run(entries)
            if logits is None:
                logits = self._run_eager(entries)
        except BaseException:
            for request, _ in batch:
                self.cache.rollback(request)
            self.cache.restore_state(saved_state)
            raise
        for request, _ in batch:
            self.cache.commit(request)
        return logits

    def _run_eager(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        requests = [entry.request for entry in entries]
        widths = tuple(
            max(1, max(len(request.tables[g]) for request in requests)) for g in range(len(self.cache.groups))
        )
        layout = StepLayout(
            tokens=sum(len(entry.tokens) for entry in entries),
            rows=len(entries),
            logits=sum(len(entry.want) for entry in entries),
            table_widths=widths,
        )
        host = torch.empty(layout.total, dtype=torch.int32, pin_memory=True)
        max_q, max_kv = self.fill(entries, layout, host.numpy())
        device_buffer = host.to(self.device, non_blocking=True)
        self.take_sampled(device_buffer, layout, self.sampled_source(entries))
        step, tables = self.view(device_buffer, layout, max_q, max_kv)
        step.row_tokens = tuple(len(entry.tokens) for entry in entries)
        step.rows_alike = self.rows_alike(entries)
        return self.model.forward(step, self.cache.layer_caches(tables))
