"""Steps replayed from CUDA graphs.

An eager step is some nine launches a layer through Python; for a step of a few hundred
tokens the host takes several times longer over them than the device takes to run them.
A captured step is one pinned-to-device copy of the step's small integer arrays (tokens,
positions, lengths, block tables) and one graph launch.  Kernels read every length from the
device, so a graph captured at one context length serves all of them.

**Decode steps** (every request brings one token and wants its logits): one graph per exact
batch size, no padding to a larger one, as in raun6k/Pylon (src/pylon/decode/graph.py:157-242).
What a graph does freeze is the form of its launches, and the decode attention has two: one
for any lengths, and a faster one for a few requests of about equal length
(``StepView.rows_alike``).  So a batch size may have two graphs, and each step replays the
one that fits its requests' lengths.

**Steps with prompt portions** (the scheduler's mixed ticks: a token for every decoding
request beside portions of waiting prompts, logits wanted at most at the last token of an
entry).  The reference runs these eagerly (src/pylon/engine.py:269-300).  Here they are padded
to the next captured size — a number of one-token rows, a number of portion rows and a number
of portion tokens, each rounded up to a bucket — and replayed from the graph of that size:
rows without tokens and tokens without a row are skipped by the kernels (``StepView.padded``).
Only a model whose parts all take padding is given such steps.

A size whose capture failed is not tried again and runs eagerly; sampling stays outside the
graphs.
"""
from __future__ import annotations

import gc
import sys
import weakref
from typing import Optional, Sequence

import torch

from pylon_b200.engine.step import StepEntry, StepLayout

MAX_PADDED_GRAPHS = 192   # sizes captured at most; steps of further sizes run eagerly


def bucket_rows(count: int) -> int:
    """Rows are padded to 0, 1, 2, 4, 8, ... (powers of two)."""
    return 0 if count <= 0 else 1 << (count - 1).bit_length()


def bucket_tokens(count: int) -> int:
    """Portion tokens are padded to a multiple of 32 up to 256, of 64 up to 512, of 128 up to 2,048, of 256 beyond:
    at most an eighth more work than the step has, for a few dozen sizes."""
    for limit, grain in ((256, 32), (512, 64), (2_048, 128)):
        if count <= limit:
            return max(grain, -(-count // grain) * grain)
    return -(-count // 256) * 256


class CapturedStep:
    def __init__(self, graph: torch.cuda.CUDAGraph, layout: StepLayout, static_buffer: torch.Tensor, logits: Optional[torch.Tensor], launches: int) -> None:
        self.graph = graph
        self.layout = layout
        self.static_buffer = static_buffer
        self.logits = logits
        self.launches = launches    # kernels of this package inside the graph


class StepGraphs:
    def __init__(self, step_function) -> None:
        # a proxy, not a reference: the step function owns this object, and a cycle would leave
        # graphs to the garbage collector, which must not destroy one while another is captured
        self.step_function = weakref.proxy(step_function)
        self.cache = step_function.cache
        self.device = step_function.device
        self.captured: dict[int, CapturedStep] = {}         # by batch size: for requests of any lengths
        self.captured_alike: dict[int, CapturedStep] = {}   # by batch size: for requests of about equal length
        self.captured_padded: dict[tuple[int, int, int], CapturedStep] = {}   # by (one-token rows, portion rows, portion tokens)
        self.force_alike: Optional[bool] = None             # set while graphs are captured ahead of use
        self.failed: set = set()                            # batch sizes and padded sizes whose capture failed
        self.pool = None
        self.max_context = step_function.max_positions
        self.widths = tuple(max(1, group.pages_for(self.max_context)) for group in self.cache.groups)
        self.pad_steps = step_function.model.takes_padding()
        self.seen_padded: dict[tuple[int, int, int], int] = {}   # how often a size without a graph has come up
        self.capture_at_once = False                         # set while graphs are captured ahead of use
        self.replays = {"decode": 0, "padded": 0}

    # -- which steps -----------------------------------------------------------------------
    @staticmethod
    def decode_only(entries: Sequence[StepEntry]) -> bool:
        return all(len(entry.tokens) == 1 and tuple(entry.want) == (0,) for entry in entries)

    @staticmethod
    def scheduler_shaped(entries: Sequence[StepEntry]) -> bool:
        """Logits wanted nowhere or at the last token of an entry: what a scheduler's ticks ask for."""
        return all(len(entry.want) == 0 or tuple(entry.want) == (len(entry.tokens) - 1,) for entry in entries)

    def run(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs a prepared step from a graph; ``None`` if it has none (the caller then runs eagerly)."""
        if self.decode_only(entries):
            return self.run_decode(entries)
        if self.pad_steps and self.scheduler_shaped(entries):
            return self.run_padded(entries)
        return None

    # -- capture -----------------------------------------------------------------------------
    def _capture(self, key, step, caches, layout: StepLayout, static_buffer: torch.Tensor, state_of: Sequence[StepEntry]) -> Optional[CapturedStep]:
        from pylon_b200.kernels import ops

        function = self.step_function
        collector_was_on = gc.isenabled()
        gc.disable()   # destroying an old graph or a pinned buffer in mid-capture would invalidate it
        try:
            # One eager run first: libraries are built and loaded, kernels configured, the
            # allocator warmed.  It writes the same cache slots the replay writes again; a state
            # of fixed size, which a second run would advance twice, is put back after it.
            saved_state = self.cache.save_state([entry.request for entry in state_of])
            function.model.forward(step, caches)
            self.cache.restore_state(saved_state)
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            before = ops.launches[0]
            with torch.cuda.graph(graph, pool=self.pool):
                logits = function.model.forward(step, caches)
            launches = ops.launches[0] - before
            if self.pool is None:
                self.pool = graph.pool()
        except Exception as error:
            # raun6k/Pylon logs "cuda_graph_capture_failed" and goes on eagerly
            # (src/pylon/decode/warmup.py:123-137); so does this engine.
            self.failed.add(key)
            print(f"[pylon_b200] cuda graph capture failed for step size {key}: {error!r}", file=sys.stderr, flush=True)
            torch.cuda.synchronize(self.device)
            return None
        finally:
            if collector_was_on:
                gc.enable()
        return CapturedStep(graph, layout, static_buffer, logits, launches)

    def _replay(self, captured: CapturedStep, host: torch.Tensor, kind: str, sampled: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        from pylon_b200.kernels import ops

        captured.static_buffer.copy_(host, non_blocking=True)
        self.step_function.take_sampled(captured.static_buffer, captured.layout, sampled)   # tokens the host does not know yet
        captured.graph.replay()
        ops.launches[0] += captured.launches
        self.replays[kind] += 1
        return captured.logits

    # -- decode steps: the exact batch size ----------------------------------------------------
    def _layout(self, batch: int) -> StepLayout:
        return StepLayout(tokens=batch, rows=batch, logits=batch, table_widths=self.widths)

    def capture(self, entries: Sequence[StepEntry], alike: bool) -> Optional[CapturedStep]:
        """Captures the graph of ``len(entries)`` decoding rows, in the form for requests of about equal
        length or in the one for any lengths, using ``entries`` (already prepared in the cache)
        as the example step.  Returns ``None`` and remembers the size if capture fails."""
        batch = len(entries)
        function = self.step_function
        layout = self._layout(batch)
        static_buffer = torch.zeros(layout.total, dtype=torch.int32, device=self.device)
        host = torch.empty(layout.total, dtype=torch.int32, pin_memory=True)
        function.fill(entries, layout, host.numpy())
        static_buffer.copy_(host, non_blocking=True)
        step, tables = function.view(static_buffer, layout, 1, self.max_context)
        step.rows_alike = alike
        captured = self._capture(batch, step, self.cache.layer_caches(tables), layout, static_buffer, entries)
        if captured is not None:
            (self.captured_alike if alike else self.captured)[batch] = captured
        return captured

    def run_decode(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        batch = len(entries)
        if batch in self.failed:
            return None
        alike = self.step_function.rows_alike(entries) if self.force_alike is None else self.force_alike
        captured = (self.captured_alike if alike else self.captured).get(batch)
        if captured is None:
            captured = self.capture(entries, alike)
            if captured is None:
                return None
            # the capture itself launched nothing; fall through to the first replay
        host = torch.empty(captured.layout.total, dtype=torch.int32, pin_memory=True)
        self.step_function.fill(entries, captured.layout, host.numpy())
        return self._replay(captured, host, "decode", self.step_function.sampled_source(entries))

    # -- steps with prompt portions: padded to a captured size ------------------------------------
    def padded_size(self, entries: Sequence[StepEntry]) -> tuple[tuple[int, int, int], list[StepEntry], list[StepEntry]]:
        ones = [entry for entry in entries if len(entry.tokens) == 1]
        portions = [entry for entry in entries if len(entry.tokens) > 1]
        key = (bucket_rows(len(ones)), bucket_rows(len(portions)), bucket_tokens(sum(len(entry.tokens) for entry in portions)))
        return key, ones, portions

    def run_padded(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        key, ones, portions = self.padded_size(entries)
        if key in self.failed:
            return None
        one_rows, portion_rows, portion_tokens = key
        wanted = sum(1 for entry in entries if entry.want)
        captured = self.captured_padded.get(key)
        function = self.step_function
        if captured is None:
            # A capture costs about two eager steps.  A size that comes up once (an odd prompt length beside an odd number
            # of decoding requests) is not worth one; a size that comes back is.
            self.seen_padded[key] = self.seen_padded.get(key, 0) + 1
            if len(self.captured_padded) >= MAX_PADDED_GRAPHS or (self.seen_padded[key] < 2 and not self.capture_at_once):
                return None
            # every row may want logits at its last token
            layout = StepLayout(tokens=one_rows + portion_tokens, rows=one_rows + portion_rows, logits=one_rows + portion_rows, table_widths=self.widths)
            static_buffer = torch.zeros(layout.total, dtype=torch.int32, device=self.device)
            host = torch.empty(layout.total, dtype=torch.int32, pin_memory=True)
            function.fill_padded(ones, portions, entries, layout, host.numpy(), one_rows)
            static_buffer.copy_(host, non_blocking=True)
            step, tables = function.view(static_buffer, layout, portion_tokens, self.max_context)
            step.padded = True
            # what the parts may plan their launches by must hold for every step of this size: rows of one token, then
            # rows that may bring up to all the portion tokens
            step.row_tokens = (1,) * one_rows + (portion_tokens,) * portion_rows
            captured = self._capture(key, step, self.cache.layer_caches(tables), layout, static_buffer, entries)
            if captured is None:
                return None
            self.captured_padded[key] = captured
        host = torch.empty(captured.layout.total, dtype=torch.int32, pin_memory=True)
        function.fill_padded(ones, portions, entries, captured.layout, host.numpy(), one_rows)
        logits = self._replay(captured, host, "padded", self.step_function.sampled_source(entries))
        return logits[:wanted] if wanted else None


DecodeGraphs = StepGraphs   # the name this class had while it replayed decode steps only
