"""Decode steps replayed from CUDA graphs, one or two graphs per batch size.

A step in which every request brings one token and wants its logits has the same launches
every time; only the small integer arrays of the step (tokens, positions, lengths, block
tables) change.  Such a step is captured once per batch size into a ``torch.cuda.CUDAGraph``
over a static copy of those arrays; afterwards a step is one pinned-to-device copy and one
graph launch.  Kernels read every length from the device, so a graph captured at one
context length serves all of them: the decode attention divides the key tiles among its
blocks inside the kernel, from the lengths of the step at hand.  What a graph does freeze is
the form of its launches, and the decode attention has two: one for any lengths, and a faster
one for a few requests of about equal length (``StepView.rows_alike``).  So a batch size may
have two graphs, and each step replays the one that fits its requests' lengths.

As in raun6k/Pylon (src/pylon/decode/graph.py:157-242): one graph per exact batch size, no
padding to a larger one; a size whose capture failed is not tried again and runs eagerly;
sampling stays outside the graph.
"""
from __future__ import annotations

import gc
import sys
import weakref
from typing import Optional, Sequence

import torch

from pylon_b200.engine.step import StepEntry, StepLayout


class CapturedStep:
    def __init__(self, graph: torch.cuda.CUDAGraph, layout: StepLayout, static_buffer: torch.Tensor, logits: torch.Tensor, launches: int) -> None:
        self.graph = graph
        self.layout = layout
        self.static_buffer = static_buffer
        self.logits = logits
        self.launches = launches    # kernels of this package inside the graph


class DecodeGraphs:
    def __init__(self, step_function) -> None:
        # a proxy, not a reference: the step function owns this object, and a cycle would leave
        # graphs to the garbage collector, which must not destroy one while another is captured
        self.step_function = weakref.proxy(step_function)
        self.cache = step_function.cache
        self.device = step_function.device
        self.captured: dict[int, CapturedStep] = {}         # by batch size: for requests of any lengths
        self.captured_alike: dict[int, CapturedStep] = {}   # by batch size: for requests of about equal length
        self.force_alike: Optional[bool] = None             # set while graphs are captured ahead of use
        self.failed: set[int] = set()
        self.pool = None
        self.max_context = step_function.max_positions
        self.widths = tuple(max(1, group.pages_for(self.max_context)) for group in self.cache.groups)

    @staticmethod
    def applies(entries: Sequence[StepEntry]) -> bool:
        return all(len(entry.tokens) == 1 and tuple(entry.want) == (0,) for entry in entries)

    def _layout(self, batch: int) -> StepLayout:
        return StepLayout(tokens=batch, rows=batch, logits=batch, table_widths=self.widths)

    def capture(self, entries: Sequence[StepEntry], alike: bool) -> Optional[CapturedStep]:
        """Captures the graph of ``len(entries)`` rows, in the form for requests of about equal
        length or in the one for any lengths, using ``entries`` (already prepared in the cache)
        as the example step.  Returns ``None`` and remembers the size if capture fails."""
        from pylon_b200.kernels import ops

        batch = len(entries)
        function = self.step_function
        layout = self._layout(batch)
        static_buffer = torch.zeros(layout.total, dtype=torch.int32, device=self.device)
        host = torch.empty(layout.total, dtype=torch.int32, pin_memory=True)
        function.fill(entries, layout, host.numpy())
        static_buffer.copy_(host, non_blocking=True)
        step, tables = function.view(static_buffer, layout, 1, self.max_context)
        step.rows_alike = alike
        caches = self.cache.layer_caches(tables)
        collector_was_on = gc.isenabled()
        gc.disable()   # destroying an old graph or a pinned buffer in mid-capture would invalidate it
        try:
            # One eager run first: libraries are built and loaded, kernels configured, the
            # allocator warmed.  It writes the same cache slots the replay writes again; a state
            # of fixed size, which a second run would advance twice, is put back after it.
            saved_state = self.cache.save_state([entry.request for entry in entries])
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
            self.failed.add(batch)
            print(f"[pylon_b200] cuda graph capture failed for batch size {batch}: {error!r}", file=sys.stderr, flush=True)
            torch.cuda.synchronize(self.device)
            return None
        finally:
            if collector_was_on:
                gc.enable()
        captured = CapturedStep(graph, layout, static_buffer, logits, launches)
        (self.captured_alike if alike else self.captured)[batch] = captured
        return captured

    def run(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs a prepared decode step from its graph; ``None`` if this size has no graph (the
        caller then runs eagerly)."""
        from pylon_b200.kernels import ops

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
        captured.static_buffer.copy_(host, non_blocking=True)
        captured.graph.replay()
        ops.launches[0] += captured.launches
        return captured.logits
