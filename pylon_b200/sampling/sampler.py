"""Chooses the next token of every row that wants one, on the device, in one launch.

Rows of a step may have different options: the kernel takes temperature, top-p and a
uniform number per row (raun6k/Pylon loops over rows when options differ,
src/pylon/engine.py:454-470).  The uniform numbers come from one counter-based generator
per request (Philox keyed by the request's seed), advanced once per sampled token, so what
a request draws does not depend on the batch it is in.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from pylon_b200.kernels import ops
from pylon_b200.sampling.params import SamplingParams


class RequestRandom:
    """The stream of uniform numbers of one request."""

    def __init__(self, seed: int) -> None:
        self._generator = np.random.Generator(np.random.Philox(key=int(seed) % (2**64)))

    def next_uniform(self) -> float:
        return float(self._generator.random(dtype=np.float32))


class SampledTokens:
    """The tokens of one sampling launch: on the device at once (``device``, int32 ``[rows]``, for a next step that
    takes its tokens from there), on the host when :meth:`result` has waited for them."""

    def __init__(self, device_tokens: torch.Tensor, host_copy: torch.Tensor, check_errors: bool, keep: tuple = ()) -> None:
        """``host_copy``: the pinned int32 ``[rows + 4]`` buffer into which the sampling kernel itself writes the tokens
        and the kernels' error words (no copy is queued behind the launch: the next step's work follows it at once).
        ``keep``: pinned buffers the kernel reads, held until it has run."""
        self.device = device_tokens
        self.rows = device_tokens.shape[0]
        self._check_errors = check_errors
        self._host = host_copy
        self._keep = keep
        self._arrived = torch.cuda.Event()
        self._arrived.record()
        self._tokens: Optional[list[int]] = None

    def result(self) -> list[int]:
        """Waits for the launch (and the step before it) and returns the tokens; raises if a kernel of the step reported
        that its result is void."""
        if self._tokens is None:
            self._arrived.synchronize()
            self._keep = ()
            if self._check_errors:
                ops.raise_on_kernel_errors(self.device.device, words=self._host[self.rows:])
            self._tokens = self._host[: self.rows].tolist()
        return self._tokens

    def __del__(self) -> None:
        # The kernel writes into pinned memory that goes back to the allocator with this object: not before it has run.
        if self._tokens is None:
            try:
                self._arrived.synchronize()
            except Exception:
                pass


class Sampler:
    def __init__(self, device: torch.device) -> None:
        self.device = torch.device(device)

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams], randoms: Sequence[Optional[RequestRandom]],
               check_errors: bool = False) -> SampledTokens:
        """``logits``: float32 ``[rows, vocab]`` on the device.  Starts the choice of one token per row and their copy to
        the host, and returns without waiting.  ``check_errors``: the kernels' error words travel with the tokens."""
        rows = logits.shape[0]
        if rows != len(params) or rows != len(randoms):
            raise ValueError("one set of sampling options and one random stream per row of logits")
        host_copy = torch.zeros((rows + 4,), dtype=torch.int32, pin_memory=True)
        if all(p.greedy for p in params):
            return SampledTokens(ops.sample(logits, host_copy=host_copy), host_copy, check_errors)
        # The kernel reads the rows' options where the host wrote them: a copy to the device would stand between this
        # step's last kernel and the next step's first.
        options = torch.empty((3, rows), dtype=torch.float32, pin_memory=True)
        values = options.numpy()
        for row, (p, random) in enumerate(zip(params, randoms)):
            values[0, row] = p.temperature
            values[1, row] = p.top_p
            values[2, row] = 0.0 if p.greedy or random is None else random.next_uniform()
        tokens = ops.sample(logits, options[0], options[1], options[2], host_copy=host_copy)
        return SampledTokens(tokens, host_copy, check_errors, keep=(options,))

    def __call__(self, logits: torch.Tensor, params: Sequence[SamplingParams], randoms: Sequence[Optional[RequestRandom]]) -> list[int]:
        """The same, waited for: one token id per row."""
        return self.launch(logits, params, randoms).result()
