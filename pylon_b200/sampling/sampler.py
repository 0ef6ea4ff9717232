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


class Sampler:
    def __init__(self, device: torch.device) -> None:
        self.device = torch.device(device)

    def __call__(self, logits: torch.Tensor, params: Sequence[SamplingParams], randoms: Sequence[Optional[RequestRandom]]) -> list[int]:
        """``logits``: float32 ``[rows, vocab]`` on the device; returns one token id per row."""
        rows = logits.shape[0]
        if rows != len(params) or rows != len(randoms):
            raise ValueError("one set of sampling options and one random stream per row of logits")
        if all(p.greedy for p in params):
            return ops.sample(logits).cpu().tolist()
        host = torch.empty((3, rows), dtype=torch.float32, pin_memory=True)
        values = host.numpy()
        for row, (p, random) in enumerate(zip(params, randoms)):
            values[0, row] = p.temperature
            values[1, row] = p.top_p
            values[2, row] = 0.0 if p.greedy or random is None else random.next_uniform()
        device_values = host.to(self.device, non_blocking=True)
        return ops.sample(logits, device_values[0], device_values[1], device_values[2]).cpu().tolist()
