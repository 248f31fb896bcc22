"""The sampler: float32 logits on the device in, one token id per row out.

The work is done by the kernels in csrc/sampling.cu.  Every request draws
from a stream of its own, keyed by (seed, request index, tokens drawn so
far), so what a request samples does not depend on who shares its batch.
"""
from __future__ import annotations

import torch

from .. import kernels
from .params import SamplingParams

MASK64 = (1 << 64) - 1


def _splitmix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    return z ^ (z >> 31)


def uniform24(seed: int, stream: int, counter: int) -> float:
    """The uniform number in [0, 1) the sampling kernel uses for (seed, stream, counter)."""
    x = _splitmix64(_splitmix64(_splitmix64(seed & MASK64) ^ (stream & 0xFFFFFFFF)) ^ (counter & MASK64))
    return (x >> 40) / 16777216.0


class Sampler:
    def __init__(self, params: SamplingParams):
        self.params = params
        self._out: dict = {}

    def __call__(self, logits: torch.Tensor, streams: torch.Tensor, counter: int) -> torch.Tensor:
        """logits [rows, vocab] float32; streams int32 [rows]; returns int32 [rows] on the device
        (a buffer of the sampler's, written again by its next call with as many rows)."""
        key = (logits.shape[0], logits.device)
        out = self._out.get(key)                 # valid until the next call with as many rows
        if out is None:
            out = self._out[key] = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
        p = self.params
        if p.greedy:
            kernels.argmax(logits, out)
        else:
            kernels.sample(logits, float(p.temperature), int(p.top_k), float(p.top_p), int(p.seed), streams,
                           int(counter), out)
        return out
