"""Sampling options, the per-request random stream, and the rule in plain Python.

The rule is bisand/kvad's (crates/llm/src/sampler.rs:55-131): temperature <= 0
is greedy (first index of the largest logit, :217-227); otherwise rank the
candidates best first with ties by lower id (:204-210), keep the first
`top_k` (0 = all), softmax of logit/temperature over what is kept, keep the
shortest prefix whose mass reaches `top_p` (if 0 < top_p < 1), draw
`target = uniform * kept mass` and walk down until it is used up (:63-71).
The stream is xorshift64* with a 24-bit uniform (crates/nervus/src/rng.rs:12-31);
every request owns one, so what one request draws does not depend on what
else is in its batch (crates/llm/src/sampler.rs:42-53).  Defaults are
`kvad run`'s (crates/llm/src/main.rs:249-252).

On the GPU the same rule runs as a kernel (`Ops.sample`); this module feeds it
one uniform number per sampling row and serves as its host-side statement.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

_MASK = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.95
    seed: int = 7

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @staticmethod
    def make_greedy() -> "SamplingParams":
        return SamplingParams(temperature=0.0, top_k=0, top_p=1.0)


class Xorshift64Star:
    def __init__(self, seed: int):
        seed &= _MASK
        self.state = seed if seed != 0 else 0x9E3779B97F4A7C15

    def next_u64(self) -> int:
        x = self.state
        x ^= x >> 12
        x ^= (x << 25) & _MASK
        x ^= x >> 27
        self.state = x
        return (x * 0x2545F4914F6CDD1D) & _MASK

    def uniform(self) -> float:
        """Uniform in [0, 1) from the top 24 bits."""
        return (self.next_u64() >> 40) / float(1 << 24)


def argmax(logits: Sequence[float]) -> int:
    best, top = 0, None
    for i, x in enumerate(logits):
        if top is None:
            best, top = i, x
            if x != x:
                top = -math.inf
        elif x > top:
            best, top = i, x
    return best


def shortlist(logits: Sequence[float], temperature: float, top_k: int, top_p: float):
    """Candidates in rank order and the probabilities the draw uses."""
    import numpy as np

    l = np.asarray(logits, dtype=np.float32)
    order = np.lexsort((np.arange(l.size), -l.astype(np.float64)))        # logit descending, then id ascending
    k = l.size if top_k <= 0 else min(top_k, l.size)
    order = order[:k]
    z = l[order] / np.float32(temperature)
    z = np.exp(z - z.max())
    probs = (z / z.sum(dtype=np.float32)).astype(np.float32)
    if 0.0 < top_p < 1.0:
        cum = np.cumsum(probs, dtype=np.float32)
        keep = int(np.searchsorted(cum, np.float32(top_p), side="left")) + 1
        keep = min(keep, probs.size)
        order, probs = order[:keep], probs[:keep]
    return order, probs


def sample_host(logits: Sequence[float], params: SamplingParams, uniform: float) -> int:
    """The rule on the host, for one row and one uniform number."""
    if params.greedy:
        return argmax(logits)
    import numpy as np

    order, probs = shortlist(logits, params.temperature, params.top_k, params.top_p)
    target = np.float32(uniform) * probs.sum(dtype=np.float32)
    for i, p in enumerate(probs):
        target -= p
        if target <= 0:
            return int(order[i])
    return int(order[-1])


class RequestSampler:
    """One request's options and stream."""

    def __init__(self, params: SamplingParams, seed: Optional[int] = None):
        self.params = params
        self.rng = Xorshift64Star(params.seed if seed is None else seed)

    def next_uniform(self) -> float:
        return 0.0 if self.params.greedy else self.rng.uniform()

    def sample(self, logits: Sequence[float]) -> int:
        return sample_host(logits, self.params, self.next_uniform())
