"""The generation loop: batches of unequal prompts, stop tokens, sequences
that end earlier, one batch after another.

The loop decides; a *backend* computes.  The backend is anything with

    open() -> slot                       a fresh sequence
    close(slot)                          give everything it holds back
    room(prompt_len) -> int              how many tokens still fit after the prompt
    step_and_sample(entries, samplers) -> list[int]
        entries: [(slot, tokens)] - the prompts in the first step of a batch,
        then one token per live sequence; returns one chosen token per entry.

so the decisions are tested with a scripted backend and no GPU.  They follow
bisand/kvad's runtime (crates/llm/src/runtime.rs): the budget is
min(max_tokens, context - prompt length) (:627); a chosen token is fed only in
the next step, if the request goes on (:759-773); a stop token ends the
request and is neither kept nor fed (:787-790); a request that ends leaves the
batch at once and the others go on (:731-754); every request draws from its
own stream (crates/llm/src/sampler.rs:42-53).  A batch starts together: no
request joins a running batch; the next batch starts when the last sequence of
this one has ended, reusing the slots that came back.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Optional, Protocol, Sequence

from ..sampling.sampler import RequestSampler, SamplingParams


@dataclass
class Request:
    prompt: Sequence[int]
    max_tokens: int = 256
    params: SamplingParams = field(default_factory=SamplingParams)
    stop_token_ids: frozenset = frozenset()
    seed: Optional[int] = None
    # filled by the loop
    generated: list = field(default_factory=list)
    finish_reason: Optional[str] = None        # "stop", "length", "context"


@dataclass
class Stats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_secs: float = 0.0
    decode_secs: float = 0.0
    batches: int = 0
    steps: int = 0

    def tokens_per_sec(self) -> float:
        return self.generated_tokens / self.decode_secs if self.decode_secs > 0 else 0.0


class Backend(Protocol):
    def open(self) -> int: ...
    def close(self, slot: int) -> None: ...
    def room(self, prompt_len: int) -> int: ...
    def step_and_sample(self, entries, samplers) -> list: ...


def _apply(requests, live, chosen, backend, opened, stats, on_token, only=None):
    """The loop's decisions for one step's chosen tokens; returns the items that go on.
    `only`: if given, items outside it are skipped (they ended a step earlier)."""
    still = []
    for it, tok in zip(live, chosen):
        if only is not None and not any(it is o for o in only):
            continue
        r = requests[it[0]]
        tok = int(tok)
        if tok in r.stop_token_ids:
            r.finish_reason = "stop"          # not kept, not fed
        else:
            r.generated.append(tok)
            stats.generated_tokens += 1
            if on_token is not None:
                on_token(it[0], tok)
            it[3] -= 1
            if it[3] == 0:
                r.finish_reason = "length" if len(r.generated) >= r.max_tokens else "context"
        if r.finish_reason is None:
            it[4] = [tok]                      # fed in the next step
            still.append(it)
        else:
            backend.close(it[1])               # leaves the batch at once
            opened.remove(it[1])
    return still


def run_batch(backend: Backend, requests: Sequence[Request], stats: Optional[Stats] = None,
              on_token: Optional[Callable[[int, int], None]] = None,
              clock: Callable[[], float] = time.perf_counter) -> None:
    """Runs one batch to its end.  Fills `generated` and `finish_reason` of every request.

    A backend that also offers `launch_step(entries, samplers, device_fed) -> handle` (with
    `handle.tokens()`) is driven one step ahead: while the host waits for a step's tokens and
    decides, the next step - fed on the device with those very tokens - is already running.  It is
    launched only when no request can end by its budget in the step before; if a request ends by a
    stop token, the step that ran ahead is still right for the others (sequences do not see one
    another) and is merely wasted for the one that ended.  The decisions and the tokens are the same
    either way."""
    stats = stats if stats is not None else Stats()
    live = []                     # [index, slot, sampler, left, pending tokens]
    for i, r in enumerate(requests):
        if len(r.prompt) == 0:
            raise ValueError("an empty prompt cannot be continued")
        left = min(int(r.max_tokens), backend.room(len(r.prompt)))
        if left < 0:
            raise ValueError(f"a prompt of {len(r.prompt)} tokens does not fit the context")
        if left == 0:
            r.finish_reason = "context" if r.max_tokens > 0 else "length"
            continue
        live.append([i, None, RequestSampler(r.params, r.seed), left, list(r.prompt)])
    opened = []
    pipelined = hasattr(backend, "launch_step")
    try:
        for item in live:
            item[1] = backend.open()
            opened.append(item[1])
        stats.batches += 1
        if not live:
            return
        # the prompts, in one step
        t0 = clock()
        chosen = backend.step_and_sample([(it[1], it[4]) for it in live], [it[2] for it in live])
        stats.prefill_secs += clock() - t0
        stats.steps += 1
        stats.prompt_tokens += sum(len(it[4]) for it in live)
        live = _apply(requests, live, chosen, backend, opened, stats, on_token)
        # then one token each
        t0 = clock()
        try:
            if not pipelined:
                while live:
                    chosen = backend.step_and_sample([(it[1], it[4]) for it in live], [it[2] for it in live])
                    stats.steps += 1
                    live = _apply(requests, live, chosen, backend, opened, stats, on_token)
            else:
                in_flight = None
                while live:
                    samplers = [it[2] for it in live]
                    if in_flight is None:
                        in_flight = backend.launch_step([(it[1], it[4]) for it in live], samplers, False)
                    ahead = None
                    if all(it[3] >= 2 for it in live):           # nobody can end by budget in the step in flight
                        ahead = backend.launch_step([(it[1], None) for it in live], samplers, True)
                    chosen = in_flight.tokens()
                    stats.steps += 1
                    still = _apply(requests, live, chosen, backend, opened, stats, on_token)
                    if len(still) == len(live):
                        in_flight = ahead
                    else:
                        if ahead is not None:                     # ran with the old company: right for those who go on
                            chosen = ahead.tokens()
                            stats.steps += 1
                            still = _apply(requests, live, chosen, backend, opened, stats, on_token, only=still)
                        in_flight = None
                    live = still
        finally:
            stats.decode_secs += clock() - t0
    finally:
        for slot in opened:
            backend.close(slot)


def run_all(backend: Backend, requests: Sequence[Request], batch_size: int, stats: Optional[Stats] = None,
            on_token: Optional[Callable[[int, int], None]] = None) -> Stats:
    """As many batches, one after another, as the requests need."""
    if batch_size <= 0:
        raise ValueError("batch_size must be positive")
    stats = stats if stats is not None else Stats()
    for start in range(0, len(requests), batch_size):
        chunk = requests[start:start + batch_size]
        cb = (lambda i, t, s=start: on_token(s + i, t)) if on_token is not None else None
        run_batch(backend, chunk, stats, cb)
    return stats
