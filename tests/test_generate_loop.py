"""The generation loop's decisions, with a scripted backend (no GPU)."""
import pytest

from kvad_b200.engine.generate import Request, Stats, run_all, run_batch
from kvad_b200.sampling import SamplingParams


class Scripted:
    """A backend whose 'model' continues a sequence with (last token + 1) % 50 and logs every call."""

    def __init__(self, context=32, n_slots=3):
        self.context, self.free, self.open_slots = context, list(range(n_slots)), set()
        self.calls, self.held = [], {}

    def open(self):
        s = self.free.pop(0)
        self.open_slots.add(s)
        self.held[s] = 0
        return s

    def close(self, slot):
        assert slot in self.open_slots, "closed twice"
        self.open_slots.remove(slot)
        self.free.append(slot)
        del self.held[slot]

    def room(self, prompt_len):
        return self.context - prompt_len

    def step_and_sample(self, entries, samplers):
        assert len(entries) == len(samplers)
        self.calls.append([(s, list(t)) for s, t in entries])
        out = []
        for (slot, toks), smp in zip(entries, samplers):
            assert slot in self.open_slots
            self.held[slot] += len(toks)
            assert self.held[slot] <= self.context
            smp.next_uniform()
            out.append((toks[-1] + 1) % 50)
        return out


def greedy(prompt, n, stop=()):
    return Request(list(prompt), n, SamplingParams.make_greedy(), frozenset(stop))


def test_prompts_in_one_step_then_one_token_each():
    b = Scripted()
    reqs = [greedy([1, 2, 3], 3), greedy([10], 3)]
    run_batch(b, reqs)
    assert [len(c) for c in b.calls] == [2, 2, 2]
    assert b.calls[0] == [(0, [1, 2, 3]), (1, [10])]
    assert b.calls[1] == [(0, [4]), (1, [11])]                  # the chosen token is fed in the next step
    assert reqs[0].generated == [4, 5, 6] and reqs[1].generated == [11, 12, 13]
    assert all(r.finish_reason == "length" for r in reqs) and not b.open_slots


def test_stop_token_ends_the_request_and_is_not_kept():
    b = Scripted()
    reqs = [greedy([1], 10, stop=[4]), greedy([20], 5)]
    run_batch(b, reqs)
    assert reqs[0].generated == [2, 3] and reqs[0].finish_reason == "stop"
    assert reqs[1].generated == [21, 22, 23, 24, 25]
    # the stopped request left the batch at once: later steps bring one row, and 4 was never fed
    assert [len(c) for c in b.calls] == [2, 2, 2, 1, 1]
    assert all(t != [4] for c in b.calls for _, t in c)


def test_budget_is_clipped_to_the_context():
    b = Scripted(context=8)
    reqs = [greedy([1, 2, 3, 4, 5], 100), greedy(list(range(8)), 5), greedy([1], 0)]
    run_batch(b, reqs)
    assert len(reqs[0].generated) == 3 and reqs[0].finish_reason == "context"
    assert reqs[1].generated == [] and reqs[1].finish_reason == "context"       # no room at all: never stepped
    assert reqs[2].generated == [] and reqs[2].finish_reason == "length"
    assert all(len(t) <= 5 for c in b.calls for _, t in c)
    with pytest.raises(ValueError, match="does not fit"):
        run_batch(b, [greedy(list(range(9)), 1)])
    with pytest.raises(ValueError, match="empty prompt"):
        run_batch(b, [greedy([], 1)])


def test_batches_run_one_after_another_and_reuse_slots():
    b = Scripted(n_slots=2)
    reqs = [greedy([i], 1 + i % 3) for i in range(5)]
    stats = run_all(b, reqs, batch_size=2)
    assert stats.batches == 3 and stats.generated_tokens == sum(1 + i % 3 for i in range(5))
    assert [r.generated for r in reqs] == [[(i + 1 + k) % 50 for k in range(1 + i % 3)] for i in range(5)]
    used = {s for c in b.calls for s, _ in c}
    assert used == {0, 1} and not b.open_slots                        # five requests went through two slots
    # no request joins a running batch: the first step of a batch brings only prompts
    firsts = [c for c in b.calls if any(len(t) == 1 and t[0] < 5 for _, t in c)]
    assert len(firsts) >= 3


def test_slots_come_back_when_the_backend_fails():
    class Failing(Scripted):
        def step_and_sample(self, entries, samplers):
            if len(self.calls) == 1:
                raise RuntimeError("boom")
            return super().step_and_sample(entries, samplers)

    b = Failing()
    with pytest.raises(RuntimeError):
        run_batch(b, [greedy([1], 5), greedy([2], 5)])
    assert not b.open_slots and sorted(b.free) == [0, 1, 2]


def test_every_request_draws_from_its_own_stream():
    seen = {}

    class Recording(Scripted):
        def step_and_sample(self, entries, samplers):
            for (slot, toks), s in zip(entries, samplers):
                seen.setdefault(id(s), []).append(s.rng.state)
            return super().step_and_sample(entries, samplers)

    def draws(batch):
        seen.clear()
        b = Recording(n_slots=4)
        run_batch(b, batch)
        return list(seen.values())

    p = SamplingParams(0.8, 40, 0.95, seed=5)
    alone = draws([Request([1], 4, p)])
    together = draws([Request([1], 4, p), Request([7, 8], 2, SamplingParams(0.8, 40, 0.95, seed=9))])
    assert together[0] == alone[0]                      # what one request draws does not depend on its batch
    assert together[1] != together[0][:len(together[1])]


def test_stats_and_on_token():
    b = Scripted()
    seen = []
    stats = Stats()
    run_batch(b, [greedy([1, 2], 2), greedy([5], 3)], stats, on_token=lambda i, t: seen.append((i, t)))
    assert stats.prompt_tokens == 3 and stats.generated_tokens == 5 and stats.steps == 3
    assert seen == [(0, 3), (1, 6), (0, 4), (1, 7), (1, 8)]


class ScriptedAhead(Scripted):
    """The same fake model with `launch_step`: steps are launched ahead and their tokens read later."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.last = {}             # slot -> the token its latest step chose (what a device-fed step continues from)
        self.launched_ahead = 0

    def step_and_sample(self, entries, samplers):
        out = super().step_and_sample(entries, samplers)
        for (slot, _), tok in zip(entries, out):
            self.last[slot] = tok
        return out

    def launch_step(self, entries, samplers, device_fed):
        if device_fed:
            self.launched_ahead += 1
            assert all(t is None for _, t in entries)
            entries = [(slot, [self.last[slot]]) for slot, _ in entries]
        else:
            assert all(t == [self.last[slot]] for slot, t in entries), "host-fed tokens must be the ones chosen"
        live = [s for s, _ in entries if s in self.open_slots]
        out = []
        self.calls.append([(s, list(t)) for s, t in entries])
        for (slot, toks), smp in zip(entries, samplers):
            self.held[slot] = self.held.get(slot, 0) + 1 if slot in self.held else 1
            smp.next_uniform()
            tok = (toks[-1] + 1) % 50
            self.last[slot] = tok
            out.append(tok)

        class Handle:
            def tokens(_self):
                return out
        return Handle()


@pytest.mark.parametrize("case", [
    [([1, 2, 3], 3, ()), ([10], 3, ())],
    [([1], 10, (4,)), ([20], 5, ())],
    [([1], 10, (3,)), ([20], 9, (24,)), ([30, 31], 6, ())],
    [([5], 1, ()), ([6], 2, ()), ([7], 7, (9,))],
])
def test_running_a_step_ahead_changes_no_decision(case):
    def run(backend):
        reqs = [greedy(p, n, stop) for p, n, stop in case]
        stats = Stats()
        run_batch(backend, reqs, stats)
        assert not backend.open_slots
        return [(r.generated, r.finish_reason) for r in reqs], stats.generated_tokens

    plain, ahead = Scripted(context=64), ScriptedAhead(context=64)
    assert run(plain) == run(ahead)
    if case[0][0] != [5]:              # (in the last case a request can end by its budget in every step)
        assert ahead.launched_ahead > 0
