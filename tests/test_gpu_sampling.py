"""The sampling kernel against the rule stated on the host, and the command line end to end."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from kvad_b200.ops import Ops, sample_force_general
from kvad_b200.sampling import SamplingParams, sample_host, shortlist
from tests.conftest import ROOT, random_tokens

pytestmark = pytest.mark.gpu


def run_kernel(logits, params, uniforms):
    ops = Ops(torch.float32)
    n = logits.shape[0]
    dev = lambda a, dt: torch.tensor(a, dtype=dt).cuda()
    out = torch.full((n,), -1, dtype=torch.int32, device="cuda")
    ops.sample(torch.tensor(logits).cuda(), dev([p.temperature for p in params], torch.float32),
               dev([p.top_k for p in params], torch.int32), dev([p.top_p for p in params], torch.float32),
               dev(uniforms, torch.float32), out)
    return out.cpu().tolist()


def on_a_boundary(logits, p, u, tok):
    """Whether `tok` is what the rule gives when its two thresholds move by no more than rounding.

    The host states the rule with 32-bit running sums, as bisand/kvad does; the kernel sums exactly in
    fixed point.  Over tens of thousands of candidates the two can place the top-p cut a few (equally
    unlikely) candidates apart, and a draw at the very end of the kept mass then lands on another of
    them.  So: rank and sum in float64, let top_p and the draw each move by 1e-5 of the mass, and ask
    whether the token's slice of the ranking can be hit."""
    l = np.asarray(logits, dtype=np.float64)
    order = np.lexsort((np.arange(l.size), -l))
    k = l.size if p.top_k <= 0 else min(p.top_k, l.size)
    order = order[:k]
    z = np.exp((l[order] - l[order[0]]) / p.temperature)
    cum = np.cumsum(z)
    total = cum[-1]
    eps = 1e-5 * total
    if 0.0 < p.top_p < 1.0:
        keep_lo = int(np.searchsorted(cum, p.top_p * total - eps, side="left")) + 1
        keep_hi = int(np.searchsorted(cum, p.top_p * total + eps, side="left")) + 1
    else:
        keep_lo = keep_hi = k
    keep_lo, keep_hi = min(keep_lo, k), min(keep_hi, k)
    where = np.nonzero(order == tok)[0]
    if where.size == 0 or where[0] >= keep_hi:
        return False
    r = int(where[0])
    below = cum[r - 1] if r > 0 else 0.0
    lo_target, hi_target = u * cum[keep_lo - 1] - eps, u * cum[keep_hi - 1] + eps
    if r == keep_hi - 1 or r == keep_lo - 1:            # the last kept candidate takes whatever is left
        return hi_target >= below - eps
    return lo_target <= cum[r] + eps and hi_target >= below - eps


@pytest.mark.parametrize("vocab", [1000, 50257])
def test_kernel_follows_the_rule(vocab):
    rng = np.random.default_rng(vocab)
    combos = [SamplingParams(0.7, 40, 0.95), SamplingParams(1.0, 0, 1.0), SamplingParams(1.3, 0, 0.9),
              SamplingParams(0.5, 5, 0.5), SamplingParams(0.0, 40, 0.95), SamplingParams(1.0, 1, 1.0),
              SamplingParams(2.0, 500, 0.999), SamplingParams(0.9, vocab + 5, 0.3)]
    rows, params, us = [], [], []
    for i in range(48):
        l = rng.standard_normal(vocab).astype(np.float32) * (1 + i % 4)
        if i % 5 == 0:
            l = np.round(l * 4) / 4                      # many exact ties: ranked by lower id
        rows.append(l)
        params.append(combos[i % len(combos)])
        us.append([0.0, 0.37, 0.999999, 0.5][i % 4] if i < 16 else float(rng.random()))
    logits = np.stack(rows)
    got = run_kernel(logits, params, us)
    again = run_kernel(logits, params, us)
    assert got == again                                  # the same logits, options and draw: the same token
    sample_force_general(True)                           # and the same whichever way the kernel takes
    try:
        assert run_kernel(logits, params, us) == got
    finally:
        sample_force_general(False)
    exact = 0
    for i, tok in enumerate(got):
        want = sample_host(logits[i], params[i], us[i])
        if tok == want:
            exact += 1
        else:
            assert on_a_boundary(logits[i], params[i], us[i], tok), (i, tok, want, params[i], us[i])
    assert exact >= 44


@pytest.mark.parametrize("vocab", [300, 5000, 70001])
def test_small_top_k_both_ways(vocab):
    """Every top-k up to the short way's limit and beyond, on rows with and without ties, NaNs and -inf:
    the short way and the selections over the whole vocabulary give the same tokens."""
    rng = np.random.default_rng(7 * vocab)
    rows, params, us = [], [], []
    for i, k in enumerate([1, 2, 7, 40, 64, 65, 250, 511, 512, 900, 1024, 1025, 3000]):
        l = rng.standard_normal(vocab).astype(np.float32) * (1 + i % 3)
        if i % 3 == 1:
            l = np.round(l * 2) / 2
        if i % 4 == 2:
            l[rng.integers(0, vocab, 20)] = np.nan
            l[rng.integers(0, vocab, 20)] = -np.inf
        rows.append(l)
        params.append(SamplingParams([0.7, 1.0, 1.6][i % 3], k, [0.95, 1.0, 0.6][(i // 2) % 3]))
        us.append(float(rng.random()))
    logits = np.stack(rows)
    got = run_kernel(logits, params, us)
    sample_force_general(True)
    try:
        assert run_kernel(logits, params, us) == got
    finally:
        sample_force_general(False)
    for i, tok in enumerate(got):
        clean = np.where(np.isnan(logits[i]), -np.inf, logits[i])
        want = sample_host(clean, params[i], us[i])
        assert tok == want or on_a_boundary(clean, params[i], us[i], tok), (i, tok, want, params[i])


def test_topk_one_and_greedy_agree_with_argmax():
    rng = np.random.default_rng(1)
    logits = rng.standard_normal((6, 777)).astype(np.float32)
    logits[2, 5] = logits[2, 700] = 9.0
    got = run_kernel(logits, [SamplingParams(1.0, 1, 1.0)] * 3 + [SamplingParams(0.0, 0, 1.0)] * 3, [0.9] * 6)
    assert got == [int(np.argmax(r)) for r in logits]


def test_command_line_runs_and_matches_the_entry_point(model_dirs, engines):
    prompt = random_tokens(77, 6, 512)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kvad"), "run", "--model", model_dirs["A"], "--tokens",
                           ",".join(map(str, prompt)), "--max-tokens", "7", "--greedy", "--dtype", "f32"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-1500:]
    ids = [int(x) for x in proc.stdout.strip().split(",")]
    assert ids == engines("A", "float32").generate([prompt], max_tokens=7, temperature=0.0)[0]
    assert "[prefill 6 tokens in" in proc.stderr and "tok/s]" in proc.stderr
    # sampled: the same seed gives the same tokens, another seed others
    e = engines("A", "float32")
    a = e.generate([prompt], max_tokens=12, temperature=0.8, top_k=40, top_p=0.95, seed=3)
    assert a == e.generate([prompt], max_tokens=12, temperature=0.8, top_k=40, top_p=0.95, seed=3)
    assert a != e.generate([prompt], max_tokens=12, temperature=0.8, top_k=40, top_p=0.95, seed=4)
    # a request's tokens do not depend on its company in the batch
    both = e.generate([prompt, random_tokens(78, 9, 512)], max_tokens=12, temperature=0.8, top_k=40, top_p=0.95, seed=3)
    assert both[0] == a[0]


def test_command_line_takes_a_text_prompt_through_tokenizer_json(model_dirs, engines, tmp_path):
    """`kvad run --prompt TEXT`: the folder's tokenizer.json turns the text into ids and the ids back into
    text; a base model's output starts with its prompt (crates/kvad/src/main.rs:1583-1599)."""
    tokenizers = pytest.importorskip("tokenizers")
    import shutil
    d = str(tmp_path / "with_tokenizer")
    shutil.copytree(model_dirs["A"], d)
    vocab = {f"w{i}": i for i in range(512)}
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="w0"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.Whitespace()
    tok.save(os.path.join(d, "tokenizer.json"))
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kvad"), "run", "--model", d, "--prompt", "w5 w17 w3 w250",
                           "--max-tokens", "6", "--greedy", "--dtype", "f32"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-1500:]
    want = engines("A", "float32").generate([[5, 17, 3, 250]], max_tokens=6, temperature=0.0)[0]
    assert proc.stdout.split() == ["w5", "w17", "w3", "w250"] + [f"w{t}" for t in want]
    # without a tokenizer a text prompt is refused with a hint, not guessed at
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kvad"), "run", "--model", model_dirs["A"], "--prompt", "w5",
                           "--max-tokens", "2"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 2 and "--tokens" in proc.stderr


class _BusyBackend:
    """The engine as the generation loop's backend, with the stream kept busy before every launch so that
    queued host-to-device copies lag far behind the host."""

    def __init__(self, engine, pipelined):
        self.e = engine
        self.ballast = torch.empty(1 << 30, dtype=torch.uint8, device=engine.device)
        self.open, self.close, self.room = engine.open, engine.close, engine.room
        if pipelined:
            self.launch_step = self._launch_step

    def _busy(self):
        for _ in range(3):
            self.ballast.zero_()

    def step_and_sample(self, entries, samplers):
        self._busy()
        return self.e.step_and_sample(entries, samplers)

    def _launch_step(self, entries, samplers, device_fed=False):
        self._busy()
        return self.e.launch_step(entries, samplers, device_fed)


def test_sampled_generation_a_step_ahead_draws_the_same_tokens(engines):
    """The loop launches a step ahead of the one it waits for; each step's sampling options and uniform
    numbers go up through a ring of staging buffers.  With the device lagging the host by several steps'
    worth of work, the tokens are those of the loop that waits for every step."""
    from kvad_b200.engine.generate import Request, run_all
    from kvad_b200.sampling import SamplingParams
    e = engines("A", "float32")
    prompts = [random_tokens(90 + i, n, 512) for i, n in enumerate([6, 3, 11, 8])]

    def run(pipelined):
        reqs = [Request(list(p), 40, SamplingParams(0.9, 50, 0.95, 100 + i), frozenset()) for i, p in enumerate(prompts)]
        run_all(_BusyBackend(e, pipelined), reqs, 4)
        return [r.generated for r in reqs]

    ahead, plain_loop = run(True), run(False)
    assert ahead == plain_loop and all(len(o) == 40 for o in ahead)
    e.cache.book.check_all_free()
