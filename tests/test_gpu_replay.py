"""bin/trace_run as a user runs it: a subprocess, JSON steps on standard input, .f32 files out.
The same requests are replayed whole, with the last 32 tokens one by one, and in batches of unequal
lengths (one batch after another, so slots are reused), in 32-bit and in bfloat16, and compared with
the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tests.conftest import ROOT, TINY, TOL, random_tokens, rel_err

pytestmark = pytest.mark.gpu
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def replay(model_dir, dtype, steps, out_dir, max_tokens):
    proc = subprocess.run([sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", str(out_dir),
                           "--max-tokens", str(max_tokens)],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps], proc.stdout[-500:]
    return proc


def read(out_dir, step, vocab):
    return np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, vocab)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("B", "bfloat16"),
                                        ("B32", "float32"), ("D", "bfloat16")])
def test_three_ways_of_cutting(model_dirs, plains, tmp_path, name, dtype):
    cfg, plain = TINY[name], plains(name, dtype)
    V, P = cfg["vocab_size"], cfg["n_positions"]
    reqs = {f"r{i}": random_tokens(900 + i, n, V) for i, n in enumerate([40, 97, 33, min(P, 150)])}
    refs = {k: plain.logits(t) for k, t in reqs.items()}
    steps, expect = [], {}
    n = 0

    def add(entries, end=()):
        nonlocal n
        steps.append({"step": n, "entries": entries, "end": list(end)})
        n += 1
        return n - 1

    # 1. each request alone and whole
    for k, t in reqs.items():
        s = add([{"id": k + "w", "tokens": t, "want": list(range(len(t)))}], end=[k + "w"])
        expect[s] = refs[k]
    # 2. the last 32 tokens one by one
    for k, t in reqs.items():
        head = len(t) - 32
        s = add([{"id": k + "d", "tokens": t[:head], "want": [head - 1]}])
        expect[s] = refs[k][head - 1:head]
        for j in range(head, len(t)):
            s = add([{"id": k + "d", "tokens": [t[j]], "want": [0]}], end=[k + "d"] if j == len(t) - 1 else [])
            expect[s] = refs[k][j:j + 1]
    # 3. batches of unequal lengths; shorter requests end earlier; twice, so that slots are reused
    for rnd in range(2):
        ids = list(reqs)
        prompt = {k: max(1, len(reqs[k]) - 6 - 3 * i) for i, k in enumerate(ids)}
        s = add([{"id": f"{k}b{rnd}", "tokens": reqs[k][:prompt[k]], "want": [prompt[k] - 1]} for k in ids])
        expect[s] = np.stack([refs[k][prompt[k] - 1] for k in ids])
        j = 0
        live = list(ids)
        while live:
            ending = [k for k in live if prompt[k] + j == len(reqs[k]) - 1]
            s = add([{"id": f"{k}b{rnd}", "tokens": [reqs[k][prompt[k] + j]], "want": [0]} for k in live],
                    end=[f"{k}b{rnd}" for k in ending])
            expect[s] = np.stack([refs[k][prompt[k] + j] for k in live])
            live = [k for k in live if k not in ending]
            j += 1

    # the cache holds exactly what the largest moment needs: all four, rounded up to pages of 64
    need = sum(-(-len(t) // 64) * 64 for t in reqs.values())
    out = tmp_path / "out"
    replay(model_dirs[name], dtype, steps, out, need)
    for s, ref in expect.items():
        got = read(out, s, V)
        assert got.shape == ref.shape, (s, got.shape, ref.shape)
        assert rel_err(got, ref) < TOL[dtype], f"step {s}: {steps[s]['entries'][0]['id']}"
    assert sorted(int(f[:-4]) for f in os.listdir(out)) == sorted(expect)


def test_steps_without_wants_write_nothing_and_bad_input_fails(model_dirs, tmp_path):
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [4], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "o"
    replay(model_dirs["A"], "float32", steps, out, 64)
    assert os.listdir(out) == ["1.f32"]
    proc = subprocess.run([sys.executable, TRACE_RUN, "--model", model_dirs["A"], "--dtype", "float32", "--out",
                           str(tmp_path / "p"), "--max-tokens", "64"],
                          input=json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [99999], "want": [0]}]}) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and "outside the vocabulary" in proc.stderr
