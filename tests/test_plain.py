"""The plain implementation against the constants and identities bisand/kvad's own unit tests pin
(crates/llm/src/tensor.rs:487-581), and against itself (no GPU)."""
import math

import numpy as np
import pytest

from tests.conftest import TINY, random_tokens
from tests.plain.gpt2_plain import PlainGpt2, round_bf16


def test_gelu_points():
    g = PlainGpt2.gelu_tanh(np.array([0.0, 3.0, -3.0, 1.0]))
    assert g[0] == 0 and g[1] == pytest.approx(2.9959, abs=1e-3) and -0.01 < g[2] < 0       # crates/llm/src/tensor.rs:575-581
    # erf table values of crates/llm/src/tensor.rs:569: erf(1) = 0.8427007929, erf(0.5) = 0.5204998778
    r2 = math.sqrt(2.0)
    e = PlainGpt2.gelu_erf(np.array([r2, 0.5 * r2]))
    assert e[0] == pytest.approx(0.5 * r2 * (1 + 0.8427007929), abs=1e-9)
    assert e[1] == pytest.approx(0.25 * r2 * (1 + 0.5204998778), abs=1e-9)
    # the two forms differ by a few 1e-4: a model run with the wrong one fails the engine tests
    x = np.linspace(-3, 3, 601)
    assert 1e-4 < np.abs(PlainGpt2.gelu_tanh(x) - PlainGpt2.gelu_erf(x)).max() < 1e-3
    assert math.sqrt(2 / math.pi) == pytest.approx(0.79788456, abs=1e-8)


def test_layer_norm_and_softmax_identities(plains):
    m = plains("A")
    y = m.layer_norm(np.array([[1.0, 2.0, 3.0, 4.0]]), np.ones(4), np.zeros(4))
    assert y.mean() == pytest.approx(0, abs=1e-12) and y.var() == pytest.approx(1, abs=1e-4)
    y = m.layer_norm(np.array([[1.0, 2.0, 3.0, 4.0]]), np.full(4, 2.0), np.full(4, 0.5))
    assert y.mean() == pytest.approx(0.5, abs=1e-12)


def test_round_bf16_is_nearest_even():
    assert round_bf16(np.array([1.0]))[0] == 1.0
    assert round_bf16(np.array([1.0 + 2**-8]))[0] == 1.0                # halfway: to even
    assert round_bf16(np.array([1.0 + 3 * 2**-8]))[0] == 1.0 + 2**-6   # halfway: to even, upwards
    assert round_bf16(np.array([1.0 + 2**-8 + 2**-12]))[0] == 1.0 + 2**-7


def test_causal_and_deterministic(plains):
    m = plains("B")
    t = random_tokens(1, 20, 1000)
    a = m.logits(t)
    t2 = list(t)
    t2[15] = (t2[15] + 1) % 1000
    b = m.logits(t2)
    assert np.array_equal(a[:15], b[:15]) and not np.allclose(a[15:], b[15:])
    assert np.allclose(m.logits(t[:7]), a[:7], atol=1e-12)


def test_options_matter(model_dirs, tmp_path):
    """Every option of the configuration changes the logits, so a kernel that ignores one cannot pass."""
    import json, os, shutil
    base = PlainGpt2(model_dirs["B"])
    t = random_tokens(2, 12, 1000)
    ref = base.logits(t)
    for key, val in [("activation_function", "gelu_new"), ("scale_attn_by_inverse_layer_idx", False),
                     ("layer_norm_epsilon", 1e-2)]:
        d = tmp_path / key
        shutil.copytree(model_dirs["B"], d)
        cfg = json.load(open(d / "config.json"))
        cfg[key] = val
        json.dump(cfg, open(d / "config.json", "w"))
        other = PlainGpt2(str(d)).logits(t)
        assert np.abs(other - ref).max() / np.abs(ref).max() > 2e-5, key


def test_grouped_heads_read_the_right_kv_head(plains):
    m = plains("C")
    assert m.H == 6 and m.Hkv == 2 and m.hd == 16 and not m.tied
    q = np.zeros((1, 96)); k = np.zeros((1, 32)); v = np.arange(32, dtype=float)[None]
    out = m.attention(q, k, v, 0)
    assert np.array_equal(out[0, :48], np.tile(np.arange(16.0), 3))           # heads 0..2 read kv head 0
    assert np.array_equal(out[0, 48:], np.tile(np.arange(16.0, 32.0), 3))     # heads 3..5 read kv head 1
