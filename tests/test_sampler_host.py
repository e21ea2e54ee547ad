"""The sampling rule on the host and the random stream (no GPU)."""
import numpy as np
import pytest

from kvad_b200.sampling import SamplingParams, Xorshift64Star, argmax, sample_host, shortlist


def test_xorshift64star_is_the_reference_generator():
    # crates/nervus/src/rng.rs:12-31: seed 0 is replaced; shifts 12, 25, 27; multiplier 0x2545F4914F6CDD1D
    r = Xorshift64Star(0)
    assert r.state == 0x9E3779B97F4A7C15
    x = 1
    x ^= x >> 12
    x ^= (x << 25) & (2**64 - 1)
    x ^= x >> 27
    assert Xorshift64Star(1).next_u64() == (x * 0x2545F4914F6CDD1D) % 2**64
    r = Xorshift64Star(7)
    us = [r.uniform() for _ in range(1000)]
    assert all(0 <= u < 1 for u in us) and 0.4 < np.mean(us) < 0.6
    assert all(float(u * 2**24).is_integer() for u in us)


def test_argmax_first_of_equals_and_nan_never_wins():
    assert argmax([1.0, 3.0, 3.0, 2.0]) == 1
    assert argmax([float("nan"), 1.0, float("nan")]) == 1
    assert argmax([-1.0]) == 0


def test_shortlist_order_topk_topp():
    logits = np.array([0.0, 2.0, 2.0, 1.0, -1.0], dtype=np.float32)
    order, probs = shortlist(logits, 1.0, 0, 1.0)
    assert order.tolist() == [1, 2, 3, 0, 4]                      # ties by lower id
    assert probs.sum() == pytest.approx(1.0, abs=1e-6)
    order, probs = shortlist(logits, 1.0, 3, 1.0)
    assert order.tolist() == [1, 2, 3] and probs.sum() == pytest.approx(1.0, abs=1e-6)
    order, probs = shortlist(logits, 1.0, 0, 0.5)                  # p(1)=p(2)=0.366: two are needed to reach 0.5
    assert order.tolist() == [1, 2]
    order, _ = shortlist(logits, 0.01, 0, 0.9)                     # a cold distribution keeps its ties only
    assert order.tolist() == [1, 2]


def test_draw_walks_the_kept_mass():
    logits = np.log(np.array([0.5, 0.3, 0.2], dtype=np.float32))
    p = SamplingParams(1.0, 0, 1.0)
    assert sample_host(logits, p, 0.0) == 0
    assert sample_host(logits, p, 0.49) == 0
    assert sample_host(logits, p, 0.51) == 1
    assert sample_host(logits, p, 0.81) == 2
    assert sample_host(logits, p, 0.999999) == 2
    assert sample_host(logits, SamplingParams(0.0, 40, 0.9), 0.9) == 0        # greedy
    # top_p draws against the kept, unrenormalised mass (crates/llm/src/sampler.rs:60-71)
    assert sample_host(logits, SamplingParams(1.0, 0, 0.7), 0.7) == 1


def test_same_seed_same_tokens():
    from kvad_b200.sampling import RequestSampler
    rng = np.random.default_rng(0)
    rows = rng.standard_normal((50, 300)).astype(np.float32)
    a = RequestSampler(SamplingParams(0.7, 40, 0.95, seed=3))
    b = RequestSampler(SamplingParams(0.7, 40, 0.95, seed=3))
    c = RequestSampler(SamplingParams(0.7, 40, 0.95, seed=4))
    ta, tb, tc = ([s.sample(r) for r in rows] for s in (a, b, c))
    assert ta == tb and ta != tc
