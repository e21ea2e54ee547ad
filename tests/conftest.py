"""Shared fixtures: tiny configurations, model folders with random weights, the plain oracle."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Two tiny configurations that differ in every size and option, and a third with grouped
# key/value heads, an explicit head size and an untied head with a bias.
TINY = {
    "A": dict(model_type="gpt2", n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512, n_positions=128,
              layer_norm_epsilon=1e-5, activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False),
    "B": dict(model_type="gpt2", n_layer=3, n_embd=96, n_head=3, n_inner=320, vocab_size=1000, n_positions=256,
              layer_norm_epsilon=1e-6, activation_function="gelu", scale_attn_by_inverse_layer_idx=True),
    "C": dict(model_type="gpt2", n_layer=2, n_embd=80, n_head=6, num_key_value_heads=2, head_dim=16, n_inner=200,
              vocab_size=777, n_positions=160, layer_norm_epsilon=1e-5, activation_function="gelu_new",
              tie_word_embeddings=False),
    # heads of 64 and 1024 positions: the tensor-core prompt attention, decode attention over up to 16 pages
    "D": dict(model_type="gpt2", n_layer=2, n_embd=128, n_head=2, n_inner=384, vocab_size=1200, n_positions=1024,
              layer_norm_epsilon=1e-5, activation_function="gelu_new"),
}
SEEDS = {"A": 11, "B": 23, "C": 37, "D": 41}
# A and B once more, in folders that this library did not write: real checkpoint layout, stored in
# 32-bit with full mantissas (tests/plain/fixture.py); U: an untied head with a bias, stored in float16
TINY["A32"], TINY["B32"] = TINY["A"], TINY["B"]
TINY["U16"] = dict(TINY["A"], tie_word_embeddings=False, n_head=2)
FOREIGN = {"A32": (13, "F32", 1), "B32": (29, "F32", 3), "U16": (31, "F16", 2)}      # seed, stored dtype, shards

# How far logits may be from the plain implementation, as max |difference| / max |reference| over a
# request.  float32 against the float64 oracle: rounding of 32-bit sums (measured 2e-7 .. 6e-7).
# bfloat16 against the oracle that rounds activations to bfloat16 at the engine's storage points:
# what is left is single bfloat16 roundings that fall the other way (measured up to 2.5e-3).  That
# oracle follows the engine's storage decisions, so only the float32 runs are an independent statement.
TOL = {"float32": 5e-6, "bfloat16": 8e-3}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def rel_err(got, ref) -> float:
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    if not np.isfinite(got).all():
        return float("inf")
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """name -> folder with config.json + model.safetensors (bfloat16 storage), made once per session."""
    from kvad_b200 import write_random_model

    from tests.plain.fixture import write_gpt2_folder

    out = {}
    for name, cfg in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny{name}")
        if name in FOREIGN:
            seed, stored, shards = FOREIGN[name]
            write_gpt2_folder(str(d), cfg, seed, stored, shards)
        else:
            write_random_model(str(d), cfg, SEEDS[name])
        out[name] = str(d)
    return out


@pytest.fixture(scope="session")
def plains(model_dirs):
    """(name, dtype) -> plain implementation; the bfloat16 one rounds where the engine stores."""
    from tests.plain.gpt2_plain import PlainGpt2

    cache = {}

    def get(name, dtype="float32"):
        key = (name, dtype)
        if key not in cache:
            cache[key] = PlainGpt2(model_dirs[name], round_to="bfloat16" if dtype == "bfloat16" else None)
        return cache[key]

    return get


@pytest.fixture(scope="session")
def engines(model_dirs):
    """(name, dtype) -> Engine, made once per session (GPU tests only)."""
    cache = {}

    def get(name, dtype, max_tokens=4096):
        from kvad_b200 import Engine

        key = (name, dtype, max_tokens)
        if key not in cache:
            cache[key] = Engine.from_pretrained(model_dirs[name], dtype, max_tokens=max_tokens)
        return cache[key]

    return get


def random_tokens(seed, n, vocab):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()
