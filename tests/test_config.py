"""Configuration and registry (no GPU)."""
import json

import pytest

from kvad_b200.config import (Architecture, ConfigError, JsonView, architectures, from_model_type, load_config,
                              register, resolve, unregister)
from kvad_b200.models import gpt2
from tests.conftest import TINY


def view(**kw):
    return JsonView(dict(kw))


def test_reads_every_key_and_alias():
    c = gpt2.read_config(view(model_type="gpt2", num_hidden_layers=5, hidden_size=48, num_attention_heads=3,
                              intermediate_size=100, max_position_embeddings=77, vocab_size=99,
                              rms_norm_eps=1e-3, activation_function="gelu", scale_attn_by_inverse_layer_idx=True,
                              tie_word_embeddings=False, eos_token_id=[3, 4]))
    assert (c.n_layer, c.n_embd, c.n_head, c.n_inner, c.n_positions, c.vocab_size) == (5, 48, 3, 100, 77, 99)
    assert c.layer_norm_epsilon == pytest.approx(1e-3) and c.activation_function == "gelu"
    assert c.scale_attn_by_inverse_layer_idx and not c.tie_word_embeddings and c.eos_token_ids == (3, 4)
    assert c.head_dim == 16 and c.n_kv_head == 3


def test_defaults():
    c = gpt2.read_config(view(model_type="gpt2", n_layer=1, n_embd=32, n_head=2, vocab_size=10, n_inner=None))
    assert c.n_inner == 128 and c.n_positions == 1024 and c.layer_norm_epsilon == pytest.approx(1e-5)
    assert c.activation_function == "gelu_new" and c.tie_word_embeddings and not c.scale_attn_by_inverse_layer_idx


@pytest.mark.parametrize("drop,what", [("n_embd", "hidden size"), ("n_head", "head count"),
                                      ("n_layer", "layer count"), ("vocab_size", "vocab_size")])
def test_missing_required_key(drop, what):
    cfg = dict(TINY["A"])
    del cfg[drop]
    with pytest.raises(ConfigError, match=what):
        gpt2.read_config(JsonView(cfg))


def test_refuses_what_the_kernels_cannot_run():
    with pytest.raises(ConfigError, match="not divisible"):
        gpt2.read_config(view(model_type="gpt2", n_layer=1, n_embd=50, n_head=3, vocab_size=10))
    with pytest.raises(ConfigError, match="multiple of 16"):
        gpt2.read_config(view(model_type="gpt2", n_layer=1, n_embd=40, n_head=4, vocab_size=10))
    with pytest.raises(ConfigError, match="activation_function"):
        gpt2.read_config(view(model_type="gpt2", n_layer=1, n_embd=32, n_head=2, vocab_size=10, activation_function="relu"))
    with pytest.raises(ConfigError, match="key/value heads"):
        gpt2.read_config(view(model_type="gpt2", n_layer=1, n_embd=96, n_head=6, num_key_value_heads=4, vocab_size=10))


def test_registry_matches_exactly():
    assert from_model_type("gpt2").id == "gpt2"
    assert from_model_type("GPT2LMHeadModel").id == "gpt2"
    for near in ("gpt2_moe", "gpt", "gpt-neo", "gpt22", "llama"):
        assert from_model_type(near) is None, near


def test_unknown_architecture_lists_what_runs():
    with pytest.raises(ConfigError) as e:
        resolve(view(model_type="qwen3_next"))
    assert "unsupported architecture `qwen3_next`" in str(e.value) and "gpt2" in str(e.value)
    with pytest.raises(ConfigError, match="neither model_type nor architectures"):
        resolve(view(n_layer=1))
    assert resolve(view(architectures=["GPT2LMHeadModel"])).id == "gpt2"


def test_no_two_architectures_claim_one_type():
    clash = Architecture("other", ("GPT2",), "x", lambda v: None, lambda c: None)
    with pytest.raises(ValueError, match="both claim"):
        register(clash)
    ok = Architecture("toy-arch", ("toyarch",), "x", lambda v: None, lambda c: None)
    register(ok)
    try:
        assert "toy-arch" in [a.id for a in architectures()]
        with pytest.raises(ValueError, match="already registered"):
            register(ok)
    finally:
        unregister("toy-arch")


def test_plan_is_data_with_no_hidden_sizes():
    c = gpt2.read_config(JsonView(TINY["B"]))
    p = gpt2.plan(c)
    assert len(p.blocks) == 3 and [x.layer for x in p.order] == [0, 1, 2]
    m0, m2 = p.blocks[0].params["mixer"].params, p.blocks[2].params["mixer"].params
    assert m0["head_dim"] == 32 and m0["n_heads"] == 3
    assert m2["score_scale"] == pytest.approx(m0["score_scale"] / 3)       # inverse layer index
    assert p.blocks[1].params["feed_forward"].params["activation"] == "gelu_erf"
    assert p.blocks[1].params["feed_forward"].params["hidden"] == 320


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY["A"]))
    arch, c = load_config(str(tmp_path))
    assert arch.id == "gpt2" and c.n_embd == 64
    assert gpt2.read_config(JsonView(gpt2.write_config(c))) == c
