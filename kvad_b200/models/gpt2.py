"""GPT-2: learned positions, LayerNorm before each sub-block, fused QKV, GELU MLP.

    x = wte[token] + wpe[position]
    x = x + Attention(LayerNorm(x));  x = x + MLP(LayerNorm(x))      (n_layer times)
    logits = LayerNorm(x) . wte^T

bisand/kvad's implementation is crates/llm/src/model/gpt2.rs (registry entry
:26-33, tensor names :107-164, forward :200-287).  Config keys and their
defaults follow crates/llm/src/model/mod.rs:323-372.  Two options that
bisand/kvad does not read are honoured here because config.json gives them:
`activation_function` (`gelu_new` / `gelu_pytorch_tanh`: the tanh form
bisand/kvad hard-wires at gpt2.rs:261; `gelu`: the exact form) and
`scale_attn_by_inverse_layer_idx` (scores of block i further divided by i+1).
`num_key_value_heads` and `head_dim`, which bisand/kvad's `Spec` reads for
every architecture, are honoured too.

This module only describes: the typed configuration, the plan (which parts,
with which sizes and tensor names), and the random-weights recipe.  All
computing is in the parts.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

from ..config.json_view import ConfigError, JsonView
from ..config.registry import Architecture, register
from ..parts.base import PartSpec
from .plan import ModelPlan

_ACTIVATIONS = {"gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh", "gelu_fast": "gelu_tanh",
                "gelu": "gelu_erf"}


@dataclass(frozen=True)
class Gpt2Config:
    n_layer: int
    n_embd: int
    n_head: int
    n_kv_head: int
    head_dim: int
    n_inner: int
    n_positions: int
    vocab_size: int
    layer_norm_epsilon: float
    activation_function: str
    scale_attn_by_inverse_layer_idx: bool
    tie_word_embeddings: bool
    eos_token_ids: tuple[int, ...] = ()
    arch_id: str = "gpt2"


def read_config(view: JsonView) -> Gpt2Config:
    n_embd = view.need(["n_embd", "hidden_size"], "hidden size")
    n_head = view.need(["n_head", "num_attention_heads"], "head count")
    n_layer = view.need(["n_layer", "num_hidden_layers"], "layer count")
    vocab = view.need(["vocab_size"], "vocab_size")
    if n_head == 0 or n_embd == 0 or n_layer == 0 or vocab == 0:
        raise ConfigError("config: sizes must be positive")
    head_dim = view.num(["head_dim"])
    if head_dim is None:
        if n_embd % n_head:
            raise ConfigError(f"config: hidden size {n_embd} is not divisible by {n_head} heads")
        head_dim = n_embd // n_head
    n_kv = view.num(["num_key_value_heads"]) or n_head
    if n_head % n_kv:
        raise ConfigError(f"config: {n_head} heads do not divide into {n_kv} key/value heads")
    if head_dim % 16:
        raise ConfigError(f"config: head size {head_dim} is not a multiple of 16, which the kernels need")
    act = view.text("activation_function") or "gelu_new"
    if act not in _ACTIVATIONS:
        raise ConfigError(f"config: activation_function `{act}` is not one of {sorted(_ACTIVATIONS)}")
    tie = view.flag("tie_word_embeddings")
    return Gpt2Config(
        n_layer=n_layer, n_embd=n_embd, n_head=n_head, n_kv_head=n_kv, head_dim=head_dim,
        n_inner=view.num(["n_inner", "intermediate_size"]) or 4 * n_embd,
        n_positions=view.num(["n_positions", "n_ctx", "max_position_embeddings"]) or 1024,
        vocab_size=vocab,
        layer_norm_epsilon=view.float(["layer_norm_epsilon", "rms_norm_eps"]) or 1e-5,
        activation_function=act,
        scale_attn_by_inverse_layer_idx=bool(view.flag("scale_attn_by_inverse_layer_idx")),
        tie_word_embeddings=True if tie is None else tie,
        eos_token_ids=tuple(view.id_list("eos_token_id")),
    )


def write_config(c: Gpt2Config) -> dict:
    d = {
        "model_type": "gpt2", "architectures": ["GPT2LMHeadModel"],
        "n_layer": c.n_layer, "n_embd": c.n_embd, "n_head": c.n_head, "n_inner": c.n_inner,
        "n_positions": c.n_positions, "n_ctx": c.n_positions, "vocab_size": c.vocab_size,
        "layer_norm_epsilon": c.layer_norm_epsilon, "activation_function": c.activation_function,
        "scale_attn_by_inverse_layer_idx": c.scale_attn_by_inverse_layer_idx,
        "tie_word_embeddings": c.tie_word_embeddings,
    }
    if c.n_kv_head != c.n_head:
        d["num_key_value_heads"] = c.n_kv_head
    if c.head_dim * c.n_head != c.n_embd:
        d["head_dim"] = c.head_dim
    if c.eos_token_ids:
        d["eos_token_id"] = list(c.eos_token_ids) if len(c.eos_token_ids) > 1 else c.eos_token_ids[0]
    return d


def plan(c: Gpt2Config) -> ModelPlan:
    norm = PartSpec("layernorm", {"width": c.n_embd, "eps": c.layer_norm_epsilon})
    blocks, prefixes = [], []
    for i in range(c.n_layer):
        scale = 1.0 / math.sqrt(c.head_dim)
        if c.scale_attn_by_inverse_layer_idx:
            scale /= float(i + 1)
        mixer = PartSpec("causal_attention", {
            "width": c.n_embd, "n_heads": c.n_head, "n_kv_heads": c.n_kv_head, "head_dim": c.head_dim,
            "score_scale": scale, "stored": "in_out", "qkv_name": "c_attn.", "out_name": "c_proj."})
        ff = PartSpec("dense_mlp", {
            "width": c.n_embd, "hidden": c.n_inner, "activation": _ACTIVATIONS[c.activation_function],
            "stored": "in_out", "up_name": "c_fc.", "down_name": "c_proj."})
        blocks.append(PartSpec("pre_norm", {
            "norm1": norm, "mixer": mixer, "norm2": norm, "feed_forward": ff,
            "norm1_name": "ln_1.", "mixer_name": "attn.", "norm2_name": "ln_2.", "feed_forward_name": "mlp."}))
        prefixes.append(f"h.{i}.")
    gqa = "" if c.n_kv_head == c.n_head else f" ({c.n_kv_head} KV heads)"
    return ModelPlan(
        arch_id="gpt2", vocab_size=c.vocab_size, width=c.n_embd,
        embedding=PartSpec("token_embedding", {
            "vocab_size": c.vocab_size, "width": c.n_embd, "name": "wte.weight",
            "position": PartSpec("learned_absolute", {"n_positions": c.n_positions, "width": c.n_embd, "name": "wpe.weight"})}),
        blocks=tuple(blocks), block_prefixes=tuple(prefixes),
        head=PartSpec("lm_head", {"vocab_size": c.vocab_size, "width": c.n_embd, "norm": norm,
                                  "tied": c.tie_word_embeddings, "bias": True, "norm_name": "ln_f.", "name": "lm_head."}),
        order=ModelPlan.straight_order(c.n_layer),
        # stored causal masks and the like are buffers, not weights (crates/llm/src/weights.rs:716-721)
        ignored_suffixes=(".attn.bias", ".attn.masked_bias", "rotary_emb.inv_freq", "embeddings.position_ids"),
        eos_token_ids=c.eos_token_ids, max_positions=c.n_positions,
        summary=(f"gpt2 · {c.n_layer} layers · {c.n_head} heads{gqa} · {c.n_embd} embd · "
                 f"{c.n_positions} ctx · {c.vocab_size} vocab"),
    )


def random_tensors(c: Gpt2Config, rng) -> dict:
    """Matrices and embeddings ~N(0, 0.02); the two matrices that write to the
    residual stream ~N(0, 0.02/sqrt(2 n_layer)) (crates/nervus/src/model.rs:99-114);
    biases ~N(0, 0.01), gains ~1+N(0, 0.05), norm biases ~N(0, 0.02): away from
    0 and 1 so that a dropped bias or gain shows (crates/gpu/src/gpt2.rs:459-462)."""
    e, q, kv = c.n_embd, c.n_head * c.head_dim, c.n_kv_head * c.head_dim
    resid = 0.02 / math.sqrt(2 * c.n_layer)
    t = {"wte.weight": rng.normal((c.vocab_size, e), 0.02), "wpe.weight": rng.normal((c.n_positions, e), 0.02)}
    for i in range(c.n_layer):
        p = f"h.{i}."
        t[p + "ln_1.weight"] = rng.normal((e,), 0.05, 1.0)
        t[p + "ln_1.bias"] = rng.normal((e,), 0.02)
        t[p + "attn.c_attn.weight"] = rng.normal((e, q + 2 * kv), 0.02)       # Conv1D layout: [in, out]
        t[p + "attn.c_attn.bias"] = rng.normal((q + 2 * kv,), 0.01)
        t[p + "attn.c_proj.weight"] = rng.normal((q, e), resid)
        t[p + "attn.c_proj.bias"] = rng.normal((e,), 0.01)
        t[p + "ln_2.weight"] = rng.normal((e,), 0.05, 1.0)
        t[p + "ln_2.bias"] = rng.normal((e,), 0.02)
        t[p + "mlp.c_fc.weight"] = rng.normal((e, c.n_inner), 0.02)
        t[p + "mlp.c_fc.bias"] = rng.normal((c.n_inner,), 0.01)
        t[p + "mlp.c_proj.weight"] = rng.normal((c.n_inner, e), resid)
        t[p + "mlp.c_proj.bias"] = rng.normal((e,), 0.01)
    t["ln_f.weight"] = rng.normal((e,), 0.05, 1.0)
    t["ln_f.bias"] = rng.normal((e,), 0.02)
    if not c.tie_word_embeddings:
        t["lm_head.weight"] = rng.normal((c.vocab_size, e), 0.02)
        t["lm_head.bias"] = rng.normal((c.vocab_size,), 0.01)
    return t


ARCH = register(Architecture(
    id="gpt2", model_types=("gpt2",),
    about="GPT-2 (2019): learned positions, LayerNorm, GELU, one fused QKV matrix",
    read_config=read_config, plan=plan, write_config=write_config, random_tensors=random_tensors,
), replace=True)
