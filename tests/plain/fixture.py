"""Model folders that the library under test did not write.

This file imports nothing from `kvad_b200`.  It writes a GPT-2 checkpoint the way real ones lie
on disk, so that the plain implementation and the engine meet only at the file format and at
bisand/kvad's documented layout (crates/llm/src/model/gpt2.rs:86-97, 107-164; the reference's own
random fixture in real layout: crates/gpu/src/gpt2.rs:449-514):

* names carry the `transformer.` prefix (crates/llm/src/weights.rs:866-868);
* the four projections of a block are Conv1D matrices stored `[in, out]`; `wte`, `wpe` and an
  untied `lm_head.weight` are stored `[rows, width]` and never transposed;
* every block carries the stored causal mask `attn.bias` and `attn.masked_bias`, which are buffers
  and not weights (crates/llm/src/weights.rs:703-721);
* LayerNorm gains and all biases are random, so a dropped affine or bias shows
  (crates/gpu/src/gpt2.rs:459-462); `c_fc` is scaled up so that the tanh and the erf form of GELU
  give visibly different logits (crates/gpu/src/gpt2.rs:480-487);
* tensors are stored in F32 with values that need all 24 bits of the mantissa (or in F16 / BF16
  on request), the file is `u64 header length + JSON header + blob` (crates/llm/src/weights.rs:9-13),
  optionally cut into shards with a `model.safetensors.index.json` (crates/llm/src/weights.rs:231-239).
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


def _to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype("<u2")


def _encode(a: np.ndarray, dtype: str):
    if a.dtype.kind in "iub":
        return "I64", np.ascontiguousarray(a, dtype="<i8").tobytes()
    if dtype == "F32":
        return "F32", np.ascontiguousarray(a, dtype="<f4").tobytes()
    if dtype == "F16":
        return "F16", np.ascontiguousarray(a, dtype="<f2").tobytes()
    if dtype == "BF16":
        return "BF16", _to_bf16_bits(a).tobytes()
    raise ValueError(dtype)


def write_safetensors_file(path: str, tensors: dict, dtype: str = "F32") -> None:
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        code, raw = _encode(np.asarray(a), dtype)
        header[name] = {"dtype": code, "shape": list(np.asarray(a).shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    head = json.dumps({"__metadata__": {"format": "pt"}, **header}, separators=(",", ":")).encode()
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for raw in blobs:
            f.write(raw)


def gpt2_tensors(cfg: dict, seed: int) -> dict:
    """Random GPT-2 tensors in the real checkpoint layout, float32 with full mantissas."""
    rng = np.random.default_rng(seed)
    E, L, H = cfg["n_embd"], cfg["n_layer"], cfg["n_head"]
    I = cfg.get("n_inner") or 4 * E
    V, P = cfg["vocab_size"], cfg["n_positions"]
    hd = cfg.get("head_dim") or E // H
    Hkv = cfg.get("num_key_value_heads") or H
    qkv_out = H * hd + 2 * Hkv * hd

    def normal(shape, std, mean=0.0):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std) + np.float32(mean)).astype(np.float32)

    t = {"transformer.wte.weight": normal((V, E), 0.02), "transformer.wpe.weight": normal((P, E), 0.02)}
    mask = np.tril(np.ones((P, P), dtype=np.int64)).reshape(1, 1, P, P) if P <= 256 else None
    for i in range(L):
        p = f"transformer.h.{i}."
        t[p + "ln_1.weight"] = normal((E,), 0.1, 1.0)
        t[p + "ln_1.bias"] = normal((E,), 0.05)
        t[p + "attn.c_attn.weight"] = normal((E, qkv_out), 0.05)          # Conv1D: [in, out]
        t[p + "attn.c_attn.bias"] = normal((qkv_out,), 0.02)
        t[p + "attn.c_proj.weight"] = normal((H * hd, E), 0.05 / math.sqrt(2 * L))
        t[p + "attn.c_proj.bias"] = normal((E,), 0.02)
        if mask is not None:
            t[p + "attn.bias"] = mask                                       # buffers, not weights
        t[p + "attn.masked_bias"] = np.asarray(-10000.0, dtype=np.float32)
        t[p + "ln_2.weight"] = normal((E,), 0.1, 1.0)
        t[p + "ln_2.bias"] = normal((E,), 0.05)
        t[p + "mlp.c_fc.weight"] = normal((E, I), 3.0 / math.sqrt(E))       # pre-activations of a few units: the GELU forms part
        t[p + "mlp.c_fc.bias"] = normal((I,), 0.1)
        t[p + "mlp.c_proj.weight"] = normal((I, E), 0.05 / math.sqrt(2 * L))
        t[p + "mlp.c_proj.bias"] = normal((E,), 0.02)
    t["transformer.ln_f.weight"] = normal((E,), 0.1, 1.0)
    t["transformer.ln_f.bias"] = normal((E,), 0.05)
    if not cfg.get("tie_word_embeddings", True):
        t["lm_head.weight"] = normal((V, E), 0.02)
        t["lm_head.bias"] = normal((V,), 0.05)
    return t


def write_gpt2_folder(model_dir: str, cfg: dict, seed: int, dtype: str = "F32", shards: int = 1) -> str:
    """config.json + model.safetensors (or `shards` files and an index) in `model_dir`."""
    os.makedirs(model_dir, exist_ok=True)
    tensors = gpt2_tensors(cfg, seed)
    if shards <= 1:
        write_safetensors_file(os.path.join(model_dir, "model.safetensors"), tensors, dtype)
    else:
        names = list(tensors)
        weight_map, total = {}, 0
        for s in range(shards):
            fn = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
            part = {n: tensors[n] for n in names[s::shards]}
            write_safetensors_file(os.path.join(model_dir, fn), part, dtype)
            weight_map.update({n: fn for n in part})
            total += sum(int(np.asarray(a).nbytes) for a in part.values())
        with open(os.path.join(model_dir, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f)
    out = dict(cfg)
    out.setdefault("architectures", ["GPT2LMHeadModel"])
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(out, f, indent=1)
    return model_dir
