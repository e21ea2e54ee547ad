"""A plain, slow GPT-2: whole sequences, no cache, one function per part.

Written from bisand/kvad's formulas (each function cites file:line of
/crates/...).  bisand/kvad's own model code cannot be compiled here (it is
Rust; no cargo or rustc on this machine), so this file rests on the formulas
and not on a run of the reference.  It shares no code with `kvad_b200`: it
reads safetensors with its own few lines, takes config.json's keys itself and
computes with NumPy in float64 (the oracle) - or, with `round_to="bfloat16"`,
rounds activations to bfloat16 at the places where a bfloat16 engine stores
them, and matrices to bfloat16 as a bfloat16 engine holds them, so that a
bfloat16 run can be compared tightly.  That second mode follows the engine's
storage decisions (which activations and which tensors are held in bfloat16);
only the float64 mode is a statement independent of the engine.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# ----------------------------------------------------------------------------- files
def read_model_files(model_dir):
    """`model.safetensors`, or the shards that `model.safetensors.index.json` names in its
    `weight_map` (crates/llm/src/weights.rs:231-239, 269-282).  Returns (tensors, stored dtypes)."""
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        files = [single]
    else:
        with open(os.path.join(model_dir, "model.safetensors.index.json")) as f:
            files = sorted({os.path.join(model_dir, fn) for fn in json.load(f)["weight_map"].values()})
    tensors, dtypes = {}, {}
    for fn in files:
        t, d = read_safetensors(fn, with_dtypes=True)
        tensors.update(t)
        dtypes.update(d)
    return tensors, dtypes


def read_safetensors(path, with_dtypes=False):
    """u64 header length, JSON header, blob (crates/llm/src/weights.rs:9-13)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    out, dtypes = {}, {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = blob[lo:hi]
        dt = info["dtype"]
        if dt == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif dt == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif dt == "F16":
            a = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        elif dt in ("I64", "I32"):
            a = np.frombuffer(raw, dtype="<i8" if dt == "I64" else "<i4")
        else:
            raise ValueError(f"plain reader: dtype {dt}")
        out[name] = a.reshape(info["shape"])
        dtypes[name] = dt
    return (out, dtypes) if with_dtypes else out


def round_bf16(a):
    """Round-to-nearest-even to bfloat16, kept in float64."""
    f = np.asarray(a, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64)


class PlainGpt2:
    def __init__(self, model_dir, round_to=None):
        with open(os.path.join(model_dir, "config.json")) as f:
            c = json.load(f)
        self.c = c
        w, stored = read_model_files(model_dir)
        # names may carry a prefix (crates/llm/src/weights.rs:866-868)
        self.w = {}
        for k, v in w.items():
            dt = stored[k]
            for p in ("transformer.", "model."):
                if k.startswith(p):
                    k = k[len(p):]
            # a bfloat16 engine holds everything in bfloat16 except vectors that the file stores in 32-bit
            if round_to == "bfloat16" and v.dtype.kind == "f" and not (dt == "F32" and v.ndim <= 1):
                v = round_bf16(v)
            self.w[k] = v
        # keys and defaults: crates/llm/src/model/mod.rs:343-364
        self.E = c.get("n_embd", c.get("hidden_size"))
        self.H = c.get("n_head", c.get("num_attention_heads"))
        self.L = c.get("n_layer", c.get("num_hidden_layers"))
        self.hd = c.get("head_dim") or self.E // self.H
        self.Hkv = c.get("num_key_value_heads") or self.H
        self.eps = c.get("layer_norm_epsilon", 1e-5)
        self.act = c.get("activation_function", "gelu_new")
        self.inv_layer = bool(c.get("scale_attn_by_inverse_layer_idx", False))
        self.tied = c.get("tie_word_embeddings", True)
        self.r = (lambda a: round_bf16(a)) if round_to == "bfloat16" else (lambda a: a)

    # ------------------------------------------------------------------------- parts
    def embed(self, tokens, pos0=0):
        """x[i] = wte[token_i] + wpe[pos0 + i]  (crates/llm/src/model/gpt2.rs:200-213)."""
        tokens = np.asarray(tokens)
        return self.w["wte.weight"][tokens] + self.w["wpe.weight"][pos0 + np.arange(len(tokens))]

    def layer_norm(self, x, g, b):
        """mean; biased variance; 1/sqrt(var+eps); gain and bias (crates/llm/src/tensor.rs:245-255)."""
        mean = x.mean(axis=-1, keepdims=True)
        var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
        return (x - mean) / np.sqrt(var + self.eps) * g + b

    @staticmethod
    def linear(x, w_in_out, b):
        """x . W + b with W stored [in, out] (Conv1D; crates/llm/src/model/gpt2.rs:86-97, 235);
        the bias is added after the product (crates/llm/src/quant.rs:849-857)."""
        return x @ w_in_out + b

    @staticmethod
    def gelu_tanh(t):
        """0.5 t (1 + tanh(C (t + 0.044715 t^3))), C = sqrt(2/pi) (crates/llm/src/tensor.rs:263-269)."""
        c = math.sqrt(2.0 / math.pi)
        return 0.5 * t * (1.0 + np.tanh(c * (t + 0.044715 * t ** 3)))

    @staticmethod
    def gelu_erf(t):
        """x Phi(x) through erf (crates/llm/src/tensor.rs:276-281)."""
        from math import erf
        return 0.5 * t * (1.0 + np.vectorize(erf)(t / math.sqrt(2.0)))

    def attention(self, q, k, v, layer, window=None):
        """Per head: scores = q.k * 1/sqrt(head_dim) over positions <= own; softmax with the maximum
        subtracted; weighted sum of values (crates/llm/src/model/mod.rs:769-819,
        crates/llm/src/tensor.rs:297-308).  Query head h reads KV head h // group
        (crates/llm/src/model/mod.rs:792).  With scale_attn_by_inverse_layer_idx the scores of
        block `layer` are further divided by layer + 1 (not in bisand/kvad; config.json's meaning)."""
        T = q.shape[0]
        group = self.H // self.Hkv
        scale = 1.0 / math.sqrt(self.hd)
        if self.inv_layer:
            scale /= (layer + 1)
        out = np.zeros((T, self.H * self.hd))
        causal = np.tril(np.ones((T, T), dtype=bool))
        if window:                                  # a row sees its latest `window` positions only (itself included)
            causal &= ~np.tril(np.ones((T, T), dtype=bool), -int(window))
        for h in range(self.H):
            kv = h // group
            qh = q[:, h * self.hd:(h + 1) * self.hd]
            kh = k[:, kv * self.hd:(kv + 1) * self.hd]
            vh = v[:, kv * self.hd:(kv + 1) * self.hd]
            s = (qh @ kh.T) * scale
            s = np.where(causal, s, -np.inf)
            s = s - s.max(axis=-1, keepdims=True)
            p = np.exp(s)
            p = p / p.sum(axis=-1, keepdims=True)
            out[:, h * self.hd:(h + 1) * self.hd] = p @ vh
        return out

    def block(self, x, i, window=None, rotate=None):
        """x += Attn(LN1(x)); x += MLP(LN2(x))  (crates/llm/src/model/gpt2.rs:229-266).
        `window` and `rotate` (a function of (q, k) -> (q, k)) serve tests of toy variants."""
        w, r = self.w, self.r
        p = f"h.{i}."
        h = r(self.layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"]))
        qkv = r(self.linear(h, w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"]))
        qw, kw = self.H * self.hd, self.Hkv * self.hd
        q, k, v = qkv[:, :qw], qkv[:, qw:qw + kw], qkv[:, qw + kw:]
        if rotate is not None:
            q, k = rotate(q, k)
        a = r(self.attention(q, k, v, i, window))
        x = x + self.linear(a, w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"])
        h = r(self.layer_norm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"]))
        hid = self.linear(h, w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"])
        hid = r(self.gelu_erf(hid) if self.act == "gelu" else self.gelu_tanh(hid))
        return x + self.linear(hid, w[p + "mlp.c_proj.weight"], w[p + "mlp.c_proj.bias"])

    def head(self, x):
        """logits = LN_f(x) . wte^T, or the checkpoint's own head and bias when untied
        (crates/llm/src/model/gpt2.rs:139-149, 177-179, 275-287)."""
        w = self.w
        h = self.r(self.layer_norm(x, w["ln_f.weight"], w["ln_f.bias"]))
        if self.tied:
            return h @ w["wte.weight"].T
        out = h @ w["lm_head.weight"].T
        if "lm_head.bias" in w:
            out = out + w["lm_head.bias"]
        return out

    # ------------------------------------------------------------------------- whole
    def logits(self, tokens, order=None, rows=None):
        """Logits at every position of one whole sequence, float64 [len, vocab]; with `rows`, only at
        those positions (the whole sequence still runs through the blocks)."""
        x = self.embed(tokens)
        for i in (range(self.L) if order is None else order):
            x = self.block(x, i)
        return self.head(x if rows is None else x[np.asarray(rows)])

    def greedy(self, prompt, n, stop=()):
        """Greedy continuation, recomputing the whole sequence for each token."""
        ids = list(prompt)
        out = []
        for _ in range(n):
            t = int(np.argmax(self.logits(ids)[-1]))
            if t in stop:
                break
            ids.append(t)
            out.append(t)
        return out
