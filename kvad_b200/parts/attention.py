"""Causal self-attention over the cache, as a mixer.

One fused projection gives queries, keys and values (`q` first, then `k`,
then `v`; inside each, heads are contiguous groups of `head_dim` columns -
crates/llm/src/model/gpt2.rs:235-246, crates/llm/src/model/mod.rs:788-792).
This step's keys and values are written to the cache before any row attends
(crates/llm/src/model/gpt2.rs:237-242); each row then attends over its own
sequence's positions up to its own, scores scaled by `score_scale`
(1/sqrt(head_dim) in bisand/kvad, crates/llm/src/model/mod.rs:777), softmax
in 32-bit, and the output projection adds into the residual stream.
Several query heads may share one key/value head (`n_kv_heads < n_heads`),
and `window` limits each row to the latest positions.

A call with `writes_cache=False` reads the keys and values another call
wrote to the same cache entry and adds none of its own.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.layout import KVNeed
from .base import Mixer, PartSpec, build_part, register_part
from .linear import Linear


class CausalSelfAttention(Mixer):
    graph_safe = True

    def __init__(self, prefix: str, width: int, n_heads: int, head_dim: int, score_scale: float,
                 n_kv_heads: Optional[int] = None, window: Optional[int] = None, bias: bool = True,
                 stored: str = "out_in", qkv_name: str = "qkv.", out_name: str = "out.",
                 position: Optional[PartSpec] = None):
        super().__init__(prefix)
        self.width, self.n_heads, self.head_dim = int(width), int(n_heads), int(head_dim)
        self.n_kv_heads = int(n_kv_heads) if n_kv_heads else self.n_heads
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_heads} heads do not divide into {self.n_kv_heads} key/value heads")
        if self.head_dim % 16:
            raise ValueError(f"head size {self.head_dim} is not a multiple of 16")
        self.score_scale, self.window = float(score_scale), window
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv_heads * self.head_dim
        self.qkv = Linear(prefix + qkv_name, self.width, self.q_width + 2 * self.kv_width, bias=bias, stored=stored)
        self.out = Linear(prefix + out_name, self.q_width, self.width, bias=bias, stored=stored)
        self.position = build_part("position", position, prefix) if position is not None else None

    def children(self):
        return [self.qkv, self.out] + ([self.position] if self.position is not None else [])

    def cache_need(self):
        return KVNeed(self.n_kv_heads, self.head_dim, self.window)

    def forward(self, ctx, h, residual, call):
        n = h.shape[0]
        ops, view = ctx.ops, ctx.kv(call.cache)
        if (ctx.batch.is_decode and call.writes_cache and self.position is None and ops.fast_decode and ops.decode_takes(self.head_dim)
                and ops.sums_take(n, self.qkv.weight, self.head_dim, view.k_pages.shape[2])):
            # a few single-token rows: the q/k/v product leaves 32-bit sums, and the attention kernel finishes them
            # (bias, rounding, the cache write) where it reads them
            sums, clear = ops.linear_sums(h, self.qkv.weight)
            mixed = ctx.buffer((n, self.q_width))
            splits = ops.decode_splits(n, self.n_heads, view.page_table.shape[1])
            scratch = ctx.buffer((n * self.n_heads * splits * (self.head_dim + 2),), torch.float32) if splits > 1 else None
            ops.attention_decode_sums(sums, self.qkv.bias, self.q_width, self.q_width + self.kv_width, clear, mixed, ctx.row_seq,
                                      ctx.row_pos, view.page_table, view.k_pages, view.v_pages, self.n_heads, self.score_scale,
                                      view.window or 0, n_splits=splits, scratch=scratch)
            self.out.forward(ctx, mixed, residual, "residual")
            return
        qkv = ctx.buffer((n, self.q_width + 2 * self.kv_width))
        self.qkv.forward(ctx, h, qkv)
        q = qkv[:, : self.q_width]
        k = qkv[:, self.q_width: self.q_width + self.kv_width]
        v = qkv[:, self.q_width + self.kv_width:]
        if self.position is not None:
            self.position.rotate(ctx, q, k)
        view = ctx.kv(call.cache)
        mixed = ctx.buffer((n, self.q_width))
        self.attend(ctx, q, k, v, mixed, view, call.writes_cache)
        self.out.forward(ctx, mixed, residual, "residual")

    def attend(self, ctx, q, k, v, out, view, writes_cache: bool = True) -> None:
        """Writes the rows' keys and values to the cache entry (if this call owns it) and lets every
        row attend over its sequence up to its own position.  The kernels are chosen by the step's
        shape class (single-token rows or prompts) and this mixer's head size, never by lengths."""
        ops, b, n_heads, scale = ctx.ops, ctx.batch, self.n_heads, self.score_scale
        hd = self.head_dim
        if b.is_decode and ops.fast_decode and ops.decode_takes(hd):
            splits = ops.decode_splits(ctx.n_rows, n_heads, view.page_table.shape[1])
            scratch = ctx.buffer((ctx.n_rows * n_heads * splits * (hd + 2),), torch.float32) if splits > 1 else None
            ops.attention_decode(q, out, ctx.row_seq, ctx.row_pos, view.page_table, view.k_pages, view.v_pages,
                                 n_heads, scale, view.window or 0, n_splits=splits, scratch=scratch,
                                 k_new=k if writes_cache else None, v_new=v if writes_cache else None,
                                 merge_in_kernel=True)
            return
        if writes_cache:
            ops.kv_store(k, v, ctx.row_seq, ctx.row_pos, view.page_table, view.k_pages, view.v_pages)
        if (not b.is_decode) and ops.tensor_core_prefill and ops.prefill_takes(hd):
            ops.attention_prefill(q, out, ctx.seq_starts, ctx.kv_lens, ctx.n_seqs, b.max_new, view.page_table,
                                  view.k_pages, view.v_pages, n_heads, scale, view.window or 0)
        elif (not b.is_decode) and ops.tiled_prompt and ops.prompt_takes(hd, view.k_pages.shape[2]):
            ops.attention_prompt(q, out, ctx.seq_starts, ctx.kv_lens, ctx.n_seqs, b.max_new, view.page_table,
                                 view.k_pages, view.v_pages, n_heads, scale, view.window or 0)
        else:
            ops.attention(q, out, ctx.row_seq, ctx.row_pos, view.page_table, view.k_pages, view.v_pages,
                          n_heads, scale, view.window or 0)


register_part("mixer", "causal_attention", CausalSelfAttention)
