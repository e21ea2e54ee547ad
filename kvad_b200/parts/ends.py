"""The two ends of a model: token embedding at the bottom, output head on top.

`token_embedding`: x[r] = table[token[r]] (+ the position encoding's table
row, if it has one), into the 32-bit residual stream
(crates/llm/src/model/gpt2.rs:200-213).  `lm_head`: the final norm over the
rows whose logits are wanted, then one product with the `[vocab, width]`
matrix - the embedding table itself when the head is tied, so no second copy
exists (crates/llm/src/model/gpt2.rs:139-149, 177-179, 275-287).  Logits are
32-bit.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..weights.source import TensorRequest
from .base import Part, PartSpec, build_part, register_part
from .linear import Linear


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, prefix: str, vocab_size: int, width: int, name: str = "wte.weight",
                 position: Optional[PartSpec] = None):
        super().__init__(prefix)
        self.vocab_size, self.width, self.name = int(vocab_size), int(width), name
        self.weight: Optional[torch.Tensor] = None
        self.position = build_part("position", position, prefix) if position is not None else None

    def children(self):
        return [self.position] if self.position is not None else []

    def own_requests(self):
        return [TensorRequest(self.prefix + self.name, (self.vocab_size, self.width))]

    def load_own(self, fetch):
        self.weight = fetch(self.prefix + self.name)

    def own_tensors(self):
        return [self.weight]

    @property
    def max_positions(self):
        return self.position.max_positions if self.position is not None else None

    def forward(self, ctx) -> torch.Tensor:
        x = ctx.buffer((ctx.n_rows, self.width), torch.float32)
        table = self.position.table() if self.position is not None else None
        ctx.ops.embed(ctx.tokens, ctx.row_pos, self.weight, table, x)
        return x


class LMHead(Part):
    graph_safe = True

    def __init__(self, prefix: str, vocab_size: int, width: int, norm: PartSpec, tied: bool,
                 norm_name: str = "ln_f.", name: str = "lm_head.", bias: bool = False,
                 embedding: Optional[TokenEmbedding] = None):
        super().__init__(prefix)
        self.vocab_size, self.width, self.tied = int(vocab_size), int(width), bool(tied)
        self.norm = build_part("norm", norm, prefix + norm_name)
        self.embedding = embedding
        if self.tied and embedding is None:
            raise ValueError("a tied head needs the embedding it is tied to")
        # an untied head may bring a bias; a tied one never reads `lm_head.*`
        self.proj = Linear(prefix + name, self.width, self.vocab_size, bias=(bias and not self.tied),
                           bias_optional=True, has_weight=not self.tied)
        self.skipped = [prefix + name + "weight", prefix + name + "bias"] if self.tied else []

    def children(self):
        return [self.norm, self.proj]

    def forward(self, ctx, x) -> torch.Tensor:
        n = ctx.n_want
        logits = ctx.buffer((n, self.vocab_size), torch.float32)
        if n == 0:
            return logits
        h = self.norm.forward(ctx, x, rows=ctx.want_rows, n_rows=n)
        if self.tied:
            self.proj.weight = self.embedding.weight
        self.proj.forward(ctx, h, logits, "store_f32")
        return logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
