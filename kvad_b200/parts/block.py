"""Block arrangements.  `pre_norm`: x += mixer(norm1(x)); x += ff(norm2(x))
(crates/llm/src/model/gpt2.rs:6-9, 229-266).  The residual stream stays in
32-bit; the parts add into it.
"""
from __future__ import annotations

from .base import Block, PartSpec, build_part, register_part


class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, prefix: str, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, feed_forward: PartSpec,
                 norm1_name: str = "norm1.", mixer_name: str = "mixer.", norm2_name: str = "norm2.",
                 feed_forward_name: str = "ff."):
        super().__init__(prefix)
        self.norm1 = build_part("norm", norm1, prefix + norm1_name)
        self.mixer = build_part("mixer", mixer, prefix + mixer_name)
        self.norm2 = build_part("norm", norm2, prefix + norm2_name)
        self.feed_forward = build_part("feed_forward", feed_forward, prefix + feed_forward_name)

    def children(self):
        return [self.norm1, self.mixer, self.norm2, self.feed_forward]

    def forward(self, ctx, x, call):
        h = self.norm1.forward(ctx, x, n_rows=ctx.n_rows)
        self.mixer.forward(ctx, h, x, call)
        h = self.norm2.forward(ctx, x, n_rows=ctx.n_rows)
        self.feed_forward.forward(ctx, h, x)


register_part("block", "pre_norm", PreNormBlock)
