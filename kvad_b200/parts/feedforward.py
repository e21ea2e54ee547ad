"""Feed-forwards.  `dense_mlp`: widen, activate, come back, add to the
residual stream (crates/llm/src/model/gpt2.rs:256-265).  The activation is a
parameter: `gelu_tanh` is bisand/kvad's hard-wired form
(crates/llm/src/tensor.rs:263-269), `gelu_erf` the exact one
(crates/llm/src/tensor.rs:276-281).  Bias and activation ride in the first
product's epilogue, bias and the residual sum in the second's.
"""
from __future__ import annotations

from .base import FeedForward, register_part
from .linear import Linear

ACTIVATIONS = {"gelu_tanh": "gelu_tanh", "gelu_erf": "gelu_erf"}


class DenseMLP(FeedForward):
    graph_safe = True

    def __init__(self, prefix: str, width: int, hidden: int, activation: str, bias: bool = True,
                 stored: str = "out_in", up_name: str = "up.", down_name: str = "down."):
        super().__init__(prefix)
        if activation not in ACTIVATIONS:
            raise ValueError(f"dense_mlp has no activation `{activation}`; it has {sorted(ACTIVATIONS)}")
        self.width, self.hidden, self.activation = int(width), int(hidden), activation
        self.up = Linear(prefix + up_name, self.width, self.hidden, bias=bias, stored=stored)
        self.down = Linear(prefix + down_name, self.hidden, self.width, bias=bias, stored=stored)

    def children(self):
        return [self.up, self.down]

    def forward(self, ctx, h, residual):
        hid = ctx.buffer((h.shape[0], self.hidden))
        self.up.forward(ctx, h, hid, ACTIVATIONS[self.activation])
        self.down.forward(ctx, hid, residual, "residual")


register_part("feed_forward", "dense_mlp", DenseMLP)
