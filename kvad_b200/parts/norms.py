"""Norms.  `layernorm`: centre, scale to unit variance (biased, eps inside the
root), then gain and bias - bisand/kvad's `layer_norm`
(crates/llm/src/tensor.rs:245-255).  Computed in 32-bit from the 32-bit
residual stream; gain and bias stay in 32-bit if the checkpoint stores them so.
"""
from __future__ import annotations

from ..weights.source import TensorRequest
from .base import Norm, register_part


class LayerNorm(Norm):
    graph_safe = True

    def __init__(self, prefix: str, width: int, eps: float, bias: bool = True):
        super().__init__(prefix)
        self.width, self.eps, self.has_bias = int(width), float(eps), bias
        self.gain = None
        self.bias = None

    def own_requests(self):
        out = [TensorRequest(self.prefix + "weight", (self.width,))]
        if self.has_bias:
            out.append(TensorRequest(self.prefix + "bias", (self.width,)))
        return out

    def load_own(self, fetch):
        self.gain = fetch(self.prefix + "weight", keep_f32=True)
        if self.has_bias:
            self.bias = fetch(self.prefix + "bias", keep_f32=True)
            if self.bias.dtype != self.gain.dtype:      # one dtype for the pair
                self.bias = self.bias.float()
                self.gain = self.gain.float()

    def own_tensors(self):
        return [t for t in (self.gain, self.bias) if t is not None]

    def forward(self, ctx, x, rows=None, n_rows=None):
        n = n_rows if n_rows is not None else (x.shape[0] if rows is None else rows.numel())
        out = ctx.buffer((n, self.width))
        ctx.ops.layernorm(x, self.gain, self.bias, self.eps, out, rows)
        return out


register_part("norm", "layernorm", LayerNorm)
