"""A linear map with an optional bias: the matrix product every other part uses.

Held `[out, in]` (rows are outputs), which is the layout both operands of the
tensor-core kernel want and the layout a tied output head already has.  A
checkpoint may store it `[in, out]` (GPT-2's Conv1D); then it is transposed
once while loading, as bisand/kvad's `matrix_t` does
(crates/llm/src/model/gpt2.rs:86-97, crates/llm/src/qcache.rs:539-544).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..weights.source import TensorRequest
from .base import Part


class Linear(Part):
    graph_safe = True

    def __init__(self, prefix: str, in_features: int, out_features: int, *, bias: bool = True,
                 stored: str = "out_in", shared_weight: Optional[torch.Tensor] = None,
                 bias_optional: bool = False, has_weight: bool = True):
        super().__init__(prefix)
        if stored not in ("out_in", "in_out"):
            raise ValueError("stored must be `out_in` or `in_out`")
        self.in_features, self.out_features = int(in_features), int(out_features)
        self.has_bias, self.bias_optional, self.stored = bias, bias_optional, stored
        self.has_weight = has_weight            # False: the weight is lent by another part (a tied head)
        self.weight: Optional[torch.Tensor] = shared_weight
        self.bias: Optional[torch.Tensor] = None

    def own_requests(self):
        out = []
        if self.has_weight:
            shape = (self.out_features, self.in_features) if self.stored == "out_in" else (self.in_features, self.out_features)
            out.append(TensorRequest(self.prefix + "weight", shape))
        if self.has_bias:
            out.append(TensorRequest(self.prefix + "bias", (self.out_features,), optional=self.bias_optional))
        return out

    def load_own(self, fetch):
        if self.has_weight:
            self.weight = fetch(self.prefix + "weight", transpose=self.stored == "in_out")
        if self.has_bias:
            self.bias = fetch(self.prefix + "bias", keep_f32=True, optional=self.bias_optional)

    def own_tensors(self):
        return [t for t in ((self.weight if self.has_weight else None), self.bias) if t is not None]

    def forward(self, ctx, a, out: torch.Tensor, epilogue: str = "store") -> torch.Tensor:
        """out = epilogue(a . W^T + b)."""
        ctx.ops.linear(a, self.weight, self.bias, out, epilogue)
        return out
