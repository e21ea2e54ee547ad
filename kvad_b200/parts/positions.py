"""Position encodings.

`learned_absolute`: one learned vector per position, added to the token
embedding at the bottom of the model (bisand/kvad: `wpe`,
crates/llm/src/model/gpt2.rs:71-75, 200-213).  It bounds a sequence's length:
there is no row past the table's end.  `none`: no position information of its
own (a mixer may still bring one).
"""
from __future__ import annotations

from ..weights.source import TensorRequest
from .base import PositionEncoding, register_part


class LearnedAbsolute(PositionEncoding):
    graph_safe = True

    def __init__(self, prefix: str, n_positions: int, width: int, name: str = "wpe.weight"):
        super().__init__(prefix)
        self.max_positions, self.width, self.name = int(n_positions), int(width), name
        self.weight = None

    def own_requests(self):
        return [TensorRequest(self.prefix + self.name, (self.max_positions, self.width))]

    def load_own(self, fetch):
        self.weight = fetch(self.prefix + self.name)

    def own_tensors(self):
        return [self.weight]

    def table(self):
        return self.weight


class NoPositions(PositionEncoding):
    graph_safe = True

    def __init__(self, prefix: str = ""):
        super().__init__(prefix)


register_part("position", "learned_absolute", LearnedAbsolute)
register_part("position", "none", NoPositions)
