"""Random-weights mode: a model folder from a configuration and a seed.

Writes `config.json` and `model.safetensors` so that everything downstream
(the loader, the audit, generation, trace replay, the benchmark) runs exactly
as it does for a trained checkpoint.  Which tensors exist and how each is
distributed is the architecture's business (`Architecture.random_tensors`);
this module only owns the generator, the storage dtype and the files.

bisand/kvad has no such engine mode; its tests write random checkpoints in the
real layout (crates/gpu/src/gpt2.rs:449-514, crates/llm/tests/common/mod.rs:243-277)
with gains and biases away from 1 and 0 so that a dropped affine shows.
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch

from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
          "f32": torch.float32, "float16": torch.float16, "f16": torch.float16}


class SeededNormal:
    """Seeded normal and uniform draws (PCG64 through NumPy)."""

    def __init__(self, seed: int):
        self._rng = np.random.default_rng(int(seed))

    def normal(self, shape, std: float = 1.0, mean: float = 0.0) -> torch.Tensor:
        a = self._rng.standard_normal(size=tuple(shape), dtype=np.float32)
        if std != 1.0:
            a *= np.float32(std)
        if mean != 0.0:
            a += np.float32(mean)
        return torch.from_numpy(a)

    def integers(self, low: int, high: int, shape) -> torch.Tensor:
        return torch.from_numpy(self._rng.integers(low, high, size=tuple(shape), dtype=np.int64))


def write_random_model(model_dir: str, config, seed: int, *, arch_id: str | None = None,
                       store_dtype: str = "bfloat16") -> str:
    """Creates `model_dir` with config.json and model.safetensors.

    `config` is either an architecture's typed configuration or a dict in
    config.json's own keys (then the architecture is found by its
    `model_type`).  Floating tensors are stored in `store_dtype`; storing in
    bfloat16 gives the 32-bit and the bfloat16 engines the same values.
    """
    from ..config import JsonView, by_id, resolve
    from .. import models  # noqa: F401  (registers the built-in architectures)

    if isinstance(config, dict):
        view = JsonView(config)
        arch = by_id(arch_id) if arch_id else resolve(view)
        typed = arch.read_config(view)
    else:
        typed = config
        arch = by_id(arch_id or getattr(config, "arch_id", ""))
    if arch is None or arch.random_tensors is None or arch.write_config is None:
        raise ValueError("this architecture has no random-weights mode")
    if store_dtype not in _STORE:
        raise ValueError(f"store_dtype must be one of {sorted(_STORE)}")
    dtype = _STORE[store_dtype]

    os.makedirs(model_dir, exist_ok=True)
    tensors = arch.random_tensors(typed, SeededNormal(seed))
    stored = {n: (t.to(dtype) if t.is_floating_point() else t) for n, t in tensors.items()}
    write_safetensors(os.path.join(model_dir, "model.safetensors"), stored,
                      metadata={"format": "pt", "seed": str(seed)})
    cfg = dict(arch.write_config(typed))
    cfg["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=2)
        f.write("\n")
    return model_dir
