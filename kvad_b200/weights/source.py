"""A model's view of a checkpoint: tensors asked for by name, and one audit.

A model states every tensor it needs (name, stored shape, float or integer)
before any byte is read.  `WeightSource.check` compares that list with what
the files hold and raises ONE error that lists everything wrong at once:
tensors that are missing, tensors nobody asked for, and tensors whose stored
shape is not what the configuration implies.  Only then are tensors read.

bisand/kvad does the same in two halves: its loader remembers what was read
and refuses a checkpoint with unread tensors (crates/llm/src/qcache.rs:1391-1403,
names collapsed as `h.*.x (12 tensors)` by crates/llm/src/weights.rs:730-757),
and reports a missing tensor by name (crates/llm/src/weights.rs:922).  Names
may carry a `transformer.` or `model.` prefix (crates/llm/src/weights.rs:866-868);
buffers that are not weights are let pass (crates/llm/src/weights.rs:716-721).
"""
from __future__ import annotations

import re
import sys
from dataclasses import dataclass
from typing import Iterable, Optional, Sequence

import torch

from .safetensors_io import Checkpoint

SPELLINGS = ("", "transformer.", "model.")


class WeightsError(ValueError):
    """The checkpoint does not hold the model the configuration describes."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=(), wrong_kind=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_kind = list(wrong_kind)


@dataclass(frozen=True)
class TensorRequest:
    name: str                       # the architecture's spelling, without a file-level prefix
    shape: tuple[int, ...]          # as stored in the checkpoint
    kind: str = "float"             # "float" or "int"
    optional: bool = False


def collapse(names: Iterable[str]) -> list[str]:
    """`h.0.x, h.1.x, ...` -> `h.*.x (N tensors)`; single names stay."""
    groups: dict[str, list[str]] = {}
    for n in sorted(names):
        groups.setdefault(re.sub(r"(?<![A-Za-z0-9_])\d+(?![A-Za-z0-9_])", "*", n), []).append(n)
    out = []
    for pattern, members in groups.items():
        out.append(members[0] if len(members) == 1 else f"{pattern} ({len(members)} tensors)")
    return out


class WeightSource:
    def __init__(self, checkpoint: Checkpoint, *, ignored_suffixes: Sequence[str] = (),
                 spellings: Sequence[str] = SPELLINGS):
        self.checkpoint = checkpoint
        self.spellings = tuple(spellings)
        self.ignored_suffixes = tuple(ignored_suffixes)
        self._resolved: dict[str, str] = {}
        self._skipped: set[str] = set()

    # -- names -----------------------------------------------------------------
    def resolve(self, name: str) -> Optional[str]:
        hit = self._resolved.get(name)
        if hit is not None:
            return hit
        for prefix in self.spellings:
            if prefix + name in self.checkpoint:
                self._resolved[name] = prefix + name
                return prefix + name
        return None

    def skip(self, name: str) -> None:
        """A tensor the model knows about and deliberately does not read."""
        stored = self.resolve(name)
        if stored is not None:
            self._skipped.add(stored)

    def has(self, name: str) -> bool:
        return self.resolve(name) is not None

    # -- the audit ---------------------------------------------------------------
    def check(self, requests: Sequence[TensorRequest]) -> None:
        missing, wrong_shape, wrong_kind = [], [], []
        asked: set[str] = set()
        for r in requests:
            stored = self.resolve(r.name)
            if stored is None:
                if not r.optional:
                    missing.append(r.name)
                continue
            asked.add(stored)
            e = self.checkpoint.entries[stored]
            if (r.kind == "float" and not e.is_float) or (r.kind == "int" and not e.is_int):
                wrong_kind.append((r.name, e.dtype, r.kind))
            if tuple(e.shape) != tuple(r.shape):
                wrong_shape.append((r.name, tuple(e.shape), tuple(r.shape)))
        unexpected = [
            n for n in self.checkpoint.names()
            if n not in asked and n not in self._skipped
            and not any(n.endswith(s) for s in self.ignored_suffixes)
        ]
        if not (missing or unexpected or wrong_shape or wrong_kind):
            return
        lines = ["the checkpoint does not match the configuration:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(collapse(missing)))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(collapse(unexpected)))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + ", ".join(
                f"{n} is {list(have)}, the configuration needs {list(want)}" for n, have, want in wrong_shape))
        if wrong_kind:
            lines.append(f"  wrong kind ({len(wrong_kind)}): " + ", ".join(
                f"{n} is stored as {have}, needs {want}" for n, have, want in wrong_kind))
        raise WeightsError("\n".join(lines), missing, unexpected, wrong_shape, wrong_kind)

    # -- reading -----------------------------------------------------------------
    def fetch(self, name: str, *, compute_dtype: torch.dtype, device, transpose: bool = False,
              keep_f32: bool = False) -> torch.Tensor:
        """Reads one tensor onto `device`.

        Floating tensors go to `compute_dtype`, except that with
        `keep_f32=True` a tensor stored in 32-bit stays in 32-bit whatever the
        compute dtype is (small vectors: gains, biases).  Integer tensors
        become int32.  `transpose` flips a 2-D tensor so that a projection
        stored `[in, out]` is held `[out, in]`.
        """
        stored = self.resolve(name)
        if stored is None:
            raise WeightsError(f"tensor `{name}` not found in checkpoint", missing=[name])
        e = self.checkpoint.entries[stored]
        t = self.checkpoint.read(stored)
        if e.is_int:
            t = t.to(torch.int32)
        elif e.is_float:
            if e.dtype == "F32" and (keep_f32 or compute_dtype == torch.float32):
                pass
            else:
                if e.dtype == "F32" and compute_dtype != torch.float32 and not getattr(self, "_told", False):
                    print(f"[kvad_b200] note: 32-bit matrices of this checkpoint are held in {compute_dtype} "
                          f"(first: {name})", file=sys.stderr)
                    self._told = True
                t = t.to(compute_dtype)
        if transpose:
            if t.dim() != 2:
                raise WeightsError(f"tensor `{name}` is rank {t.dim()}, cannot be transposed")
            t = t.t()
        return t.contiguous().to(device)
