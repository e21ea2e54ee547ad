"""One registry from an architecture's name to its model.

An `Architecture` is data: its id, the `model_type` strings it answers to, a
one-line description, a function that reads its typed configuration out of a
config.json, and the model class that is built from that configuration.  The
shape follows bisand/kvad's `Architecture` / `registry()`
(crates/llm/src/model/arch.rs:39-74, 134-206): matching is exact on a
normalised stem, and a `model_type` nobody claims is an error that lists what
this build runs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Optional

from .json_view import ConfigError, JsonView, read_model_type


@dataclass(frozen=True)
class Architecture:
    id: str
    model_types: tuple[str, ...]
    about: str
    #: JsonView -> typed configuration (a frozen dataclass)
    read_config: Callable[[JsonView], Any]
    #: typed configuration -> kvad_b200.models.plan.ModelPlan
    plan: Callable[[Any], Any]
    #: typed configuration -> dict for config.json (random-weights mode)
    write_config: Optional[Callable[[Any], dict]] = None
    #: (typed configuration, rng) -> {tensor name: (array, dtype name)} (random-weights mode)
    random_tensors: Optional[Callable[[Any, Any], dict]] = None


_REGISTRY: dict[str, Architecture] = {}


def _stem(model_type: str) -> str:
    """`GPT2LMHeadModel` and `gpt2` reduce to the same stem
    (crates/llm/src/model/arch.rs:134-153)."""
    s = model_type.lower()
    for suffix in ("forcausallm", "lmheadmodel", "model"):
        if s.endswith(suffix):
            s = s[: -len(suffix)]
            break
    return s.replace("_", "").replace("-", "")


def register(arch: Architecture, *, replace: bool = False) -> Architecture:
    """Adds an architecture.  Two architectures may not claim one model_type."""
    for other in _REGISTRY.values():
        if other.id == arch.id:
            continue
        clash = {_stem(t) for t in other.model_types} & {_stem(t) for t in arch.model_types}
        if clash:
            raise ValueError(f"architectures `{other.id}` and `{arch.id}` both claim {sorted(clash)}")
    if arch.id in _REGISTRY and not replace:
        raise ValueError(f"architecture `{arch.id}` is already registered")
    _REGISTRY[arch.id] = arch
    return arch


def unregister(arch_id: str) -> None:
    _REGISTRY.pop(arch_id, None)


def by_id(arch_id: str) -> Optional[Architecture]:
    return _REGISTRY.get(arch_id)


def from_model_type(model_type: str) -> Optional[Architecture]:
    stem = _stem(model_type)
    for arch in _REGISTRY.values():
        if any(_stem(t) == stem for t in arch.model_types):
            return arch
    return None


def architectures() -> list[Architecture]:
    return sorted(_REGISTRY.values(), key=lambda a: a.id)


def supported() -> str:
    return ", ".join(a.id for a in architectures())


def resolve(view: JsonView) -> Architecture:
    """The architecture a config.json names, or an error that lists what runs
    (crates/llm/src/model/mod.rs:334-336)."""
    model_type = read_model_type(view)
    arch = from_model_type(model_type)
    if arch is None:
        raise ConfigError(f"unsupported architecture `{model_type}`.\nThis build runs: {supported()}.")
    return arch
