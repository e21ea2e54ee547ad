"""Lookups in a config.json tree, with key aliases.

The same quantity has different names in different eras of config.json
(`n_layer` became `num_hidden_layers`), so every lookup takes a list of keys
and answers with the first that is present and of the right kind.  A key that
is present but `null` counts as absent, which is how a GPT-2 config with
`"n_inner": null` falls to its default.

Behaviour follows bisand/kvad's `Json` (crates/llm/src/model/mod.rs:226-296).
"""
from __future__ import annotations

import json
import os
from typing import Any, Iterable, Optional


class ConfigError(ValueError):
    """A config.json that cannot describe a model this library runs."""


class JsonView:
    def __init__(self, tree: dict):
        if not isinstance(tree, dict):
            raise ConfigError("config.json must hold a JSON object")
        self._tree = tree

    @classmethod
    def from_file(cls, path: str) -> "JsonView":
        with open(path, "r", encoding="utf-8") as f:
            return cls(json.load(f))

    @property
    def tree(self) -> dict:
        return self._tree

    def get(self, key: str) -> Any:
        return self._tree.get(key)

    def num(self, keys: Iterable[str]) -> Optional[int]:
        """First of `keys` that holds a non-negative whole number."""
        for k in keys:
            v = self._tree.get(k)
            if isinstance(v, bool):
                continue
            if isinstance(v, int) and v >= 0:
                return int(v)
        return None

    def float(self, keys: Iterable[str]) -> Optional[float]:
        for k in keys:
            v = self._tree.get(k)
            if isinstance(v, bool):
                continue
            if isinstance(v, (int, float)):
                return float(v)
        return None

    def flag(self, key: str) -> Optional[bool]:
        v = self._tree.get(key)
        return v if isinstance(v, bool) else None

    def text(self, key: str) -> Optional[str]:
        v = self._tree.get(key)
        return v if isinstance(v, str) else None

    def need(self, keys: Iterable[str], what: str) -> int:
        """A number the architecture cannot run without."""
        v = self.num(keys)
        if v is None:
            raise ConfigError(f"config: no {what}")
        return v

    def id_list(self, key: str) -> list[int]:
        """A token id or a list of them (`eos_token_id` is written both ways)."""
        v = self._tree.get(key)
        if isinstance(v, bool):
            return []
        if isinstance(v, int):
            return [v]
        if isinstance(v, list):
            return [int(x) for x in v if isinstance(x, int) and not isinstance(x, bool)]
        return []


def read_model_type(view: JsonView) -> str:
    """`model_type`, else the first of `architectures`, lower-cased
    (crates/llm/src/model/mod.rs:326-332)."""
    mt = view.text("model_type")
    if mt is None:
        archs = view.get("architectures")
        if isinstance(archs, list) and archs and isinstance(archs[0], str):
            mt = archs[0]
    if mt is None:
        raise ConfigError("config.json has neither model_type nor architectures")
    return mt.lower()


def config_path(model_dir: str) -> str:
    return os.path.join(model_dir, "config.json")
