"""Typed configuration and the architecture registry."""
from .json_view import ConfigError, JsonView, read_model_type
from .registry import (Architecture, architectures, by_id, from_model_type, register,
                       resolve, supported, unregister)


def load_config(model_dir: str):
    """(architecture, typed configuration) of a model folder."""
    import os

    view = JsonView.from_file(os.path.join(model_dir, "config.json"))
    # Registering the built-in architectures is a side effect of importing them.
    from .. import models  # noqa: F401

    arch = resolve(view)
    return arch, arch.read_config(view)


__all__ = [
    "Architecture", "ConfigError", "JsonView", "architectures", "by_id", "from_model_type",
    "load_config", "read_model_type", "register", "resolve", "supported", "unregister",
]
