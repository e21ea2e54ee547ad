"""Architectures this build runs.  Importing a module registers it."""
from .plan import LayerCall, Model, ModelPlan
from . import gpt2  # noqa: F401

__all__ = ["LayerCall", "Model", "ModelPlan", "gpt2"]
