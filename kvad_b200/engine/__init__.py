"""The engine: step function, generation loop, trace replay."""
from .batch import HostBatch, MetaLayout, StepEntry, pack
from .generate import Request, Stats, run_all, run_batch

__all__ = ["HostBatch", "MetaLayout", "StepEntry", "pack", "Request", "Stats", "run_all", "run_batch", "Engine"]


def __getattr__(name):
    if name == "Engine":
        from .engine import Engine
        return Engine
    raise AttributeError(name)
