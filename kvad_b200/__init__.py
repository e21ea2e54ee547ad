"""kvad_b200: a small, whole GPT-2 inference library for one B200.

    from kvad_b200 import Engine
    engine = Engine.from_pretrained("model_dir", dtype="bfloat16")
    outputs = engine.generate([[5, 17, 3], [8, 1]], max_tokens=32, temperature=0)
"""
from .engine.batch import StepEntry
from .sampling.sampler import SamplingParams

__version__ = "0.1.0"
__all__ = ["Engine", "StepEntry", "SamplingParams", "write_random_model", "architectures"]


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    if name == "write_random_model":
        from .weights.random_init import write_random_model
        return write_random_model
    if name == "architectures":
        from .config import architectures
        from . import models  # noqa: F401
        return architectures
    raise AttributeError(name)
