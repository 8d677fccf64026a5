"""vosti_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a)."""
from . import config  # registers the built-in architecture

__version__ = "0.1.0"


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    raise AttributeError(name)
