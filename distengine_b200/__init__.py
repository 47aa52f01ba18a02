"""distengine_b200: a single-GPU inference engine for the Llama decoder on B200 (sm_100a).

    from distengine_b200 import Engine, EngineConfig, generate_greedy
"""

__version__ = "0.1.0"

from .config import EngineConfig, LlamaConfig  # noqa: E402
from .registry import register_architecture  # noqa: E402


def __getattr__(name):
    # the engine pulls in the kernels; load it on first use so that configuration, weights and
    # cache bookkeeping import without a GPU
    if name in ("Engine", "generate_greedy"):
        from .engine import engine as _engine
        return getattr(_engine, name)
    raise AttributeError(name)


__all__ = ["Engine", "EngineConfig", "LlamaConfig", "generate_greedy", "register_architecture"]
