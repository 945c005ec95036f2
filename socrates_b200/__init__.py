"""socrates_b200: a small, whole LLM inference engine for one B200 (sm_100a).

    from socrates_b200 import Engine
    engine = Engine("path/to/model_folder")
    req = engine.submit([1, 2, 3])
    engine.run()
    print(req.output)

The package imports without a GPU (configuration, weights, cache manager and
scheduler are host code); building an `Engine` needs CUDA and compiles the kernels at
first use.
"""

from .config import EngineConfig, Qwen3Config, load_config, register_architecture

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "Request", "QueueFull", "TooLong"):
        from .engine import engine as _e
        return getattr(_e, name)
    raise AttributeError(name)


__all__ = ["Engine", "EngineConfig", "Qwen3Config", "load_config", "register_architecture"]
