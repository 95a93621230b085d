"""A small, whole inference engine for one NVIDIA B200: Qwen3 dense decoders from a model folder to tokens."""
__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "EngineConfig", "SamplingParams"):
        from . import engine as _engine
        return getattr(_engine, name)
    raise AttributeError(name)
