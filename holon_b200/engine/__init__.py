"""The step function, the scheduler above it, and the engine a user calls."""
from ..config.engine import EngineConfig
from ..sampling.params import SamplingParams
from .batch import StepEntry
from .build import Built, build
from .engine import Engine, Logprobs, TokenDelta
from .runner import Runner, StepError
from .scheduler import Request, Scheduler

__all__ = ["Built", "Engine", "EngineConfig", "Request", "Runner", "SamplingParams", "Scheduler", "StepEntry",
           "StepError", "TokenDelta", "Logprobs", "build"]
