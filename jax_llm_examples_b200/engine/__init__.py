from .engine import Engine, EngineError, StepEntry
from .generate import Batch, Generator, decode_step, generate, prefill
from .scheduler import PlannedEntry, Request, Scheduler

__all__ = ["Batch", "Engine", "EngineError", "Generator", "PlannedEntry", "Request", "Scheduler", "StepEntry", "decode_step",
           "generate", "prefill"]
