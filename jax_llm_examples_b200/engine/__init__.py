from .engine import Engine, EngineError, StepEntry
from .generate import Generator, generate
from .scheduler import PlannedEntry, Request, Scheduler

__all__ = ["Engine", "EngineError", "Generator", "PlannedEntry", "Request", "Scheduler", "StepEntry", "generate"]
