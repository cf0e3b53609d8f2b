from .context import GroupView, StepContext
from .factory import load_engine, make_engine, parse_dtype, random_engine
from .step import Engine, Entry, StepError

__all__ = ["GroupView", "StepContext", "load_engine", "make_engine", "parse_dtype",
           "random_engine", "Engine", "Entry", "StepError"]
