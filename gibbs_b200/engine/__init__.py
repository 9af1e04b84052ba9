from .step import Engine, StepEntry, StepError, StepState
from .loading import load_model, random_model, parse_dtype

__all__ = ["Engine", "StepEntry", "StepError", "StepState", "load_model", "random_model", "parse_dtype"]
