from .step import Engine, StepEntry, StepError, StepState
from .loading import load_model, random_model, parse_dtype
from .scheduler import FinishReason, Scheduler, StepOutput
from .api import Generator

__all__ = ["Engine", "StepEntry", "StepError", "StepState", "load_model", "random_model", "parse_dtype",
           "FinishReason", "Scheduler", "StepOutput", "Generator"]
