from .engine import Engine, OutOfPages, SamplingParams, StepEntry, StepError

__all__ = ["Engine", "OutOfPages", "SamplingParams", "StepEntry", "StepError"]
