from .engine import PREVIOUS, Engine, OutOfPages, SamplingParams, StepEntry, StepError

__all__ = ["PREVIOUS", "Engine", "OutOfPages", "SamplingParams", "StepEntry", "StepError"]
