from .runner import ModelRunner, StepEntry, StepError

__all__ = ["ModelRunner", "StepEntry", "StepError"]
