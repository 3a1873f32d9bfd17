from .runner import ModelRunner, StepEntry

__all__ = ["ModelRunner", "StepEntry"]
