from .step import Engine, StepEntry

__all__ = ["Engine", "StepEntry"]
