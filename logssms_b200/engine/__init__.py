from .step import Engine, StepEntry
from .scheduler import Request, Scheduler, StepDecision
from .llm import LLM, Output

__all__ = ["Engine", "StepEntry", "Request", "Scheduler", "StepDecision", "LLM", "Output"]
