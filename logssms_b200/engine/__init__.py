from .plan import StepEntry, StepPlanner
from .step import Engine
from .scheduler import Request, Scheduler, StepDecision
from .llm import LLM, Output

__all__ = ["Engine", "StepEntry", "StepPlanner", "Request", "Scheduler", "StepDecision", "LLM", "Output"]
