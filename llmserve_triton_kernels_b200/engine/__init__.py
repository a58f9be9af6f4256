from .batch import StepContext, StepEntry  # noqa: F401
from .llm import LLM, RequestOutput  # noqa: F401
from .scheduler import EngineStats, Request, Scheduler, Status, TokenEvent  # noqa: F401
from .step import StepFunction  # noqa: F401
