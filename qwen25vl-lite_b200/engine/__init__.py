"""The step function, the scheduler above it, the Python entry point and trace replay."""

from .llm import LLM  # noqa: F401
from .runner import ModelRunner, Request, StepContext, StepEntry  # noqa: F401
from .scheduler import EngineStats, LLMEngine, RequestOutput, Sequence  # noqa: F401
