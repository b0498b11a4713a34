"""The engine: model, step function, scheduler, request-level interface, trace replay."""
from .batch import StepBatch, StepEntry
from .model import Model, declared_weights
from .runner import ModelRunner, StepError

__all__ = ["StepBatch", "StepEntry", "Model", "declared_weights", "ModelRunner", "StepError"]
from .llm_engine import LLMEngine  # noqa: E402
from .scheduler import RequestTooLarge, ScheduledPortion, Scheduler  # noqa: E402
from .sequence import Sequence, SequenceStatus  # noqa: E402

__all__ += ["LLMEngine", "RequestTooLarge", "ScheduledPortion", "Scheduler", "Sequence", "SequenceStatus"]
