"""The engine: model, step function, scheduler, request-level interface, trace replay."""
from .batch import StepBatch, StepEntry
from .model import Model, declared_weights
from .runner import ModelRunner, StepError

__all__ = ["StepBatch", "StepEntry", "Model", "declared_weights", "ModelRunner", "StepError"]
