from .batch import StepBatch, StepEntry, build_batch
from .runner import ModelRunner, load_model, random_model, resolve_dtype

__all__ = ["ModelRunner", "StepBatch", "StepEntry", "build_batch", "load_model", "random_model", "resolve_dtype"]
