from .batch import StepContext, StepEntry, attention_work_arrays
from .runner import ModelRunner, build_model

__all__ = ["StepContext", "StepEntry", "attention_work_arrays", "ModelRunner", "build_model"]
