from .batch import GroupBatch, StepBatch, StepEntry, build_step_batch
from .model import Model
from .runner import ModelRunner, StepError, resolve_dtype

__all__ = ["GroupBatch", "StepBatch", "StepEntry", "build_step_batch", "Model", "ModelRunner", "StepError",
           "resolve_dtype"]
