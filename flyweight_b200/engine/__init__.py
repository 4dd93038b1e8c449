from .batch import Segment, StepBatch, StepContext
from .loading import load_model, parse_dtype, random_model
from .runner import ModelRunner, StepError

__all__ = ["Segment", "StepBatch", "StepContext", "load_model", "parse_dtype", "random_model",
           "ModelRunner", "StepError"]
