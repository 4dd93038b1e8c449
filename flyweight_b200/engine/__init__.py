from .batch import Segment, StepBatch, StepContext
from .loading import load_model, parse_dtype, random_model
from .runner import ModelRunner, StepError, StepPlanner
from .runtime import EngineConfig, GenerationResult, Model, Runtime
from .scheduler import (EVENT_ERROR, EVENT_FINISHED, EVENT_PROGRESS, EVENT_TOKEN, QueueFull,
                        Scheduler, Task)

__all__ = ["Segment", "StepBatch", "StepContext", "load_model", "parse_dtype", "random_model",
           "ModelRunner", "StepError", "StepPlanner", "EngineConfig", "GenerationResult", "Model", "Runtime",
           "EVENT_ERROR", "EVENT_FINISHED", "EVENT_PROGRESS", "EVENT_TOKEN", "QueueFull",
           "Scheduler", "Task"]
