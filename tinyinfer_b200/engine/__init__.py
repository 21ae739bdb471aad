from .batch import BatchBuffers, CacheView, StepContext, StepEntry
from .loading import build_random_model, load_model
from .replay import TraceSession
from .runner import ModelRunner

__all__ = ["BatchBuffers", "CacheView", "StepContext", "StepEntry", "build_random_model",
           "load_model", "TraceSession", "ModelRunner"]
