from .batch import BatchBuilder, StepContext, StepEntry, Workspace
from .engine import InferenceEngine
from .request import Request, RequestState
from .runner import ModelRunner, decode_buckets
from .scheduler import Scheduler

__all__ = ["BatchBuilder", "StepContext", "StepEntry", "Workspace", "InferenceEngine", "Request",
           "RequestState", "ModelRunner", "decode_buckets", "Scheduler"]
