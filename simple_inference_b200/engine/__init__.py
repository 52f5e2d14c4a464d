from .batch import BatchBuilder, StepContext, StepEntry, Workspace
from .runner import ModelRunner, decode_buckets

__all__ = ["BatchBuilder", "StepContext", "StepEntry", "Workspace", "ModelRunner", "decode_buckets"]
