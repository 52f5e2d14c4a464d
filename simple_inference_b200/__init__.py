"""A small, whole inference engine for Llama-family decoders on one NVIDIA B200.

From a model folder (``config.json`` + safetensors) to generated tokens: typed
configuration and architecture registry, weights by name, a model put together
from parts, a paged cache manager, one step function for mixed batches, a
continuous-batching scheduler, sampling, and hand-written sm_100a kernels.
"""

from .config import ConfigError, LlamaConfig, known_architectures, read_config, register_architecture
from .engine import InferenceEngine, ModelRunner, Request, RequestState, Scheduler, StepEntry
from .cache import CacheManager
from .models.load import load_model, random_model
from .sampling import SamplingParams
from .weights import WeightError, write_random_model

__all__ = ["ConfigError", "LlamaConfig", "known_architectures", "read_config",
           "register_architecture", "InferenceEngine", "ModelRunner", "Request", "RequestState",
           "Scheduler", "StepEntry", "CacheManager", "load_model", "random_model",
           "SamplingParams", "WeightError", "write_random_model"]
