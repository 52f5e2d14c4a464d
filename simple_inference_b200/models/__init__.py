from .plan import DecoderModel, LayerPlan, ModelPlan, RunStep
from . import llama  # noqa: F401  (registers LlamaForCausalLM)

__all__ = ["DecoderModel", "LayerPlan", "ModelPlan", "RunStep"]
