from .plan import DecoderModel, LayerPlan, ModelPlan, RunStep
from . import llama  # noqa: F401  (registers LlamaForCausalLM)
from . import sapanex  # noqa: F401  (registers Sapanex)

__all__ = ["DecoderModel", "LayerPlan", "ModelPlan", "RunStep"]
