from .model import LayerCall, Model
from . import llama  # registers LlamaForCausalLM

__all__ = ["LayerCall", "Model", "llama"]
