from . import llama  # noqa: F401  (registers LlamaForCausalLM)
from .decoder import DecoderModel

__all__ = ["DecoderModel"]
