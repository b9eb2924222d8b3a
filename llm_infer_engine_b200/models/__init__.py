from . import dofipel, ganupel, llama, zemivik  # noqa: F401  (register LlamaForCausalLM, Zemivik, Dofipel, Ganupel)
from .decoder import DecoderModel

__all__ = ["DecoderModel"]
