from . import burinex, dofipel, ganupel, llama, zemivik  # noqa: F401  (register LlamaForCausalLM, Zemivik, Dofipel, Ganupel, Burinex)
from .decoder import DecoderModel

__all__ = ["DecoderModel"]
