from . import kemitar, lfm2  # noqa: F401  (register the architectures)
from .kemitar import KemitarForCausalLM
from .lfm2 import Lfm2ForCausalLM

__all__ = ["KemitarForCausalLM", "Lfm2ForCausalLM"]
