from . import diforax, kemitar, lfm2  # noqa: F401  (register the architectures)
from .diforax import DiforaxForCausalLM
from .kemitar import KemitarForCausalLM
from .lfm2 import Lfm2ForCausalLM

__all__ = ["DiforaxForCausalLM", "KemitarForCausalLM", "Lfm2ForCausalLM"]
