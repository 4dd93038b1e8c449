from . import lfm2  # noqa: F401  (registers the architecture)
from .lfm2 import Lfm2ForCausalLM

__all__ = ["Lfm2ForCausalLM"]
