from .buzopel import Model
from .config import ModelConfig
from .language import LanguageModel

__all__ = ["Model", "ModelConfig", "LanguageModel"]
