from .config import ModelConfig
from .language import LanguageModel
from .sonulorn import Model

__all__ = ["Model", "ModelConfig", "LanguageModel"]
