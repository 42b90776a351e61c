from .config import ModelConfig
from .language import LanguageModel
from .vadelix import Model

__all__ = ["Model", "ModelConfig", "LanguageModel"]
