from .config import ModelConfig
from .language import LanguageModel
from .lilosun import Model

__all__ = ["Model", "ModelConfig", "LanguageModel"]
