from . import buvuzen, dobepel, fovenex, kapuvik, qwen3  # register the architectures
from .decoder import DecoderModel

__all__ = ["DecoderModel", "buvuzen", "dobepel", "fovenex", "kapuvik", "qwen3"]
