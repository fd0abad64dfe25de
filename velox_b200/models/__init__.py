from . import buvuzen, dobepel, kapuvik, qwen3  # register the architectures
from .decoder import DecoderModel

__all__ = ["DecoderModel", "buvuzen", "dobepel", "kapuvik", "qwen3"]
