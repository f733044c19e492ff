from .decoder import DecoderModel

__all__ = ["DecoderModel"]
