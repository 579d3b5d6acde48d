from .decoder import DecoderModel, load_model

__all__ = ["DecoderModel", "load_model"]
