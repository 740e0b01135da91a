"""Models: the generic decoder and the loading of a model folder."""
from .decoder import DecoderModel, parameter_shapes
from .loading import load_model

__all__ = ["DecoderModel", "parameter_shapes", "load_model"]
