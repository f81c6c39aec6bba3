from . import bizetar, llama, sebilorn, vapelix, vomotar  # noqa: F401  (register the architectures)
from .decoder import DecoderModel, expected_tensors
from .loading import load_model

__all__ = ["DecoderModel", "expected_tensors", "load_model"]
