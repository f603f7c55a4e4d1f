"""Models assembled from plans, and loading a model folder."""
from .model import Model, expected_tensors
from .loading import load_model, random_model

__all__ = ["Model", "expected_tensors", "load_model", "random_model"]
