"""Architectures.  Importing this package registers them."""
from . import qwen2  # noqa: F401
from .model import Model, compute_dtype, load_model, random_model_on_device, weight_specs_of

__all__ = ["Model", "compute_dtype", "load_model", "random_model_on_device", "weight_specs_of"]
