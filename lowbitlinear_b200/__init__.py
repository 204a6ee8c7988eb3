"""B200-native W4A16 linear layer: group-64 asymmetric INT4 weights, FP16 activations.

Drop-in for the reference package's public surface (``lowbitlinear/__init__.py:1-4``):
importing loads the native library if it has been built, and ``QuantizedLinear`` is the one
exported class.  ``tensor_parallel`` adds the N-split / K-split sharding helpers.
"""
from . import _extension
from .linear import QuantizedLinear

__all__ = ["QuantizedLinear"]
