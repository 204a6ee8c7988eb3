"""The reference's import name on top of this library.

Put this directory's parent (``lowbitlinear_b200/compat``) on ``PYTHONPATH`` and code written
against NanjinLin/LowBitLinear -- ``from lowbitlinear import QuantizedLinear``,
``lowbitlinear.quantization``, ``lowbitlinear.linear``, ``lowbitlinear._extension``
(lowbitlinear/__init__.py:1-4 of the reference) -- runs on the B200 kernels unchanged.  The
submodules are the very module objects of ``lowbitlinear_b200``, not copies, so patching one
patches the other.
"""
import importlib
import sys

from lowbitlinear_b200 import QuantizedLinear

for _name in ("_extension", "quantization", "linear"):
    _module = importlib.import_module("lowbitlinear_b200." + _name)
    sys.modules[__name__ + "." + _name] = _module
    globals()[_name] = _module
del _name, _module

__all__ = ["QuantizedLinear"]
