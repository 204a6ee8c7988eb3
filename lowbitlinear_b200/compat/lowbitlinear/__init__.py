"""The reference's import name on top of this library.

Put this directory's parent (``lowbitlinear_b200/compat``) on ``PYTHONPATH`` and code written
against NanjinLin/LowBitLinear -- ``from lowbitlinear import QuantizedLinear``,
``lowbitlinear.quantization``, ``lowbitlinear.linear``, ``lowbitlinear._extension``
(lowbitlinear/__init__.py:1-4 of the reference) -- runs on the B200 kernels unchanged.  The
submodules are the very module objects of ``lowbitlinear_b200``, not copies, so patching one
patches the other.  With ``LOWBITLINEAR_REFERENCE_GEMM_POLICY=1`` in the environment the any-shape
operator also reproduces the reference GEMM's FP16-rounded-weight numerics on the shapes where
this library would otherwise keep the FP32 scale (``_ops.set_reference_gemm_policy``).
"""
import importlib
import os
import sys

from lowbitlinear_b200 import QuantizedLinear

for _name in ("_extension", "quantization", "linear"):
    _module = importlib.import_module("lowbitlinear_b200." + _name)
    sys.modules[__name__ + "." + _name] = _module
    globals()[_name] = _module
del _name, _module

if os.environ.get("LOWBITLINEAR_REFERENCE_GEMM_POLICY") == "1":
    from lowbitlinear_b200 import _ops as _ops_module

    _ops_module.set_reference_gemm_policy(True)
    del _ops_module

__all__ = ["QuantizedLinear"]
