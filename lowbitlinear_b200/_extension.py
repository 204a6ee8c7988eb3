"""Finds and loads the native library once; importing never compiles anything.

Same contract as the reference's ``lowbitlinear/_extension.py:10-34``: exactly one ``_C*``
shared object beside the package is loaded through ``torch.ops.load_library``; a second
call is a no-op; ``required=True`` turns "no library" (or CPU-only PyTorch) into an
``ImportError`` that tells the user how to build; a broken library is never hidden.

What differs is the library itself: it is a plain C-ABI object (``include/lowbitlinear_b200.h``)
rather than a torch extension, so after loading it this module binds the entry points with
``ctypes`` and registers the reference's two operators
(``lowbitlinear_ext::w4a16_gemv_warp_vec`` and ``lowbitlinear_cute_w4a16::gemm``, CUDA
dispatch key only) on top of them -- see ``_ops.py``.
"""
import sys
import warnings
from importlib.machinery import EXTENSION_SUFFIXES
from pathlib import Path

import torch

_loaded_library = None
_native = None  # ctypes handle with typed entry points, set by load_cuda_extension


def _is_out_of_date():
    """True when this tree records a build whose sources differ from the present ones."""
    from ._fingerprint import recorded_build, source_fingerprint

    recorded = recorded_build()
    if recorded is None:
        return False
    fingerprint, flags, defines = recorded
    return source_fingerprint(flags, defines) != fingerprint


def _candidate_libraries():
    package_dir = Path(__file__).resolve().parent
    found = set()
    for suffix in EXTENSION_SUFFIXES:
        found.update(package_dir.glob(f"_C*{suffix}"))
    return sorted(found)


def load_cuda_extension(*, required=False):
    """Load the native library and register the operators.  Returns True when loaded."""
    global _loaded_library, _native
    if _loaded_library is not None:
        return True
    libraries = _candidate_libraries()
    if torch.version.cuda is None or not libraries:
        if required:
            raise ImportError(
                "lowbitlinear_b200 native CUDA library is unavailable. Use CUDA-enabled PyTorch "
                "and build it with: python -m lowbitlinear_b200.build  "
                "(the reference's equivalent is: python -m pip install -e . --no-build-isolation)"
            )
        return False
    if len(libraries) != 1:
        raise ImportError(f"Ambiguous lowbitlinear_b200 native libraries: {libraries}")
    path = libraries[0]
    if _is_out_of_date():
        # Checked before the loader touches the file: a library that was loaded once stays
        # mapped for the life of the process, even after a rebuild.
        message = (f"{path} was built from older sources; rebuild it with: "
                   "python -m lowbitlinear_b200.build")
        if required:
            raise ImportError(message)
        if "lowbitlinear_b200.build" not in getattr(sys, "orig_argv", ()):  # not while rebuilding
            warnings.warn(message, RuntimeWarning, stacklevel=2)
        return False
    # Errors from the dynamic loader propagate: a CUDA installation with a broken library
    # must fail loudly.
    torch.ops.load_library(str(path))
    from . import _ops

    _native = _ops.bind(str(path))
    _ops.register_operators(_native)
    _loaded_library = path
    return True


def native():
    """The bound C-ABI library (loads it on first use; ImportError if it is missing)."""
    load_cuda_extension(required=True)
    return _native


load_cuda_extension()
