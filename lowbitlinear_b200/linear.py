"""W4A16 linear layer: public module, forward dispatch and the FP32 reference path.

Mirrors the reference's ``lowbitlinear/linear.py``:

* ``QuantizedLinear(packed_weight, scales, zeros, group_size=64, *, in_features)`` keeps
  exactly three buffers (``packed_weight`` INT32 ``[N, ceil(K/8)]``, ``scales`` FP32 and
  ``zeros`` INT32 ``[N, ceil(K/group_size)]``); reference ``linear.py:76-84``.
* ``QuantizedLinear.from_float(weight, bits=4, group_size=64)``; reference ``linear.py:86-93``.
* ``forward(x)`` re-validates state and input on every call and dispatches
  (reference ``linear.py:95-129``): CUDA tensors with ``group_size == 64`` always run a
  hand-written sm_100a kernel through one of the two registered operators -- the M = 1
  operator when ``K % 64 == 0`` and ``N % 128 == 0``, the any-shape operator otherwise;
  a missing native library is an ``ImportError``, never a silent fallback.  CPU tensors and
  other group sizes take ``linear_int4_reference``.
* ``linear_int4_reference`` unpacks, dequantises to FP32, multiplies in FP32 and rounds to
  FP16; reference ``linear.py:43-70``.  It is the semantics every kernel is checked against.

Which kernel runs inside each operator (streaming GEMV, split-K GEMV, tcgen05 GEMM or the
masked any-shape kernel) is decided by size inside the native library.
"""
import torch

from ._extension import load_cuda_extension
from .quantization import (
    _validate_matrix,
    _validate_metadata,
    dequantize_int4,
    quantize_pack_int4,
    unpack_int4,
)


def _validate_packed_weight(packed_weight, scales, zeros, group_size, in_features):
    """State checks in the reference's order (``linear.py:10-33``)."""
    _validate_matrix(packed_weight, "packed_weight", (torch.int32,))
    if isinstance(in_features, bool) or not isinstance(in_features, int) or in_features <= 0:
        raise ValueError("in_features must be a positive integer")
    rows, words = packed_weight.shape
    if words != (in_features + 7) // 8:
        raise ValueError("Invalid packed_weight shape")
    _validate_metadata(scales, zeros, rows, in_features, group_size, packed_weight.device)


def _validate_input(x, packed_weight, in_features):
    """Activation checks (``linear.py:35-40``): FP16, nonempty 2-D, matching K and device."""
    _validate_matrix(x, "x", (torch.float16,))
    if x.shape[1] != in_features:
        raise ValueError("x and packed_weight have incompatible K")
    if x.device != packed_weight.device:
        raise ValueError("All tensors must be on the same device")


def linear_int4_reference(x, packed_weight, scales, zeros, group_size=64):
    """``fp16(x.float() @ dequant(packed).T)`` with FP32 dequantisation and accumulation.

    ``x`` is ``[M, K]`` FP16.  A caller that wants an IEEE FP32 answer on a GPU must switch
    TF32 matmul off.
    """
    _validate_matrix(x, "x", (torch.float16,))
    k = x.shape[1]
    _validate_packed_weight(packed_weight, scales, zeros, group_size, k)
    _validate_input(x, packed_weight, k)
    levels = unpack_int4(packed_weight, original_k=k)
    weight = dequantize_int4(levels, scales, zeros, group_size)
    return (x.float() @ weight.T).to(torch.float16)


class QuantizedLinear(torch.nn.Module):
    """Inference-only linear layer with group-wise asymmetric INT4 weights and FP16 input."""

    def __init__(self, packed_weight, scales, zeros, group_size=64, *, in_features):
        super().__init__()
        _validate_packed_weight(packed_weight, scales, zeros, group_size, in_features)
        self.group_size = group_size
        self.in_features = in_features
        self.out_features = packed_weight.shape[0]
        self.register_buffer("packed_weight", packed_weight)
        self.register_buffer("scales", scales)
        self.register_buffer("zeros", zeros)

    @classmethod
    def from_float(cls, weight, bits=4, group_size=64):
        if isinstance(bits, bool) or bits != 4:
            raise ValueError("Only bits=4 is supported")
        with torch.no_grad():
            packed, scales, zeros = quantize_pack_int4(weight, group_size)
        return cls(packed, scales, zeros, group_size, in_features=weight.shape[1])

    def _state_key(self, packed_weight, scales, zeros):
        """Everything ``_validate_packed_weight`` looks at: types, shapes, dtypes, devices and the
        two integers.  Equal keys mean an equal verdict, so a key that passed once need not be
        checked again; replacing or reshaping a buffer changes the key."""
        return (
            type(packed_weight), packed_weight.shape, packed_weight.dtype, packed_weight.device,
            type(scales), scales.shape, scales.dtype, scales.device,
            type(zeros), zeros.shape, zeros.dtype, zeros.device,
            type(self.group_size), self.group_size, type(self.in_features), self.in_features,
        )

    def forward(self, x):
        packed_weight, scales, zeros = self.packed_weight, self.scales, self.zeros
        # The reference validates the stored state on every call (``linear.py:96-99``), which
        # costs more host time than a decode kernel runs.  Same checks, same errors, but a state
        # that has passed is recognised by its key.
        try:
            key = self._state_key(packed_weight, scales, zeros)
        except AttributeError:  # a buffer was replaced by something that is not a tensor
            key = None
        if key is None or key != self.__dict__.get("_validated_key"):
            _validate_packed_weight(packed_weight, scales, zeros, self.group_size, self.in_features)
            self.__dict__["_validated_key"] = key
        _validate_input(x, packed_weight, self.in_features)
        if not x.is_contiguous():
            raise ValueError("CUDA input x must be contiguous")
        if not (x.is_cuda and self.group_size == 64):
            return linear_int4_reference(x, packed_weight, scales, zeros, self.group_size)
        load_cuda_extension(required=True)
        decode_shape = (
            x.shape[0] == 1 and self.in_features % 64 == 0 and self.out_features % 128 == 0
        )
        if decode_shape:
            return torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(
                x, packed_weight, scales, zeros, self.group_size
            )
        return torch.ops.lowbitlinear_cute_w4a16.gemm(x, packed_weight, scales, zeros)
