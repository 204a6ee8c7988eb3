"""Group-wise asymmetric INT4 storage format (pure torch, CPU or CUDA tensors).

This module defines the bit-exact contract every kernel of the library consumes:

* ``quantize_int4``   -- per row and per ``group_size`` columns: the value range is widened
  to contain 0, ``scale = (hi - lo) / 15`` (1 for an all-zero group),
  ``zero = clamp(round(-lo / scale), 0, 15)`` and
  ``q = clamp(round(w / scale + zero), 0, 15)`` with round-half-even, all in FP32.
  Follows the reference ``lowbitlinear/quantization.py:33-86``.
* ``pack_int4``       -- eight unsigned nibbles per INT32 word, nibble ``i`` of word ``j`` is
  column ``8 j + i`` (low nibble first); the last word is zero padded and a top nibble of 8
  or more yields a negative word.  Reference ``lowbitlinear/quantization.py:112-141``.
* ``unpack_int4``     -- the inverse, cropping to ``original_k``.
  Reference ``lowbitlinear/quantization.py:143-171``.
* ``dequantize_int4`` -- ``w = (q - zero) * scale`` in FP32.
  Reference ``lowbitlinear/quantization.py:88-110``.

The reference walks the groups in a Python loop; here every function is a handful of
whole-tensor operations (a zero-padded ``[N, groups, group_size]`` view for the quantiser, a
byte view for the packer).  Every elementwise operation and its operand order is the same as
the reference's, so results are bit-identical to it on the same device: zero padding cannot
change a group's clamped minimum or maximum, and packing is pure integer work.
"""
import torch

_ROW_CHUNK_ELEMENTS = 1 << 24  # bounds the FP32 temporaries of quantize/dequantize (64 MiB each)


def _validate_matrix(tensor, name, dtypes):
    """Type, dtype, rank/emptiness and device checks shared by the whole package.

    Same exception types and message fragments as the reference
    (``lowbitlinear/quantization.py:4-12``): callers match on "Tensor", "dtype",
    "nonempty 2D" and "CPU or CUDA".
    """
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a Tensor")
    if tensor.dtype not in dtypes:
        raise TypeError(f"{name} has unsupported dtype {tensor.dtype}")
    if tensor.ndim != 2 or tensor.shape[0] <= 0 or tensor.shape[1] <= 0:
        raise ValueError(f"{name} must be a nonempty 2D tensor")
    if tensor.device.type != "cpu" and tensor.device.type != "cuda":
        raise ValueError(f"{name} must be on CPU or CUDA")


def _validate_group_size(k, group_size):
    """``group_size`` is a positive int and not a bool (reference ``quantization.py:15-21``)."""
    if isinstance(group_size, bool) or not isinstance(group_size, int) or group_size <= 0:
        raise ValueError("group_size must be a positive integer")


def _validate_metadata(scales, zeros, n, k, group_size, device):
    """Scales FP32 and zero points INT32, both ``[n, ceil(k / group_size)]`` on ``device``.

    Check order follows the reference (``quantization.py:24-31``): group size, dtypes and
    rank, shape, then device.
    """
    _validate_group_size(k, group_size)
    _validate_matrix(scales, "scales", (torch.float32,))
    _validate_matrix(zeros, "zeros", (torch.int32,))
    groups = -(-k // group_size)
    if tuple(scales.shape) != (n, groups) or zeros.shape != scales.shape:
        raise ValueError("Invalid scales or zeros shape")
    if scales.device != device or zeros.device != device:
        raise ValueError("All tensors must be on the same device")


def _row_chunks(n, k):
    rows = max(1, _ROW_CHUNK_ELEMENTS // max(k, 1))
    for start in range(0, n, rows):
        yield start, min(n, start + rows)


def quantize_int4(weight, group_size=64):
    """Quantise ``weight`` ``[N, K]`` (FP16 or FP32) group-wise along K.

    Returns ``(q [N, K] uint8, scales [N, G] float32, zeros [N, G] int32)`` with
    ``G = ceil(K / group_size)``; the last group may be shorter than ``group_size``.
    """
    _validate_matrix(weight, "weight", (torch.float16, torch.float32))
    n, k = weight.shape
    _validate_group_size(k, group_size)
    groups = -(-k // group_size)
    tail = groups * group_size - k

    q = torch.empty((n, k), dtype=torch.uint8, device=weight.device)
    scales = torch.empty((n, groups), dtype=torch.float32, device=weight.device)
    zeros = torch.empty((n, groups), dtype=torch.int32, device=weight.device)
    for r0, r1 in _row_chunks(n, k):
        block = weight[r0:r1].float()
        if tail:
            # Zeros never move a minimum clamped to <= 0 or a maximum clamped to >= 0.
            block = torch.nn.functional.pad(block, (0, tail))
        block = block.reshape(r1 - r0, groups, group_size)
        lo = block.amin(dim=-1).clamp(max=0)
        hi = block.amax(dim=-1).clamp(min=0)
        step = (hi - lo) / 15.0
        step = torch.where(step > 0, step, torch.ones_like(step))
        zero = torch.round(-lo / step).clamp(0, 15).to(torch.int32)
        level = torch.round(block / step.unsqueeze(-1) + zero.unsqueeze(-1)).clamp(0, 15)
        q[r0:r1] = level.to(torch.uint8).reshape(r1 - r0, groups * group_size)[:, :k]
        scales[r0:r1] = step
        zeros[r0:r1] = zero
    return q, scales, zeros


def quantize_pack_int4(weight, group_size=64):
    """``quantize_int4`` followed by ``pack_int4``: ``(packed [N, ceil(K/8)] int32, scales, zeros)``.

    A CUDA weight with ``group_size == 64`` goes through the library's one-pass quantiser kernel
    when the native library is built; its results are bit-identical to this module's CPU
    arithmetic (the torch CUDA ops may differ from the CPU in the last bit of a scale).  Every
    other case runs the two torch functions.
    """
    _validate_matrix(weight, "weight", (torch.float16, torch.float32))
    _validate_group_size(weight.shape[1], group_size)
    if weight.is_cuda and group_size == 64:
        from ._extension import load_cuda_extension

        if load_cuda_extension(required=False):
            from . import _ops

            return _ops.quantize_pack(weight, group_size)
    levels, scales, zeros = quantize_int4(weight, group_size)
    return pack_int4(levels), scales, zeros


def dequantize_int4(qweight, scales, zeros, group_size=64):
    """``(q - zero) * scale`` per group, FP32 ``[N, K]``."""
    _validate_matrix(qweight, "qweight", (torch.uint8,))
    n, k = qweight.shape
    _validate_metadata(scales, zeros, n, k, group_size, qweight.device)
    column_group = torch.arange(k, device=qweight.device) // group_size
    out = torch.empty((n, k), dtype=torch.float32, device=qweight.device)
    for r0, r1 in _row_chunks(n, k):
        zero = zeros[r0:r1].float().index_select(1, column_group)
        scale = scales[r0:r1].index_select(1, column_group)
        out[r0:r1] = (qweight[r0:r1].float() - zero) * scale
    return out


def pack_int4(qweight):
    """Pack ``[N, K]`` uint8 levels (0..15) into ``[N, ceil(K / 8)]`` INT32 words.

    Two nibbles make a byte (even column in the low half) and four bytes make a word in
    little-endian order, which puts column ``8 j + i`` at bits ``4 i .. 4 i + 3`` of word
    ``j`` exactly as the reference's shift-and-or loop does.
    """
    _validate_matrix(qweight, "qweight", (torch.uint8,))
    n, k = qweight.shape
    if bool((qweight > 15).any()):
        raise ValueError("qweight values must be in [0, 15]")
    words = (k + 7) // 8
    if words * 8 != k:
        qweight = torch.nn.functional.pad(qweight, (0, words * 8 - k), value=0)
    pairs = qweight.reshape(n, words * 4, 2)
    packed_bytes = (pairs[..., 0] | (pairs[..., 1] << 4)).contiguous()
    return packed_bytes.view(torch.int32)


def unpack_int4(packed, original_k=None):
    """Unpack ``[N, W]`` INT32 words into ``[N, 8 W]`` uint8 levels, cropped to ``original_k``."""
    _validate_matrix(packed, "packed", (torch.int32,))
    n, words = packed.shape
    as_bytes = packed.contiguous().view(torch.uint8)
    levels = torch.stack((as_bytes & 0xF, as_bytes >> 4), dim=-1).reshape(n, words * 8)
    if original_k is None:
        return levels
    if (
        isinstance(original_k, bool)
        or not isinstance(original_k, int)
        or original_k <= 0
        or (original_k + 7) // 8 != words
    ):
        raise ValueError("Invalid original_k")
    return levels[:, :original_k]
