"""ctypes binding of the C ABI and the two torch operators built on it.

The reference registers its operators from C++ (``csrc/w4a16_gemv_warp_vec.cu:197-207``,
``csrc/cute_w4a16_gemm.cu:250-257``) and checks its arguments with ``TORCH_CHECK``
(``w4a16_gemv_warp_vec.cu:118-165``, ``cute_w4a16_gemm.cu:196-223``).  Here the same schemas
are registered with ``torch.library`` for the CUDA dispatch key only, the same checks run in
the same order and raise ``RuntimeError`` with the same key phrases, the output is allocated
by torch, and the work is one call into the C ABI on the caller's current stream.  CPU
tensors never reach this code: the dispatcher raises ``NotImplementedError`` for them, as it
does for the reference.
"""
import ctypes
import threading

import torch

PATH_AUTO, PATH_GENERIC, PATH_GEMV, PATH_GEMV_SPLITK, PATH_GEMM_TC, PATH_GEMM_TC_SMALL, PATH_GEMM_WT, PATH_GEMM_TC_PAIR = range(8)
PATH_NAMES = {
    PATH_AUTO: "auto",
    PATH_GENERIC: "generic",
    PATH_GEMV: "gemv",
    PATH_GEMV_SPLITK: "gemv_splitk",
    PATH_GEMM_TC: "gemm_tc",
    PATH_GEMM_TC_SMALL: "gemm_tc_small",
    PATH_GEMM_WT: "gemm_wt",
    PATH_GEMM_TC_PAIR: "gemm_tc_pair",
}
FLAG_PDL = 1
FLAG_ROUND_WEIGHTS = 2
FLAG_INDEPENDENT = 4

GEMV_SCHEMA = (
    "w4a16_gemv_warp_vec(Tensor x, Tensor packed_w, Tensor scales, Tensor zeros, "
    "int group_size) -> Tensor"
)
GEMM_SCHEMA = "gemm(Tensor X, Tensor packed_w, Tensor scales, Tensor zeros) -> Tensor"



class GroupProblem(ctypes.Structure):
    """``lbl_w4a16_problem`` of the C ABI."""
    _fields_ = [("x", ctypes.c_void_p), ("packed_w", ctypes.c_void_p), ("scales", ctypes.c_void_p),
                ("zeros", ctypes.c_void_p), ("y", ctypes.c_void_p), ("M", ctypes.c_int64),
                ("N", ctypes.c_int64), ("K", ctypes.c_int64), ("reduce", ctypes.c_int32),
                ("reserved", ctypes.c_int32)]


_lib = None
_registered = []  # keeps the torch.library.Library objects alive
ERR_WORKSPACE = -3  # LBL_ERR_WORKSPACE
_flags = 0
_workspaces = {}
_workspace_lock = threading.Lock()


def bind(path):
    """Open the shared object and declare every entry point of ``lowbitlinear_b200.h``."""
    global _lib
    lib = ctypes.CDLL(path)
    p, i64, i32, u32, sz = (ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_uint,
                            ctypes.c_size_t)
    lib.lbl_version.restype = i32
    lib.lbl_version.argtypes = []
    lib.lbl_last_error.restype = ctypes.c_char_p
    lib.lbl_last_error.argtypes = []
    lib.lbl_w4a16_select_path.restype = i32
    lib.lbl_w4a16_select_path.argtypes = [i64, i64, i64, i32]
    lib.lbl_w4a16_workspace_bytes.restype = sz
    lib.lbl_w4a16_workspace_bytes.argtypes = [i64, i64, i64, i32]
    lib.lbl_w4a16_workspace_init.restype = i32
    lib.lbl_w4a16_workspace_init.argtypes = [p, sz, i32, p]
    lib.lbl_w4a16_gemv.restype = i32
    lib.lbl_w4a16_gemv.argtypes = [p, p, p, p, p, i64, i64, i32, p, sz, u32, i32, p]
    lib.lbl_w4a16_gemm.restype = i32
    lib.lbl_w4a16_gemm.argtypes = [p, p, p, p, p, i64, i64, i64, p, sz, u32, i32, p]
    lib.lbl_w4a16_linear.restype = i32
    lib.lbl_w4a16_linear.argtypes = [p, p, p, p, p, i64, i64, i64, i32, i32, p, sz, u32, i32, p,
                                     ctypes.POINTER(ctypes.c_int)]
    lib.lbl_device_status.restype = i32
    lib.lbl_device_status.argtypes = [i32, ctypes.POINTER(ctypes.c_int)]
    lib.lbl_peer_buffer_bytes.restype = sz
    lib.lbl_peer_buffer_bytes.argtypes = [i64]
    lib.lbl_peer_buffer_create.restype = i32
    lib.lbl_peer_buffer_create.argtypes = [sz, i32, ctypes.POINTER(p)]
    lib.lbl_peer_buffer_export.restype = i32
    lib.lbl_peer_buffer_export.argtypes = [p, p]
    lib.lbl_peer_buffer_peek.restype = i32
    lib.lbl_peer_buffer_peek.argtypes = [p, sz, p, sz, i32]
    lib.lbl_peer_buffer_open.restype = i32
    lib.lbl_peer_buffer_open.argtypes = [p, i32, ctypes.POINTER(p)]
    lib.lbl_peer_buffer_close.restype = i32
    lib.lbl_peer_buffer_close.argtypes = [p, i32]
    lib.lbl_peer_buffer_destroy.restype = i32
    lib.lbl_peer_buffer_destroy.argtypes = [p, i32]
    lib.lbl_w4a16_gemv_allreduce.restype = i32
    lib.lbl_w4a16_gemv_allreduce.argtypes = [p, p, p, p, p, i64, i64, i32, i32, i32, ctypes.POINTER(p), i64,
                                             p, sz, u32, i32, p]
    lib.lbl_peer_gemm_buffer_bytes.restype = sz
    lib.lbl_peer_gemm_buffer_bytes.argtypes = [i64, i64, i32]
    lib.lbl_w4a16_gemm_scatter.restype = i32
    lib.lbl_w4a16_gemm_scatter.argtypes = [p, p, p, p, i64, i64, i64, i32, i32, ctypes.POINTER(p), sz, u32, i32, p]
    lib.lbl_peer_gemm_allreduce_finish.restype = i32
    lib.lbl_peer_gemm_allreduce_finish.argtypes = [p, i64, i64, i32, i32, ctypes.POINTER(p), sz, i32, p]
    lib.lbl_w4a16_gemm_allreduce.restype = i32
    lib.lbl_w4a16_gemm_allreduce.argtypes = [p, p, p, p, p, i64, i64, i64, i32, i32, ctypes.POINTER(p), sz, u32,
                                             i32, p]
    lib.lbl_w4a16_quantize.restype = i32
    lib.lbl_w4a16_quantize.argtypes = [p, i32, i64, i64, i32, p, p, p, i32, p]
    lib.lbl_w4a16_dequantize.restype = i32
    lib.lbl_w4a16_dequantize.argtypes = [p, p, p, p, i32, i64, i64, i32, i32, p]
    lib.lbl_w4a16_group_create.restype = i32
    lib.lbl_w4a16_group_create.argtypes = [ctypes.POINTER(GroupProblem), i32, i32, i32, ctypes.POINTER(p), i64, i32,
                                           ctypes.POINTER(p)]
    lib.lbl_w4a16_group_run.restype = i32
    lib.lbl_w4a16_group_run.argtypes = [p, u32, p]
    lib.lbl_w4a16_group_algorithmic_bytes.restype = i64
    lib.lbl_w4a16_group_algorithmic_bytes.argtypes = [p]
    lib.lbl_w4a16_group_destroy.restype = i32
    lib.lbl_w4a16_group_destroy.argtypes = [p]
    lib.lbl_w4a16_gemv_noalloc.restype = i32
    lib.lbl_w4a16_gemv_noalloc.argtypes = [p, p, p, p, p, i64, i64, i32, u32, i32, p]
    lib.lbl_w4a16_gemv_noalloc_scratch_bytes.restype = sz
    lib.lbl_w4a16_gemv_noalloc_scratch_bytes.argtypes = []
    _lib = lib
    return lib


def set_programmatic_dependent_launch(enabled):
    """Let consecutive decode kernels overlap: a kernel starts fetching its weights while the
    previous kernel in the stream is still finishing, and only its activation read waits.

    Safe whenever the kernel that precedes a linear in the stream does not write that linear's
    weights -- true for inference, where weights are written once.  Off by default."""
    global _flags
    _flags = (_flags | FLAG_PDL) if enabled else (_flags & ~FLAG_PDL)


def set_independent_launches(enabled):
    """Together with programmatic dependent launch: declare that consecutive calls are independent
    of each other (no call reads what the previous one writes, nor writes what it reads or writes).
    The large tensor-core GEMMs then do not wait for the previous kernel at all, and their CTAs
    start on the SMs that its last, partial wave leaves idle.  Off by default."""
    global _flags
    _flags = (_flags | FLAG_INDEPENDENT) if enabled else (_flags & ~FLAG_INDEPENDENT)


def set_reference_gemm_policy(enabled):
    """Make the any-shape operator round every dequantised weight to FP16 before the product on
    ALL shapes, as the reference GEMM does (``csrc/cute_w4a16_gemm.cu:160-162``).  By default the
    shapes it hands to the streaming kernels (M <= 8, M <= 16 when N >= 16384, or M <= 32 with a
    ragged N; K % 256 == 0)
    keep the FP32 scale, which is closer to the FP32 reference path but differs from the
    reference GEMM's own outputs by up to an FP16 step; with this switch those shapes run a
    tensor-core or the masked kernel instead (slower)."""
    global _flags
    _flags = (_flags | FLAG_ROUND_WEIGHTS) if enabled else (_flags & ~FLAG_ROUND_WEIGHTS)


def _raw_stream(device):
    """Handle of the current stream of ``device`` (what ``torch.cuda.current_stream(device)
    .cuda_stream`` returns, without building the Python stream object)."""
    return torch._C._cuda_getCurrentRawStream(device.index)


def _check(rc):
    if rc != 0:
        raise RuntimeError(_lib.lbl_last_error().decode() or f"lowbitlinear_b200 error {rc}")


def _workspace(device, stream, m, n, k, path=PATH_AUTO, exact=False):
    """Scratch for split-K, cached per (device, stream): zeroed when created, and every kernel
    leaves its counters zero again.  Returns ``(pointer, bytes)``.

    The usual call hands out the cached buffer without asking the library how much this problem
    needs (1 MiB covers the common shapes); ``exact=True`` asks, and grows the buffer if needed."""
    key = (device.index, stream)
    entry = _workspaces.get(key)
    if entry is not None and not exact:
        return entry[1], entry[2]
    need = max(_lib.lbl_w4a16_workspace_bytes(m, n, k, path), 1 << 20)
    with _workspace_lock:
        entry = _workspaces.get(key)
        if entry is None or entry[2] < need:
            buf = torch.zeros(need, dtype=torch.uint8, device=device)
            entry = (buf, buf.data_ptr(), need)
            _workspaces[key] = entry
    return entry[1], entry[2]


def _run(device, stream, m, n, k, path, call):
    """``call(ws, ws_bytes) -> rc`` with the cached scratch; if the library finds it too small,
    once more with a buffer of the size it asks for (nothing was launched by the first try)."""
    # The tensor-core kernels use scratch when it is there and do without otherwise, so problems
    # that may go to them (more than 8 rows of activations) ask for their exact need.
    rc = call(*_workspace(device, stream, m, n, k, path, exact=m > 8))
    if rc == ERR_WORKSPACE:
        rc = call(*_workspace(device, stream, m, n, k, path, exact=True))
    _check(rc)


def device_status(device=None):
    """Reads and clears the device status word (0 unless a bounded device-side wait expired)."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    value = ctypes.c_int(0)
    _check(_lib.lbl_device_status(index, ctypes.byref(value)))
    return value.value


def _require(condition, message):
    if not condition:
        raise RuntimeError(message)


def w4a16_gemv_warp_vec(x, packed_w, scales, zeros, group_size):
    """``y[1, N] = fp16(x[1, K] . dequant(W)^T)``, FP32 dequantisation and accumulation."""
    _require(x.is_cuda, "x must be CUDA")
    _require(x.dim() == 2 and x.size(0) == 1, "Expected x shape [1, K]")
    _require(x.dtype == torch.float16, "x must be FP16")
    _require(packed_w.dtype == torch.int32, "packed_w must be int32")
    _require(scales.dtype == torch.float32, "scales must be FP32")
    _require(zeros.dtype == torch.int32, "zeros must be int32")
    _require(
        x.is_contiguous() and packed_w.is_contiguous() and scales.is_contiguous()
        and zeros.is_contiguous(),
        "All tensors must be contiguous",
    )
    _require(packed_w.is_cuda and scales.is_cuda and zeros.is_cuda, "All tensors must be CUDA")
    _require(
        x.device == packed_w.device == scales.device == zeros.device,
        "All tensors must be on the same GPU",
    )
    k = x.size(1)
    _require(
        group_size == 64 and k > 0 and k % 64 == 0,
        "Expected group_size=64 and K divisible by 64",
    )
    _require(packed_w.dim() == 2, "packed_w must be 2D")
    n = packed_w.size(0)
    _require(0 < n <= 2**31 - 1 and k <= 2**31 - 1, "Invalid N or K")
    _require(packed_w.size(1) == k // 8, "Invalid packed weight shape")
    _require(
        tuple(scales.shape) == (n, k // 64) and zeros.shape == scales.shape,
        "Invalid scales or zeros shape",
    )
    _require(x.data_ptr() % 16 == 0, "x must be 16-byte aligned for vector loads")

    y = torch.empty((1, n), dtype=torch.float16, device=x.device)
    stream = _raw_stream(x.device)
    px, pw, ps, pz, py, index = (x.data_ptr(), packed_w.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                 y.data_ptr(), x.device.index)
    _run(x.device, stream, 1, n, k, PATH_AUTO,
         lambda ws, ws_bytes: _lib.lbl_w4a16_gemv(px, pw, ps, pz, py, n, k, group_size, ws, ws_bytes,
                                                  _flags, index, stream))
    return y


def w4a16_gemm(X, packed_w, scales, zeros):
    """``Y[M, N] = fp16(X[M, K] . dequant(W)^T)`` for any M, N, K >= 0, group size 64."""
    _require(
        X.is_cuda and packed_w.is_cuda and scales.is_cuda and zeros.is_cuda,
        "all tensors must be CUDA tensors",
    )
    _require(
        X.device == packed_w.device == scales.device == zeros.device,
        "all tensors must be on the same GPU",
    )
    _require(X.dtype == torch.float16, "X must be float16")
    _require(packed_w.dtype == torch.int32, "packed_w must be int32")
    _require(scales.dtype == torch.float32, "scales must be float32")
    _require(zeros.dtype == torch.int32, "zeros must be int32")
    _require(
        X.dim() == 2 and packed_w.dim() == 2 and scales.dim() == 2 and zeros.dim() == 2,
        "all tensors must be 2D",
    )
    _require(
        X.is_contiguous() and packed_w.is_contiguous() and scales.is_contiguous()
        and zeros.is_contiguous(),
        "all tensors must be contiguous",
    )
    m, k = X.shape
    n = packed_w.size(0)
    _require(packed_w.size(1) == (k + 7) // 8, "packed_w must have shape [N, ceil(K/8)]")
    groups = (k + 63) // 64
    _require(tuple(scales.shape) == (n, groups), "scales must have shape [N, ceil(K/64)]")
    _require(tuple(zeros.shape) == (n, groups), "zeros must have shape [N, ceil(K/64)]")

    Y = torch.empty((m, n), dtype=torch.float16, device=X.device)
    if m == 0 or n == 0:
        return Y
    stream = _raw_stream(X.device)
    px, pw, ps, pz, py, index = (X.data_ptr(), packed_w.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                 Y.data_ptr(), X.device.index)
    _run(X.device, stream, m, n, k, PATH_AUTO,
         lambda ws, ws_bytes: _lib.lbl_w4a16_gemm(px, pw, ps, pz, py, m, n, k, ws, ws_bytes, _flags,
                                                  index, stream))
    return Y


def linear_forced(X, packed_w, scales, zeros, path, op=1, flags=None, workspace=None):
    """Runs the dispatcher with a forced kernel path (benchmarks and tests).  Returns
    ``(Y, path_taken)``; no argument checking beyond what the C ABI does.  ``workspace`` is a
    zeroed uint8 CUDA tensor of at least ``workspace_bytes(m, n, k, path)`` that the caller owns;
    without it the per-stream cached scratch is used."""
    m, k = X.shape
    n = packed_w.size(0)
    Y = torch.empty((m, n), dtype=torch.float16, device=X.device)
    stream = _raw_stream(X.device)
    taken = ctypes.c_int(0)
    call = lambda ws, ws_bytes: _lib.lbl_w4a16_linear(
        X.data_ptr(), packed_w.data_ptr(), scales.data_ptr(), zeros.data_ptr(), Y.data_ptr(),
        m, n, k, op, path, ws, ws_bytes, _flags if flags is None else flags, X.device.index,
        stream, ctypes.byref(taken))
    if workspace is not None:
        _check(call(workspace.data_ptr(), workspace.numel()))
    else:
        _run(X.device, stream, m, n, k, path, call)
    return Y, taken.value


def workspace_bytes(m, n, k, path=PATH_AUTO):
    """Bytes of scratch the given path wants for this problem (``lbl_w4a16_workspace_bytes``)."""
    return _lib.lbl_w4a16_workspace_bytes(m, n, k, path)


def linear_out(X, packed_w, scales, zeros, out, op=None, workspace=None):
    """Dispatcher call that writes into a caller-provided ``out`` ``[M, N]`` (FP16, contiguous,
    16-byte aligned) instead of allocating: what a CUDA-graph runner with static buffers needs.
    ``op`` defaults to the operator ``QuantizedLinear.forward`` would pick.  ``workspace`` is a
    zero-initialised uint8 CUDA tensor the caller owns (at least ``lbl_w4a16_workspace_bytes``);
    without it the per-stream cached scratch is used."""
    m, k = X.shape
    n = packed_w.size(0)
    if op is None:
        op = 0 if (m == 1 and k % 64 == 0 and n % 128 == 0) else 1
    stream = _raw_stream(X.device)
    px, pw, ps, pz, py, index = (X.data_ptr(), packed_w.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                 out.data_ptr(), X.device.index)
    call = lambda ws, ws_bytes: _lib.lbl_w4a16_linear(px, pw, ps, pz, py, m, n, k, op, PATH_AUTO, ws,
                                                      ws_bytes, _flags, index, stream, None)
    if workspace is not None:
        _check(call(workspace.data_ptr(), workspace.numel()))
    else:
        _run(X.device, stream, m, n, k, PATH_AUTO, call)
    return out


def gemv_allreduce(x, packed_w, scales, zeros, exchange):
    """K-split GEMV with the all-reduce fused into the kernel: ``x`` is this rank's ``[1, K/g]``
    slice, the weights its column slice; returns the full ``[1, N]`` (identical on every rank).
    ``exchange`` is a ``tensor_parallel.PeerExchange``."""
    n, k = packed_w.size(0), x.size(1)
    y = torch.empty((1, n), dtype=torch.float16, device=x.device)
    stream = _raw_stream(x.device)
    _run(x.device, stream, 1, n, k, PATH_AUTO,
         lambda ws, ws_bytes: _lib.lbl_w4a16_gemv_allreduce(
             x.data_ptr(), packed_w.data_ptr(), scales.data_ptr(), zeros.data_ptr(), y.data_ptr(), n, k,
             64, exchange.rank, exchange.world, exchange.pointers, exchange.capacity_n, ws, ws_bytes,
             _flags, x.device.index, stream))
    return y


def gemm_scatter(x, packed_w, scales, zeros, exchange, flags=None):
    """First half of the K-split GEMM with fused all-reduce: ``x`` is this rank's ``[M, K/g]``
    slice of the activation, the weights its column slice.  Launches the tcgen05 GEMM on the
    current stream; each finished tile of partial outputs is stored from the epilogue straight
    into the exchange buffer of the rank that owns its columns.  ``exchange`` is a
    ``tensor_parallel.PeerExchange.for_gemm``; follow with ``gemm_allreduce_finish``."""
    m, k = x.shape
    n = packed_w.size(0)
    _check(_lib.lbl_w4a16_gemm_scatter(
        x.data_ptr(), packed_w.data_ptr(), scales.data_ptr(), zeros.data_ptr(), m, n, k, exchange.rank,
        exchange.world, exchange.pointers, exchange.bytes, _flags if flags is None else flags, x.device.index,
        _raw_stream(x.device)))


def gemm_allreduce_finish(y, exchange):
    """Second half: on the current stream, add the ranks' partial outputs of this rank's columns
    and gather the other ranks' columns into ``y`` ``[M, N]`` FP16 (identical on every rank).  May
    run on another stream than the GEMM if an event orders it after the GEMM, and the next
    ``gemm_scatter`` into the same exchange after it."""
    m, n = y.shape
    _check(_lib.lbl_peer_gemm_allreduce_finish(y.data_ptr(), m, n, exchange.rank, exchange.world, exchange.pointers,
                                               exchange.bytes, y.device.index, _raw_stream(y.device)))


def gemm_allreduce(x, packed_w, scales, zeros, exchange, out=None):
    """K-split GEMM and all-reduce on the current stream; returns the full ``[M, N]``."""
    y = out if out is not None else torch.empty((x.size(0), packed_w.size(0)), dtype=torch.float16, device=x.device)
    gemm_scatter(x, packed_w, scales, zeros, exchange)
    gemm_allreduce_finish(y, exchange)
    return y


class LinearGroup:
    """A list of independent decode linears (M <= 2) that run as ONE persistent launch.

    ``problems`` is a sequence of ``(x, packed_w, scales, zeros, y)`` or
    ``(x, packed_w, scales, zeros, y, reduce)`` tuples of CUDA tensors on one device: ``x``
    ``[M, K]`` FP16 and ``y`` ``[M, N]`` FP16 are static buffers that every ``run()`` reads and
    writes.  With an ``exchange`` (``tensor_parallel.PeerExchange``) the problems flagged
    ``reduce`` are K-split shards whose outputs are summed over the ranks by a second kernel over
    NVLink peer memory; every rank must then call ``run()`` the same number of times.
    The reference launches one kernel per linear (``csrc/w4a16_gemv_warp_vec.cu:171-187``)."""

    def __init__(self, problems, exchange=None):
        problems = [tuple(q) for q in problems]
        if not problems:
            raise ValueError("no problems")
        self.device = problems[0][0].device
        array = (GroupProblem * len(problems))()
        self._keep = []
        for slot, q in zip(array, problems):
            x, packed_w, scales, zeros, y = q[:5]
            reduce = bool(q[5]) if len(q) > 5 else False
            _require(all(t.is_cuda and t.device == self.device and t.is_contiguous()
                         for t in (x, packed_w, scales, zeros, y)),
                     "all tensors of a group must be contiguous CUDA tensors on one device")
            _require(x.dtype == torch.float16 and y.dtype == torch.float16 and packed_w.dtype == torch.int32
                     and scales.dtype == torch.float32 and zeros.dtype == torch.int32, "wrong dtype in a group problem")
            m, k = x.shape
            n = packed_w.size(0)
            _require(tuple(packed_w.shape) == (n, k // 8) and tuple(scales.shape) == (n, k // 64)
                     and zeros.shape == scales.shape and tuple(y.shape) == (m, n), "wrong shape in a group problem")
            slot.x, slot.packed_w, slot.scales, slot.zeros, slot.y = (x.data_ptr(), packed_w.data_ptr(),
                                                                      scales.data_ptr(), zeros.data_ptr(), y.data_ptr())
            slot.M, slot.N, slot.K, slot.reduce, slot.reserved = m, n, k, int(reduce), 0
            self._keep.append((x, packed_w, scales, zeros, y))
        self.exchange = exchange
        handle = ctypes.c_void_p()
        if exchange is not None:
            rc = _lib.lbl_w4a16_group_create(array, len(problems), exchange.rank, exchange.world,
                                             exchange.pointers, exchange.capacity_n, self.device.index,
                                             ctypes.byref(handle))
        else:
            rc = _lib.lbl_w4a16_group_create(array, len(problems), 0, 1, None, 0, self.device.index,
                                             ctypes.byref(handle))
        _check(rc)
        self._handle = handle
        self.count = len(problems)
        self.algorithmic_bytes = _lib.lbl_w4a16_group_algorithmic_bytes(handle)

    def run(self):
        """Launch on the current stream of the group's device (asynchronous)."""
        _check(_lib.lbl_w4a16_group_run(self._handle, _flags, _raw_stream(self.device)))

    def close(self):
        """Free the plan; call it after the last run has finished."""
        if self._handle is not None:
            _lib.lbl_w4a16_group_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001  (interpreter shutdown)
            pass


def quantize_pack(weight, group_size=64):
    """quantize_int4 + pack_int4 of a CUDA weight in one kernel.  Returns (packed, scales, zeros)
    in the reference layout, bit-identical to the reference's CPU result
    (lowbitlinear/quantization.py:33-86, :112-141)."""
    _require(weight.is_cuda, "weight must be a CUDA tensor")
    _require(weight.dim() == 2, "weight must have shape [out_features, in_features]")
    _require(weight.dtype in (torch.float16, torch.float32), "weight must be FP16 or FP32")
    _require(group_size == 64, "the device quantiser supports group_size=64 only")
    weight = weight.contiguous()
    n, k = weight.shape
    _require(k > 0, "in_features must be positive")
    groups = (k + 63) // 64
    packed = torch.empty((n, (k + 7) // 8), dtype=torch.int32, device=weight.device)
    scales = torch.empty((n, groups), dtype=torch.float32, device=weight.device)
    zeros = torch.empty((n, groups), dtype=torch.int32, device=weight.device)
    stream = _raw_stream(weight.device)
    _check(_lib.lbl_w4a16_quantize(weight.data_ptr(), int(weight.dtype == torch.float32), n, k, group_size,
                                   packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                   weight.device.index, stream))
    return packed, scales, zeros


def dequantize(packed_w, scales, zeros, in_features=None, dtype=torch.float16, group_size=64):
    """unpack_int4 + dequantize_int4 of CUDA buffers in one kernel: the dense ``[N, K]`` weight
    ``float(q - zero) * scale`` as FP32 (bit-identical to ``lowbitlinear/quantization.py:88-110``)
    or rounded once to FP16."""
    _require(packed_w.is_cuda and scales.is_cuda and zeros.is_cuda, "buffers must be CUDA tensors")
    _require(packed_w.dtype == torch.int32 and packed_w.dim() == 2, "packed_w must be a 2-D INT32 tensor")
    _require(dtype in (torch.float16, torch.float32), "dtype must be FP16 or FP32")
    _require(group_size == 64, "the device dequantiser supports group_size=64 only")
    n, words = packed_w.shape
    k = words * 8 if in_features is None else int(in_features)
    _require(0 < k <= words * 8 and (k + 7) // 8 == words, "in_features does not match packed_w")
    groups = (k + 63) // 64
    _require(scales.dtype == torch.float32 and tuple(scales.shape) == (n, groups), "Invalid scales or zeros shape")
    _require(zeros.dtype == torch.int32 and tuple(zeros.shape) == (n, groups), "Invalid scales or zeros shape")
    _require(packed_w.is_contiguous() and scales.is_contiguous() and zeros.is_contiguous(),
             "buffers must be contiguous")
    _require(scales.device == packed_w.device and zeros.device == packed_w.device,
             "All tensors must be on the same device")
    weight = torch.empty((n, k), dtype=dtype, device=packed_w.device)
    stream = _raw_stream(packed_w.device)
    _check(_lib.lbl_w4a16_dequantize(packed_w.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                     weight.data_ptr(), int(dtype == torch.float32), n, k, group_size,
                                     packed_w.device.index, stream))
    return weight


def select_path(m, n, k, op=1):
    return _lib.lbl_w4a16_select_path(m, n, k, op)


def register_operators(lib):
    """Define the reference's two operator schemas and implement them for CUDA tensors."""
    if _registered:
        return
    ext = torch.library.Library("lowbitlinear_ext", "FRAGMENT")
    ext.define(GEMV_SCHEMA)
    ext.impl("w4a16_gemv_warp_vec", w4a16_gemv_warp_vec, "CUDA")
    cute = torch.library.Library("lowbitlinear_cute_w4a16", "FRAGMENT")
    cute.define(GEMM_SCHEMA)
    cute.impl("gemm", w4a16_gemm, "CUDA")
    _registered.extend((ext, cute))
