"""The drop-in boundary: the native library loads, exports every entry point the header
declares, registers the reference's two operator schemas, and a missing library is an error
for CUDA work but not for CPU work.  No GPU compute happens in the CPU-marked tests.
The fresh-process schema test and the shape and error tables are adapted from NanjinLin/LowBitLinear
tests/test_api_dispatch.py (MIT)."""
import ctypes
import os
import re
import shutil
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "lowbitlinear_b200.h"
LIBRARY = ROOT / "lowbitlinear_b200" / "_C.so"

needs_library = pytest.mark.skipif(not LIBRARY.is_file(), reason="native library not built (python -m lowbitlinear_b200.build)")


def declared_entry_points():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(lbl_\w+)\s*\(", text)))


def test_header_declares_the_boundary():
    names = declared_entry_points()
    for required in ("lbl_w4a16_gemv", "lbl_w4a16_gemm", "lbl_w4a16_linear", "lbl_w4a16_workspace_bytes",
                     "lbl_w4a16_workspace_init", "lbl_w4a16_select_path", "lbl_last_error", "lbl_version",
                     "lbl_device_status"):
        assert required in names


@needs_library
def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(LIBRARY))
    for name in declared_entry_points():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    lib.lbl_version.restype = ctypes.c_int
    assert lib.lbl_version() >= 100
    lib.lbl_last_error.restype = ctypes.c_char_p
    assert lib.lbl_last_error() == b""


@needs_library
def test_argument_errors_need_no_gpu():
    """Checks that run before any CUDA call: codes and messages of the C ABI."""
    lib = ctypes.CDLL(str(LIBRARY))
    lib.lbl_last_error.restype = ctypes.c_char_p
    p, i64, i32, u32, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_uint, ctypes.c_size_t
    lib.lbl_w4a16_gemv.argtypes = [p, p, p, p, p, i64, i64, i32, p, sz, u32, i32, p]
    rc = lib.lbl_w4a16_gemv(None, None, None, None, None, 128, 65, 64, None, 0, 0, 0, None)
    assert rc == -1 and b"divisible by 64" in lib.lbl_last_error()
    rc = lib.lbl_w4a16_gemv(None, None, None, None, None, 128, 64, 32, None, 0, 0, 0, None)
    assert rc == -1 and b"group_size=64" in lib.lbl_last_error()
    rc = lib.lbl_w4a16_gemv(None, None, None, None, None, 0, 64, 64, None, 0, 0, 0, None)
    assert rc == -1 and b"Invalid N or K" in lib.lbl_last_error()
    rc = lib.lbl_w4a16_gemv(8, None, None, None, None, 128, 64, 64, None, 0, 0, 0, None)
    assert rc == -1 and b"16-byte aligned" in lib.lbl_last_error()
    lib.lbl_w4a16_gemm.argtypes = [p, p, p, p, p, i64, i64, i64, p, sz, u32, i32, p]
    assert lib.lbl_w4a16_gemm(None, None, None, None, None, 0, 32, 65, None, 0, 0, 0, None) == 0  # empty output
    assert lib.lbl_w4a16_gemm(None, None, None, None, None, -1, 32, 65, None, 0, 0, 0, None) == -1


@needs_library
def test_misaligned_workspace_is_rejected_before_anything_is_launched():
    """A sub-allocated scratch pointer that is not 16-byte aligned would fault on the device (vector
    loads, atomics); the C ABI refuses it on the host, for every entry point that takes one."""
    lib = ctypes.CDLL(str(LIBRARY))
    lib.lbl_last_error.restype = ctypes.c_char_p
    p, i64, i32, u32, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_uint, ctypes.c_size_t
    lib.lbl_w4a16_gemm.argtypes = [p, p, p, p, p, i64, i64, i64, p, sz, u32, i32, p]
    rc = lib.lbl_w4a16_gemm(16, 16, 16, 16, 16, 16, 256, 512, 1024 + 8, 1 << 20, 0, 0, None)
    assert rc == -1 and b"workspace must be 16-byte aligned" in lib.lbl_last_error()
    lib.lbl_w4a16_linear.argtypes = [p, p, p, p, p, i64, i64, i64, i32, i32, p, sz, u32, i32, p, p]
    rc = lib.lbl_w4a16_linear(16, 16, 16, 16, 16, 16, 256, 512, 1, 5, 1024 + 4, 1 << 20, 0, 0, None, None)
    assert rc == -1 and b"workspace must be 16-byte aligned" in lib.lbl_last_error()
    lib.lbl_w4a16_gemv.argtypes = [p, p, p, p, p, i64, i64, i32, p, sz, u32, i32, p]
    rc = lib.lbl_w4a16_gemv(16, 16, 16, 16, 16, 256, 4096, 64, 1024 + 2, 1 << 20, 0, 0, None)
    assert rc == -1 and b"workspace must be 16-byte aligned" in lib.lbl_last_error()
    lib.lbl_w4a16_gemv_allreduce.argtypes = [p, p, p, p, p, i64, i64, i32, i32, i32, ctypes.POINTER(p), i64,
                                             p, sz, u32, i32, p]
    buffers = (p * 2)(4096, 8192)
    rc = lib.lbl_w4a16_gemv_allreduce(16, 16, 16, 16, 16, 256, 4096, 64, 0, 2, buffers, 256, 1024 + 8, 1 << 20,
                                      0, 0, None)
    assert rc == -1 and b"workspace must be 16-byte aligned" in lib.lbl_last_error()


@needs_library
def test_group_argument_errors_need_no_gpu():
    from lowbitlinear_b200 import _ops

    lib = ctypes.CDLL(str(LIBRARY))
    lib.lbl_last_error.restype = ctypes.c_char_p
    p = ctypes.c_void_p
    lib.lbl_w4a16_group_create.argtypes = [ctypes.POINTER(_ops.GroupProblem), ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                           ctypes.POINTER(p), ctypes.c_int64, ctypes.c_int, ctypes.POINTER(p)]
    handle = p()
    problems = (_ops.GroupProblem * 1)()
    assert lib.lbl_w4a16_group_create(problems, 0, 0, 1, None, 0, 0, ctypes.byref(handle)) == -1
    assert lib.lbl_w4a16_group_create(problems, 1, 0, 1, None, 0, 0, ctypes.byref(handle)) == -1
    assert b"null tensor pointer" in lib.lbl_last_error()
    q = problems[0]
    q.x = q.packed_w = q.scales = q.zeros = q.y = 4096
    q.M, q.N, q.K = 3, 64, 256
    assert lib.lbl_w4a16_group_create(problems, 1, 0, 1, None, 0, 0, ctypes.byref(handle)) == -4
    assert b"grouped GEMV serves" in lib.lbl_last_error()
    q.M, q.reduce = 1, 1
    assert lib.lbl_w4a16_group_create(problems, 1, 0, 2, None, 0, 0, ctypes.byref(handle)) == -1
    assert b"exchange buffers" in lib.lbl_last_error()
    q.y = 4096 + 8
    assert lib.lbl_w4a16_group_create(problems, 1, 0, 1, None, 0, 0, ctypes.byref(handle)) == -1
    assert b"16-byte aligned" in lib.lbl_last_error() and handle.value is None


@needs_library
def test_gemm_allreduce_argument_errors_need_no_gpu():
    lib = ctypes.CDLL(str(LIBRARY))
    lib.lbl_last_error.restype = ctypes.c_char_p
    p, i64, i32, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
    lib.lbl_peer_gemm_buffer_bytes.restype = sz
    lib.lbl_peer_gemm_buffer_bytes.argtypes = [i64, i64, i32]
    lib.lbl_w4a16_gemm_scatter.argtypes = [p, p, p, p, i64, i64, i64, i32, i32, ctypes.POINTER(p), sz, ctypes.c_uint,
                                           i32, p]
    lib.lbl_peer_gemm_allreduce_finish.argtypes = [p, i64, i64, i32, i32, ctypes.POINTER(p), sz, i32, p]
    # world slots of [M, N / world] FP16 + one result block + the 2 KiB control block
    assert lib.lbl_peer_gemm_buffer_bytes(2048, 4096, 4) == 2048 + 2048 * 4096 * 2 + 2048 * 1024 * 2
    assert lib.lbl_peer_gemm_buffer_bytes(2048, 4096, 3) == 0 and lib.lbl_peer_gemm_buffer_bytes(0, 4096, 2) == 0
    size = lib.lbl_peer_gemm_buffer_bytes(512, 1024, 2)
    buffers = (p * 2)(4096, 8192)
    t = 1 << 20
    assert lib.lbl_w4a16_gemm_scatter(t, t, t, t, 512, 1024, 512, 0, 1, buffers, size, 0, 0, None) == -1
    assert b"rank/world" in lib.lbl_last_error()
    assert lib.lbl_w4a16_gemm_scatter(t, t, t, t, 512, 768, 512, 0, 2, buffers, size, 0, 0, None) == -4
    assert b"256 * world" in lib.lbl_last_error()
    assert lib.lbl_w4a16_gemm_scatter(t, t, t, t, 512, 1024, 512, 0, 2, buffers, size - 16, 0, 0, None) == -3
    assert b"exchange buffers hold" in lib.lbl_last_error()
    assert lib.lbl_w4a16_gemm_scatter(t, t, t, t, 512, 1024, 320, 0, 2, buffers, size, 0, 0, None) == -4
    assert b"K % 256" in lib.lbl_last_error()
    assert lib.lbl_w4a16_gemm_scatter(t, t + 4, t, t, 512, 1024, 512, 0, 2, buffers, size, 0, 0, None) == -1
    assert b"16-byte aligned" in lib.lbl_last_error()
    buffers[1] = None
    assert lib.lbl_peer_gemm_allreduce_finish(t, 512, 1024, 1, 2, buffers, size, 0, None) == -1
    assert b"rank 1" in lib.lbl_last_error()
    buffers[1] = 8192
    assert lib.lbl_peer_gemm_allreduce_finish(t + 2, 512, 1024, 1, 2, buffers, size, 0, None) == -1
    assert b"y is null or not 16-byte aligned" in lib.lbl_last_error()


@needs_library
def test_dispatcher_choices_and_scratch_sizes():
    from lowbitlinear_b200 import _ops
    from lowbitlinear_b200._extension import load_cuda_extension

    assert load_cuda_extension(required=True)
    env_backup = {k: os.environ.pop(k, None) for k in ("LBL_FORCE_PATH",)}
    try:
        name = lambda m, n, k: _ops.PATH_NAMES[_ops.select_path(m, n, k)]
        # Decode shapes stream; a small N or a long K is split across CTAs.
        assert name(1, 6144, 4096) == "gemv"
        assert name(1, 24576, 4096) == "gemv"
        assert name(1, 4096, 4096) == "gemv"
        assert name(1, 4096, 12288) == "gemv"
        assert name(1, 512, 4096) == "gemv_splitk"     # a tensor-parallel shard: 32 row tiles
        assert name(4, 4096, 12288) == "gemv"          # 96 KB of activations still fit one CTA per SM
        assert name(8, 4096, 12288) == "gemm_tc_small" # 192 KB do not: K would be cut, the tensor cores are faster
        assert _ops.PATH_NAMES[_ops.select_path(4, 4096, 12288)] == "gemv"
        # Prefill shapes go to the tensor cores; ragged shapes to the masked kernel.
        assert name(2048, 24576, 4096) == "gemm_tc_pair"   # pairs of CTAs share the dequantised weights
        assert name(256, 24576, 4096) == "gemm_tc"
        assert name(128, 4096, 12288) == "gemm_tc_small"   # weights on the M side of the MMA
        assert name(16, 24576, 4096) == "gemv"             # wide N, whole operand on chip: streaming still wins
        assert name(17, 24576, 4096) == "gemm_tc_small"
        assert name(16, 6144, 4096) == "gemm_tc_small"
        assert name(64, 24576, 4096) == "gemm_tc"          # wide N: 256-wide tiles fill the SMs
        # More than 128 rows on a shape whose 256 x 256 tiles would fill under half of the SMs: the
        # tensor-memory GEMM, which cuts K into slices (also the kernel for N % 256 == 128).
        assert name(129, 4096, 12288) == "gemm_wt"
        assert name(512, 4096, 12288) == "gemm_wt"
        assert name(2048, 512, 4096) == "gemm_wt"           # a tensor-parallel shard of O
        assert name(2048, 4096, 12288) == "gemm_tc_pair"
        assert name(300, 384, 512) == "gemm_wt"
        assert name(5, 9, 70) == "generic"
        assert name(1, 129, 64) == "generic"
        assert name(2048, 129, 4096) == "generic"
        ws = _ops._lib.lbl_w4a16_workspace_bytes
        assert ws(1, 6144, 4096, _ops.PATH_AUTO) == 0
        # fixed 64 KiB of arrival counters + nsplit * M * N floats
        assert ws(1, 4096, 4096, _ops.PATH_AUTO) == 0
        assert ws(1, 512, 4096, _ops.PATH_AUTO) == 64 * 1024 + 4 * 512 * 4
        assert ws(2048, 24576, 4096, _ops.PATH_AUTO) == 0
        # small-M tensor-core GEMM: counters + one FP32 partial tile [M, 128] per row block and
        # slice of K; 32 row blocks are cut 8 ways, 192 row blocks 3 ways (waves of 2 * 148 CTAs)
        assert ws(16, 4096, 4096, _ops.PATH_AUTO) == 64 * 1024 + 32 * 8 * 16 * 128 * 4
        assert ws(17, 24576, 4096, _ops.PATH_AUTO) == 64 * 1024 + 192 * 3 * 17 * 128 * 4
        assert ws(16, 24576, 4096, _ops.PATH_AUTO) == 0
        # tensor-memory GEMM: one FP32 partial tile [M, 256] per row block and slice (16 blocks cut 8 ways)
        assert ws(129, 4096, 12288, _ops.PATH_AUTO) == 64 * 1024 + 16 * 8 * 129 * 256 * 4
    finally:
        for k, v in env_backup.items():
            if v is not None:
                os.environ[k] = v


@needs_library
def test_autoload_registers_reference_schemas_once():
    """Fresh process: no JIT, one load_library call over three loads, exact schema strings,
    CUDA kernels registered (the contract of the reference's tests/test_api_dispatch.py:62-92)."""
    code = """
import torch
import torch.utils.cpp_extension as cpp
def forbidden(*args, **kwargs):
    raise AssertionError('JIT compilation is forbidden')
cpp.load = forbidden
cpp.load_inline = forbidden
calls = []
original = torch.ops.load_library
def record(path):
    calls.append(path)
    return original(path)
torch.ops.load_library = record
import lowbitlinear_b200
from lowbitlinear_b200._extension import load_cuda_extension
for _ in range(3):
    assert load_cuda_extension(required=True)
assert len(calls) == 1, calls
assert str(torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec.default._schema) == 'lowbitlinear_ext::w4a16_gemv_warp_vec(Tensor x, Tensor packed_w, Tensor scales, Tensor zeros, int group_size) -> Tensor'
assert str(torch.ops.lowbitlinear_cute_w4a16.gemm.default._schema) == 'lowbitlinear_cute_w4a16::gemm(Tensor X, Tensor packed_w, Tensor scales, Tensor zeros) -> Tensor'
for name in ('lowbitlinear_ext::w4a16_gemv_warp_vec', 'lowbitlinear_cute_w4a16::gemm'):
    assert torch._C._dispatch_has_kernel_for_dispatch_key(name, 'CUDA'), name
    assert not torch._C._dispatch_has_kernel_for_dispatch_key(name, 'CPU'), name
if torch.cuda.is_available():
    for m, n, k in ((1, 128, 64), (5, 9, 70), (1, 256, 512)):
        layer = lowbitlinear_b200.QuantizedLinear.from_float(torch.ones(n, k, device='cuda'))
        actual = layer(torch.ones(m, k, dtype=torch.float16, device='cuda'))
        assert torch.equal(actual, torch.full_like(actual, float(k)))
    torch.cuda.synchronize()
"""
    subprocess.run([sys.executable, "-c", code], check=True, timeout=180, cwd=ROOT)


@needs_library
def test_cpu_tensors_are_rejected_by_the_operators():
    from lowbitlinear_b200._extension import load_cuda_extension

    assert load_cuda_extension(required=True)
    args = (torch.ones(1, 64, dtype=torch.float16), torch.zeros(128, 8, dtype=torch.int32),
            torch.ones(128, 1), torch.zeros(128, 1, dtype=torch.int32))
    with pytest.raises(NotImplementedError, match="CPU"):
        torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(*args, 64)
    with pytest.raises(NotImplementedError, match="CPU"):
        torch.ops.lowbitlinear_cute_w4a16.gemm(*args)


@pytest.fixture
def python_only_package(tmp_path):
    package = tmp_path / "lowbitlinear_b200"
    package.mkdir()
    for path in (ROOT / "lowbitlinear_b200").glob("*.py"):
        shutil.copy2(path, package / path.name)
    return tmp_path


def test_cpu_api_works_without_the_native_library(python_only_package):
    tmp_path = python_only_package
    code = """
from pathlib import Path
import pytest
import torch
import lowbitlinear_b200
from lowbitlinear_b200 import QuantizedLinear
from lowbitlinear_b200._extension import load_cuda_extension
assert Path(lowbitlinear_b200.__file__).resolve().parent == Path.cwd() / 'lowbitlinear_b200'
assert not load_cuda_extension()
layer = QuantizedLinear.from_float(torch.ones(3, 65))
assert torch.equal(layer(torch.ones(2, 65, dtype=torch.float16)), torch.full((2, 3), 65., dtype=torch.float16))
with pytest.raises(ImportError, match='--no-build-isolation'):
    load_cuda_extension(required=True)
"""
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=str(tmp_path))
    subprocess.run([sys.executable, "-c", code], cwd=tmp_path, env=env, check=True, timeout=180)


@pytest.mark.gpu
def test_cuda_forward_without_the_native_library_is_an_error(python_only_package, cuda_device):
    """A missing build must never turn into a silent fallback."""
    tmp_path = python_only_package
    code = """
import pytest
import torch
from lowbitlinear_b200 import QuantizedLinear
layer = QuantizedLinear.from_float(torch.ones(128, 64, device='cuda'))
with pytest.raises(ImportError, match='python -m lowbitlinear_b200.build'):
    layer(torch.ones(1, 64, device='cuda', dtype=torch.float16))
with pytest.raises(ImportError):
    layer(torch.ones(4, 64, device='cuda', dtype=torch.float16))
"""
    env = dict(os.environ, PYTHONPATH=str(tmp_path))
    subprocess.run([sys.executable, "-c", code], cwd=tmp_path, env=env, check=True, timeout=180)


@pytest.mark.gpu
@pytest.mark.parametrize("op_name", ["gemv", "gemm"])
def test_operator_on_noncurrent_gpu(op_name, cuda_ops):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    code = """
import sys
import torch
import lowbitlinear_b200
from lowbitlinear_b200.quantization import pack_int4
with torch.cuda.device(1):
    x = torch.ones(1, 256, device='cuda:1', dtype=torch.float16)
    packed = pack_int4(torch.ones(128, 256, device='cuda:1', dtype=torch.uint8))
    scales = torch.ones(128, 4, device='cuda:1')
    zeros = torch.zeros(128, 4, device='cuda:1', dtype=torch.int32)
    torch.cuda.synchronize(1)
torch.cuda.set_device(0)
if sys.argv[1] == 'gemv':
    actual = torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(x, packed, scales, zeros, 64)
else:
    actual = torch.ops.lowbitlinear_cute_w4a16.gemm(x, packed, scales, zeros)
torch.cuda.synchronize(0)
torch.cuda.synchronize(1)
assert torch.cuda.current_device() == 0
assert actual.device == x.device
assert torch.equal(actual, torch.full_like(actual, 256.))
"""
    subprocess.run([sys.executable, "-c", code, op_name], check=True, timeout=180, cwd=ROOT)


def test_a_library_built_from_older_sources_is_reported(monkeypatch):
    """The loader compares the recorded build fingerprint with the present sources before it
    touches the shared object (a loaded library stays mapped for the life of the process)."""
    from lowbitlinear_b200 import _extension, _fingerprint

    recorded = _fingerprint.recorded_build()
    if recorded is None:
        pytest.skip("no build record in this tree")
    fingerprint, flags, defines = recorded
    assert _fingerprint.source_fingerprint(flags, defines) == fingerprint
    assert not _extension._is_out_of_date()
    monkeypatch.setattr(_fingerprint, "recorded_build", lambda: ("0" * 64, flags, defines))
    assert _extension._is_out_of_date()
    monkeypatch.setattr(_fingerprint, "recorded_build", lambda: None)
    assert not _extension._is_out_of_date()
