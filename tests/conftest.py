"""Shared fixtures: deterministic setup, the numpy oracle as checker, seeded layer inputs.

Tests marked ``gpu`` need a B200 and the built native library and call the kernels through
the C ABI (``torch.ops`` -> ctypes -> ``_C.so``); everything else runs on CPU.
"""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from oracle import w4a16_oracle as oracle  # noqa: E402  (checker only)

GOLDEN = ROOT / "tests" / "golden"
ATOL, RTOL = 2e-3, 1e-3  # kernel tolerance of the reference's tests (tests/test_cuda_gemv.py:7)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200) and the native library")


@pytest.fixture(scope="session", autouse=True)
def ieee_fp32_matmul():
    previous = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32 = previous


@pytest.fixture(autouse=True)
def reproducible_randomness():
    devices = list(range(torch.cuda.device_count())) if torch.cuda.is_available() else []
    with torch.random.fork_rng(devices=devices):
        torch.manual_seed(42)
        yield


@pytest.fixture(scope="session")
def golden_small():
    data = np.load(GOLDEN / "small_cases.npz")
    cases = {}
    for key in data.files:
        name, field = key.split("/")
        cases.setdefault(name, {})[field] = data[key]
    return cases


@pytest.fixture
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA GPU")
    device = torch.device("cuda", torch.cuda.current_device())
    yield device
    torch.cuda.synchronize(device)  # asynchronous errors belong to the test that caused them


@pytest.fixture
def cuda_ops(cuda_device):
    """The native library must be loaded and both operators registered for CUDA: on a GPU
    machine a missing build is a failure, not a skip."""
    from lowbitlinear_b200 import _ops
    from lowbitlinear_b200._extension import load_cuda_extension

    load_cuda_extension(required=True)
    for name in ("lowbitlinear_ext::w4a16_gemv_warp_vec", "lowbitlinear_cute_w4a16::gemm"):
        assert torch._C._dispatch_has_kernel_for_dispatch_key(name, "CUDA"), name
    yield cuda_device
    torch.cuda.synchronize(cuda_device)
    assert _ops.device_status(cuda_device) == 0, "a bounded device-side wait expired"


def seeded_layer(m, n, k, seed, std=0.02, device="cpu"):
    """W ~ N(0, std) and x ~ N(0, 1), FP16, from a CPU generator (same bits everywhere),
    quantised on CPU by the package and moved to ``device``."""
    from lowbitlinear_b200.quantization import pack_int4, quantize_int4

    g = torch.Generator("cpu").manual_seed(seed)
    weight = (torch.randn(n, k, generator=g) * std).half()
    x = torch.randn(m, k, generator=g).half()
    q, scales, zeros = quantize_int4(weight, 64)
    packed = pack_int4(q)
    return tuple(t.to(device) for t in (x, packed, scales, zeros))


@pytest.fixture
def make_layer():
    return seeded_layer


def oracle_linear(x, packed, scales, zeros, group_size=64, *, mma=False):
    """The numpy oracle applied to torch tensors; returns a CPU FP16 tensor."""
    y = oracle.linear_int4_reference(
        x.detach().cpu().numpy(), packed.detach().cpu().numpy(), scales.detach().cpu().numpy(),
        zeros.detach().cpu().numpy(), group_size, round_weights_fp16=mma)
    return torch.from_numpy(y)


@pytest.fixture
def packed_reference():
    return oracle_linear


def torch_fp32_linear(x, packed, scales, zeros, *, mma=False):
    """Independent FP32 evaluation on the tensors' own device, for sizes the numpy oracle would
    take too long on: int64 shifts for the nibbles, gathered metadata, one FP32 matmul."""
    k = x.shape[1]
    shifts = torch.arange(8, device=x.device) * 4
    q = ((packed.to(torch.int64)[..., None] >> shifts) & 15).reshape(packed.shape[0], -1)[:, :k]
    groups = torch.arange(k, device=x.device) // 64
    weight = (q.float() - zeros[:, groups].float()) * scales[:, groups]
    if mma:
        weight = weight.half().float()
    return (x.float() @ weight.T).half()


def assert_north_star_parity(actual, expected):
    """Output tolerance of the benchmark spec: relative L2 <= 1e-3 and no element further than
    1e-2 + 1e-2 |expected|."""
    a = actual.detach().float().cpu()
    e = expected.detach().float().cpu()
    rel_l2 = ((a - e).norm() / e.norm().clamp_min(1e-30)).item()
    assert rel_l2 <= 1e-3, f"relative L2 error {rel_l2:.3e}"
    worst = ((a - e).abs() - (1e-2 + 1e-2 * e.abs())).max().item()
    assert worst <= 0, f"element outside 1e-2 + 1e-2|y| by {worst:.3e}"


def expected_for_operator(x, packed, scales, zeros):
    """Oracle output for the any-shape operator.  Shapes that its dispatcher hands to the
    streaming kernel keep the FP32 scale (the reference-path semantics); the tensor-core and
    masked kernels round each dequantised weight to FP16 first, as the reference GEMM does."""
    from lowbitlinear_b200 import _ops

    path = _ops.select_path(x.shape[0], packed.shape[0], x.shape[1])
    fp32_scale = path in (_ops.PATH_GEMV, _ops.PATH_GEMV_SPLITK)
    return oracle_linear(x, packed, scales, zeros, mma=not fp32_scale)
