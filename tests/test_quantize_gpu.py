"""Device quantiser (lbl_w4a16_quantize): packed words, scales and zero points must equal the
reference's CPU results bit for bit -- against the reference-generated fixtures, against the
numpy oracle on seeded and adversarial inputs, and against the reference's hashes at benchmark
size."""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from oracle import w4a16_oracle as oracle  # noqa: E402

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def _device_quantize(weight_np, device):
    from lowbitlinear_b200 import _ops

    packed, scales, zeros = _ops.quantize_pack(torch.from_numpy(weight_np).to(device), 64)
    torch.cuda.synchronize(device)
    return packed.cpu().numpy(), scales.cpu().numpy(), zeros.cpu().numpy()


def _assert_bit_exact(weight_np, device):
    q, scales, zeros = oracle.quantize_int4(weight_np, 64)
    packed = oracle.pack_int4(q)
    got_packed, got_scales, got_zeros = _device_quantize(weight_np, device)
    assert got_packed.shape == packed.shape and got_packed.dtype == np.int32
    assert np.array_equal(got_zeros, zeros)
    assert np.array_equal(got_scales.view(np.uint32), scales.view(np.uint32))
    assert np.array_equal(got_packed, packed)


def test_reference_fixtures(cuda_ops, golden_small):
    checked = 0
    for name, case in golden_small.items():
        if int(case["group_size"]) != 64:
            continue
        packed, scales, zeros = _device_quantize(case["weight"], cuda_ops)
        assert np.array_equal(packed, case["packed"]), name
        assert np.array_equal(scales.view(np.uint32), case["scales"].view(np.uint32)), name
        assert np.array_equal(zeros, case["zeros"]), name
        checked += 1
    assert checked >= 5


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("n,k", [(1, 1), (3, 7), (5, 8), (2, 63), (4, 64), (5, 65), (7, 100),
                                 (9, 127), (16, 129), (33, 1000), (128, 4096), (17, 4104)])
def test_seeded_shapes(cuda_ops, n, k, dtype):
    rng = np.random.default_rng(1000 * n + k)
    weight = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)).astype(dtype)
    _assert_bit_exact(weight, cuda_ops)


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_adversarial_groups(cuda_ops, dtype):
    """Groups that exercise every branch: all zero, constant, one-signed, ties at .5, the FP16
    extremes, subnormals, and a wide spread of magnitudes."""
    rng = np.random.default_rng(7)
    k = 64 * 12
    rows = []
    base = rng.standard_normal((4, k), dtype=np.float32)
    rows.append(np.zeros((1, k), np.float32))
    rows.append(np.full((1, k), 0.375, np.float32))
    rows.append(np.full((1, k), -0.375, np.float32))
    rows.append(np.abs(base[:1]))
    rows.append(-np.abs(base[1:2]))
    rows.append(np.tile(np.arange(64, dtype=np.float32) * 0.5, k // 64)[None])          # exact ties
    rows.append(np.tile((np.arange(64, dtype=np.float32) - 32.0) * 0.25, k // 64)[None])
    rows.append(np.where(rng.random((1, k)) < 0.5, 65504.0, -65504.0).astype(np.float32))
    rows.append((base[2:3] * 6e-8))                                                     # FP16 subnormals
    rows.append(base[3:4] * np.exp2(rng.integers(-14, 15, (1, k))).astype(np.float32))
    sparse = np.zeros((1, k), np.float32)
    sparse[0, ::64] = 1.0
    rows.append(sparse)
    weight = np.concatenate(rows).astype(dtype)
    assert np.isfinite(weight.astype(np.float32)).all()
    _assert_bit_exact(weight, cuda_ops)
    _assert_bit_exact(np.ascontiguousarray(weight[:, :k - 37]), cuda_ops)


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("name", ["o_proj", "down_proj"])
def test_benchmark_size_hashes(cuda_ops, name):
    """Benchmark-size linears against the hashes of the reference's own outputs."""
    spec = json.loads((GOLDEN / "full_size.json").read_text())[name]
    g = torch.Generator("cpu").manual_seed(spec["seed"])
    weight = (torch.randn(spec["n"], spec["k"], generator=g) * spec["std"]).half()
    assert _sha(weight.numpy()) == spec["weight_sha256"], "torch CPU generator changed"
    packed, scales, zeros = _device_quantize(weight.numpy(), cuda_ops)
    assert _sha(packed) == spec["packed_sha256"]
    assert _sha(scales) == spec["scales_sha256"]
    assert _sha(zeros) == spec["zeros_sha256"]


def test_from_float_on_device_equals_cpu(cuda_ops):
    """QuantizedLinear.from_float of a CUDA weight uses the device quantiser: same buffers as
    from_float on the CPU copy, and a working forward."""
    from lowbitlinear_b200 import QuantizedLinear

    g = torch.Generator("cpu").manual_seed(11)
    weight = (torch.randn(256, 1024, generator=g) * 0.02).half()
    x = torch.randn(1, 1024, generator=g).half()
    on_cpu = QuantizedLinear.from_float(weight)
    on_gpu = QuantizedLinear.from_float(weight.to(cuda_ops))
    assert on_gpu.packed_weight.device.type == "cuda"
    assert torch.equal(on_gpu.packed_weight.cpu(), on_cpu.packed_weight)
    assert torch.equal(on_gpu.scales.cpu(), on_cpu.scales)
    assert torch.equal(on_gpu.zeros.cpu(), on_cpu.zeros)
    y = on_gpu(x.to(cuda_ops)).float().cpu()
    torch.testing.assert_close(y, on_cpu(x).float(), atol=2e-3, rtol=1e-3)


def test_non_contiguous_and_other_group_sizes(cuda_ops):
    """A strided view is made contiguous first; group sizes other than 64 keep the torch path."""
    from lowbitlinear_b200 import QuantizedLinear, _ops
    from lowbitlinear_b200.quantization import quantize_pack_int4

    rng = np.random.default_rng(3)
    wide = (rng.standard_normal((12, 256), dtype=np.float32) * 0.1).astype(np.float16)
    view = torch.from_numpy(wide).to(cuda_ops)[:, 64:192]
    packed, scales, zeros = quantize_pack_int4(view, 64)
    q, s, z = oracle.quantize_int4(np.ascontiguousarray(wide[:, 64:192]), 64)
    assert np.array_equal(packed.cpu().numpy(), oracle.pack_int4(q))
    assert np.array_equal(scales.cpu().numpy(), s) and np.array_equal(zeros.cpu().numpy(), z)

    layer = QuantizedLinear.from_float(torch.from_numpy(wide).to(cuda_ops), group_size=32)
    assert layer.scales.shape == (12, 8)
    with pytest.raises(RuntimeError, match="group_size=64"):
        _ops.quantize_pack(torch.from_numpy(wide).to(cuda_ops), 32)


# ---- device dequantiser (lbl_w4a16_dequantize) ------------------------------------------------

def _device_dequantize(packed, scales, zeros, k, dtype, device):
    from lowbitlinear_b200 import _ops

    out = _ops.dequantize(*(torch.from_numpy(a).to(device) for a in (packed, scales, zeros)),
                          in_features=k, dtype=dtype)
    torch.cuda.synchronize(device)
    return out.cpu().numpy()


@pytest.mark.parametrize("n,k", [(1, 1), (3, 7), (5, 8), (4, 64), (5, 65), (7, 100), (33, 1000),
                                 (128, 4096), (17, 4104)])
def test_dequantize_matches_oracle(cuda_ops, n, k):
    rng = np.random.default_rng(2000 * n + k)
    weight = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)).astype(np.float16)
    q, scales, zeros = oracle.quantize_int4(weight, 64)
    packed = oracle.pack_int4(q)
    expected = oracle.dequantize_int4(oracle.unpack_int4(packed, original_k=k), scales, zeros, 64)
    as_fp32 = _device_dequantize(packed, scales, zeros, k, torch.float32, cuda_ops)
    assert as_fp32.shape == (n, k)
    assert np.array_equal(as_fp32.view(np.uint32), expected.view(np.uint32))
    as_fp16 = _device_dequantize(packed, scales, zeros, k, torch.float16, cuda_ops)
    assert np.array_equal(as_fp16.view(np.uint16), expected.astype(np.float16).view(np.uint16))


def test_dequantize_reference_fixtures(cuda_ops, golden_small):
    for name, case in golden_small.items():
        if int(case["group_size"]) != 64:
            continue
        k = case["weight"].shape[1]
        expected = oracle.dequantize_int4(case["q"], case["scales"], case["zeros"], 64)
        got = _device_dequantize(case["packed"], case["scales"], case["zeros"], k, torch.float32, cuda_ops)
        assert np.array_equal(got.view(np.uint32), expected.view(np.uint32)), name


def test_dequantize_every_level_and_zero_point(cuda_ops):
    """All 16 x 16 combinations of level and zero point under an awkward scale."""
    levels = np.tile(np.arange(16, dtype=np.uint8), 4)[None].repeat(16, 0)        # [16, 64]
    zeros = np.arange(16, dtype=np.int32)[:, None]
    scales = np.full((16, 1), 0.0123456789, np.float32)
    packed = oracle.pack_int4(levels)
    got = _device_dequantize(packed, scales, zeros, 64, torch.float32, cuda_ops)
    expected = oracle.dequantize_int4(levels, scales, zeros, 64)
    assert np.array_equal(got.view(np.uint32), expected.view(np.uint32))


def test_round_trip_at_benchmark_size(cuda_ops):
    """Size-independent properties on a 4096 x 12288 linear, without the CPU: the device
    dequantiser equals the package's torch arithmetic on the same buffers bit for bit, the
    reconstruction error stays within one quantisation step (half from rounding the level, half
    from rounding the zero point), and the dense FP16 matrix
    multiplied by x agrees with the GEMV kernel on the packed form."""
    from lowbitlinear_b200 import _ops
    from lowbitlinear_b200.quantization import dequantize_int4, unpack_int4

    g = torch.Generator("cpu").manual_seed(21)
    weight = (torch.randn(4096, 12288, generator=g) * 0.02).half().to(cuda_ops)
    x = torch.randn(1, 12288, generator=g).half().to(cuda_ops)
    packed, scales, zeros = _ops.quantize_pack(weight)
    dense = _ops.dequantize(packed, scales, zeros, dtype=torch.float32)
    assert torch.equal(dense, dequantize_int4(unpack_int4(packed), scales, zeros, 64))
    error = (dense - weight.float()).abs()
    bound = scales.repeat_interleave(64, dim=1) * (1 + 1e-5)
    assert bool((error <= bound).all()), "reconstruction error exceeds one step"
    dense_fp16 = _ops.dequantize(packed, scales, zeros, dtype=torch.float16)
    assert torch.equal(dense_fp16, dense.half())
    y = _ops.w4a16_gemv_warp_vec(x, packed, scales, zeros, 64).float()
    expected = x.float() @ dense.t()
    torch.testing.assert_close(y, expected, atol=1e-2, rtol=1e-2)
