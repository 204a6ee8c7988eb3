"""Public module on CPU: reference path against the oracle and the reference's fixtures, state
handling, validation.  Adapted from NanjinLin/LowBitLinear tests/test_linear.py (MIT): the constructor, forward-error and
device cases follow that file closely (its parametrisations pin the API contract); the oracle,
the golden fixtures and the no-library CPU test are this repository's."""
import numpy as np
import pytest
import torch

from conftest import oracle_linear
from lowbitlinear_b200 import QuantizedLinear
from lowbitlinear_b200.linear import linear_int4_reference
from lowbitlinear_b200.quantization import pack_int4, quantize_int4


def _close_to_fp16_step(actual, expected):
    a, e = actual.float(), expected.float()
    return bool(((a - e).abs() <= torch.maximum(e.abs() * 2.0 ** -10, torch.tensor(2.0 ** -24))).all())


@pytest.mark.parametrize("m,n,k,group_size", [(1, 129, 256, 64), (16, 5, 65, 64), (5, 9, 70, 32), (9, 17, 129, 63), (1, 1, 1, 1)])
def test_reference_path_against_oracle(m, n, k, group_size):
    x = torch.randn(m, k, dtype=torch.float16)
    q, scales, zeros = quantize_int4(torch.randn(n, k), group_size)
    args = x, pack_int4(q), scales, zeros
    actual = linear_int4_reference(*args, group_size)
    assert actual.dtype == torch.float16 and actual.shape == (m, n)
    assert _close_to_fp16_step(actual, oracle_linear(*args, group_size))


def test_reference_path_reproduces_reference_outputs(golden_small):
    """Same torch operations on the same CPU values as the reference: identical bits."""
    for name, case in golden_small.items():
        gs = int(case["group_size"])
        y = linear_int4_reference(torch.from_numpy(case["x"]), torch.from_numpy(case["packed"]),
                                  torch.from_numpy(case["scales"]), torch.from_numpy(case["zeros"]), gs)
        assert np.array_equal(y.numpy().view(np.int16), case["y"].view(np.int16)), name


def test_tiny_config_end_to_end(golden_small):
    """Benchmark config 1: N=128, K=256, M=1, seed 0, through from_float and forward on CPU."""
    case = golden_small["tiny"]
    layer = QuantizedLinear.from_float(torch.from_numpy(case["weight"]))
    assert layer.packed_weight.shape == (128, 32) and layer.scales.shape == layer.zeros.shape == (128, 4)
    assert np.array_equal(layer.packed_weight.numpy(), case["packed"])
    assert np.array_equal(layer.zeros.numpy(), case["zeros"])
    assert np.array_equal(layer.scales.numpy(), case["scales"])
    y = layer(torch.from_numpy(case["x"]))
    assert y.shape == (1, 128) and y.dtype == torch.float16
    assert np.array_equal(y.numpy().view(np.int16), case["y"].view(np.int16))


@pytest.mark.parametrize("m,n,k,group_size", [(1, 129, 256, 64), (5, 9, 70, 64), (9, 17, 129, 63)])
@pytest.mark.parametrize("weight_dtype", [torch.float16, torch.float32])
def test_state_dict_roundtrip(m, n, k, group_size, weight_dtype):
    layer = QuantizedLinear.from_float(torch.randn(n, k, dtype=weight_dtype, requires_grad=True), group_size=group_size)
    x = torch.randn(m, k, dtype=torch.float16)
    expected = layer(x)
    assert layer.in_features == k and layer.out_features == n and layer.group_size == group_size
    assert expected.dtype == torch.float16 and expected.shape == (m, n)
    assert _close_to_fp16_step(expected, oracle_linear(x, layer.packed_weight, layer.scales, layer.zeros, group_size))
    assert set(layer.state_dict()) == {"packed_weight", "scales", "zeros"}
    assert list(layer.parameters()) == []
    assert all(not b.requires_grad for b in layer.buffers())
    restored = QuantizedLinear.from_float(torch.zeros(n, k), group_size=group_size)
    restored.load_state_dict(layer.state_dict())
    assert torch.equal(restored(x), expected)


def test_direct_constructor_with_partial_word():
    q, scales, zeros = quantize_int4(torch.randn(9, 70))
    packed = pack_int4(q)
    layer = QuantizedLinear(packed, scales, zeros, in_features=70)
    x = torch.randn(5, 70, dtype=torch.float16)
    assert _close_to_fp16_step(layer(x), oracle_linear(x, packed, scales, zeros))


@pytest.mark.parametrize("bits", [2, 3, 8, 16, True])
def test_unsupported_bits(bits):
    with pytest.raises(ValueError, match="bits=4"):
        QuantizedLinear.from_float(torch.ones(2, 64), bits=bits)


@pytest.mark.parametrize("x,error,match", [
    (None, TypeError, "Tensor"),
    (torch.ones(1, 64), TypeError, "dtype"),
    (torch.ones(1, 64, dtype=torch.bfloat16), TypeError, "dtype"),
    (torch.ones(64, dtype=torch.float16), ValueError, "2D"),
    (torch.ones(1, 32, dtype=torch.float16), ValueError, "incompatible K"),
    (torch.ones(0, 64, dtype=torch.float16), ValueError, "nonempty"),
    (torch.ones(1, 128, dtype=torch.float16)[:, ::2], ValueError, "contiguous"),
])
def test_invalid_forward_input(x, error, match):
    layer = QuantizedLinear.from_float(torch.ones(2, 64))
    with pytest.raises(error, match=match):
        layer(x)


@pytest.mark.parametrize("field,error,match", [
    ("packed_dtype", TypeError, "dtype"), ("packed_shape", ValueError, "shape"),
    ("scales_dtype", TypeError, "dtype"), ("zeros_dtype", TypeError, "dtype"),
    ("scales_shape", ValueError, "shape"), ("zeros_shape", ValueError, "shape"),
    ("group_size", ValueError, "group_size"),
])
def test_invalid_constructor_metadata(field, error, match):
    packed = torch.zeros(2, 8, dtype=torch.int32)
    scales = torch.ones(2, 1)
    zeros = torch.zeros(2, 1, dtype=torch.int32)
    group_size = 64
    if field == "packed_dtype":
        packed = packed.long()
    elif field == "packed_shape":
        packed = packed[:, :-1]
    elif field == "scales_dtype":
        scales = scales.half()
    elif field == "zeros_dtype":
        zeros = zeros.long()
    elif field == "scales_shape":
        scales = scales.repeat(1, 2)
    elif field == "zeros_shape":
        zeros = zeros.repeat(1, 2)
    elif field == "group_size":
        group_size = 0
    with pytest.raises(error, match=match):
        QuantizedLinear(packed, scales, zeros, group_size, in_features=64)


@pytest.mark.parametrize("in_features", [0, -1, True, 1.5, None, 65])
def test_invalid_in_features(in_features):
    with pytest.raises(ValueError, match="in_features|shape"):
        QuantizedLinear(torch.zeros(2, 8, dtype=torch.int32), torch.ones(2, 1),
                        torch.zeros(2, 1, dtype=torch.int32), in_features=in_features)


def test_forward_revalidates_changed_buffers():
    layer = QuantizedLinear.from_float(torch.ones(2, 64))
    layer.scales = torch.ones(2, 2)
    with pytest.raises(ValueError, match="shape"):
        layer(torch.ones(1, 64, dtype=torch.float16))


def test_cpu_forward_never_touches_the_native_library(monkeypatch):
    import lowbitlinear_b200.linear as linear_module

    def forbidden(*args, **kwargs):
        pytest.fail("the reference path must not load the native library")

    monkeypatch.setattr(linear_module, "load_cuda_extension", forbidden)
    for m, gs in ((1, 64), (16, 64), (5, 63)):
        layer = QuantizedLinear.from_float(torch.randn(5, 129), group_size=gs)
        x = torch.randn(m, 129, dtype=torch.float16)
        assert _close_to_fp16_step(layer(x), oracle_linear(x, layer.packed_weight, layer.scales, layer.zeros, gs))


@pytest.mark.gpu
def test_forward_device_mismatch(cuda_device):
    layer = QuantizedLinear.from_float(torch.ones(2, 64))
    with pytest.raises(ValueError, match="same device"):
        layer(torch.ones(1, 64, dtype=torch.float16, device=cuda_device))


@pytest.mark.gpu
def test_constructor_device_mismatch(cuda_device):
    with pytest.raises(ValueError, match="same device"):
        QuantizedLinear(torch.zeros(2, 8, dtype=torch.int32), torch.ones(2, 1, device=cuda_device),
                        torch.zeros(2, 1, dtype=torch.int32), in_features=64)


@pytest.mark.gpu
def test_module_to_cuda_moves_all_buffers(cuda_ops):
    layer = QuantizedLinear.from_float(torch.randn(9, 70)).to(cuda_ops)
    assert all(b.device == cuda_ops for b in layer.buffers())
    x = torch.randn(5, 70, device=cuda_ops, dtype=torch.float16)
    expected = oracle_linear(x, layer.packed_weight, layer.scales, layer.zeros, mma=True)
    torch.testing.assert_close(layer(x).cpu(), expected, atol=2e-3, rtol=1e-3)
