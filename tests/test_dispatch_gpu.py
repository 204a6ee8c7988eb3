"""forward() picks the operator the reference picks and the selected native kernel really runs.
Mirrors the intent of the reference's tests/test_api_dispatch.py:16-59."""
from unittest.mock import Mock

import pytest
import torch

import lowbitlinear_b200.linear as linear_module
from conftest import ATOL, RTOL, expected_for_operator, oracle_linear
from lowbitlinear_b200 import QuantizedLinear

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k,route", [
    (1, 128, 64, "gemv"), (1, 256, 256, "gemv"), (1, 4096, 4096, "gemv"),
    (1, 127, 256, "gemm"), (1, 129, 256, "gemm"), (1, 128, 65, "gemm"), (16, 128, 64, "gemm"),
    (1, 1, 1, "gemm"), (5, 9, 70, "gemm"), (9, 17, 129, "gemm"), (256, 256, 256, "gemm"),
])
def test_cuda_dispatch_executes_selected_operator(m, n, k, route, cuda_ops, monkeypatch):
    layer = QuantizedLinear.from_float(torch.randn(n, k, device=cuda_ops, dtype=torch.float16))
    x = torch.randn(m, k, device=cuda_ops, dtype=torch.float16)
    if route == "gemm":
        expected = expected_for_operator(x, layer.packed_weight, layer.scales, layer.zeros)
    else:
        expected = oracle_linear(x, layer.packed_weight, layer.scales, layer.zeros)
    gemv = Mock(wraps=torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec)
    gemm = Mock(wraps=torch.ops.lowbitlinear_cute_w4a16.gemm)
    monkeypatch.setattr(torch.ops.lowbitlinear_ext, "w4a16_gemv_warp_vec", gemv)
    monkeypatch.setattr(torch.ops.lowbitlinear_cute_w4a16, "gemm", gemm)

    def forbidden(*args, **kwargs):
        pytest.fail("CUDA tensors with group_size 64 must run a native kernel")

    monkeypatch.setattr(linear_module, "linear_int4_reference", forbidden)
    actual = layer(x)
    selected, other = (gemv, gemm) if route == "gemv" else (gemm, gemv)
    selected.assert_called_once()
    other.assert_not_called()
    assert selected.call_args.args[0] is x
    assert selected.call_args.args[1] is layer.packed_weight
    assert len(selected.call_args.args) == (5 if route == "gemv" else 4)
    if route == "gemv":
        assert selected.call_args.args[4] == 64
    torch.testing.assert_close(actual.cpu(), expected, atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("m,group_size", [(1, 32), (5, 63)])
def test_other_group_sizes_take_the_reference_path_on_cuda(m, group_size, cuda_device, monkeypatch):
    layer = QuantizedLinear.from_float(torch.randn(5, 129, device=cuda_device), group_size=group_size)
    x = torch.randn(m, 129, device=cuda_device, dtype=torch.float16)
    expected = oracle_linear(x, layer.packed_weight, layer.scales, layer.zeros, group_size)
    reference = Mock(wraps=linear_module.linear_int4_reference)
    monkeypatch.setattr(linear_module, "linear_int4_reference", reference)

    def forbidden(*args, **kwargs):
        pytest.fail("the reference path must not need the native library")

    monkeypatch.setattr(linear_module, "load_cuda_extension", forbidden)
    torch.testing.assert_close(layer(x).cpu(), expected, atol=ATOL, rtol=RTOL)
    reference.assert_called_once()
