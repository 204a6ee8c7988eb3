"""M = 1 operator on the GPU, through the C ABI: every kernel path against the numpy oracle,
edge nibbles, the error contract, stream semantics, reproducibility and full benchmark sizes.
Adapted from NanjinLin/LowBitLinear tests/test_cuda_gemv.py (MIT): the shape list, the edge-nibble case
and the error table follow that file; forced paths, split-K, graph capture and the full-size
benchmark shapes are this repository's."""
import pytest
import torch

from conftest import ATOL, RTOL, assert_north_star_parity, oracle_linear, seeded_layer, torch_fp32_linear
from lowbitlinear_b200.quantization import pack_int4, quantize_int4

pytestmark = pytest.mark.gpu


@pytest.fixture
def gemv_inputs(cuda_ops):
    def make(n=129, k=256, seed=42):
        g = torch.Generator(device=cuda_ops).manual_seed(seed)
        x = torch.randn(1, k, device=cuda_ops, dtype=torch.float16, generator=g)
        w = torch.randn(n, k, device=cuda_ops, dtype=torch.float16, generator=g)
        q, scales, zeros = quantize_int4(w)
        return x, pack_int4(q), scales, zeros
    return make


# K % 256 == 0 takes the streaming kernel, everything else the masked kernel.
@pytest.mark.parametrize("n,k", [(1, 64), (3, 128), (127, 256), (128, 256), (129, 256), (1024, 1024),
                                 (257, 4096), (16, 512), (4096, 1536), (100, 768), (2048, 2048)])
@pytest.mark.parametrize("seed", [42, 123])
def test_gemv_against_oracle(n, k, seed, gemv_inputs):
    args = gemv_inputs(n, k, seed)
    actual = torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(*args, 64)
    assert actual.shape == (1, n) and actual.dtype == torch.float16 and actual.device == args[0].device
    torch.testing.assert_close(actual.cpu(), oracle_linear(*args), atol=ATOL, rtol=RTOL)


def test_extreme_nibbles_and_zero_points(cuda_ops):
    for n, k in ((5, 256), (5, 192)):
        q = (torch.arange(n * k, device=cuda_ops).reshape(n, k) % 16).byte()
        packed = pack_int4(q)
        scales = torch.full((n, k // 64), 0.125, device=cuda_ops)
        zeros = (torch.arange(n * (k // 64), device=cuda_ops).reshape(n, -1) % 2 * 15).int()
        x = torch.linspace(-1, 1, k, dtype=torch.float16, device=cuda_ops)[None, :]
        assert torch.any(packed < 0)  # negative words must still be read as unsigned nibbles
        args = x, packed, scales, zeros
        actual = torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(*args, 64)
        torch.testing.assert_close(actual.cpu(), oracle_linear(*args), atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("n,k", [(128, 64), (256, 512), (48, 4096)])
def test_integer_inputs_are_exact(n, k, cuda_ops):
    """Small integers survive every path exactly: all-ones gives K, and a one-hot activation
    returns a column of dequantised weights."""
    from lowbitlinear_b200 import QuantizedLinear

    layer = QuantizedLinear.from_float(torch.ones(n, k, device=cuda_ops))
    ones = torch.ones(1, k, dtype=torch.float16, device=cuda_ops)
    y = torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(ones, layer.packed_weight, layer.scales, layer.zeros, 64)
    assert torch.equal(y, torch.full_like(y, float(k)))
    q = torch.randint(0, 16, (n, k), device=cuda_ops, dtype=torch.uint8)
    scales = torch.full((n, k // 64), 0.5, device=cuda_ops)
    zeros = torch.randint(0, 16, (n, k // 64), device=cuda_ops, dtype=torch.int32)
    for column in (0, 1, 5, 63, k - 1):
        x = torch.zeros(1, k, dtype=torch.float16, device=cuda_ops)
        x[0, column] = 2.0
        y = torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(x, pack_int4(q), scales, zeros, 64)
        expected = (q[:, column].float() - zeros[:, column // 64].float()) * 0.5 * 2.0
        assert torch.equal(y[0].float(), expected), column


@pytest.mark.parametrize("path", ["generic", "gemv", "gemv_splitk"])
@pytest.mark.parametrize("m,n,k", [(1, 512, 1024), (1, 1000, 4096), (3, 130, 2048), (8, 64, 4096),
                                   (9, 48, 1024), (16, 200, 2048), (17, 96, 1024), (32, 40, 1024)])
def test_forced_paths_agree_with_oracle(path, m, n, k, cuda_ops):
    from lowbitlinear_b200 import _ops

    x, packed, scales, zeros = seeded_layer(m, n, k, seed=7 + m, std=1.0, device=cuda_ops)
    code = {v: c for c, v in _ops.PATH_NAMES.items()}[path]
    y, taken = _ops.linear_forced(x, packed, scales, zeros, code, op=0)
    if path == "generic":
        assert taken == _ops.PATH_GENERIC
    else:
        assert taken in (_ops.PATH_GEMV, _ops.PATH_GEMV_SPLITK)
        if path == "gemv_splitk":
            assert taken == _ops.PATH_GEMV_SPLITK
    torch.testing.assert_close(y.cpu(), oracle_linear(x, packed, scales, zeros), atol=ATOL, rtol=RTOL)


def test_split_k_is_bit_reproducible_and_leaves_scratch_clean(cuda_ops):
    from lowbitlinear_b200 import _ops

    x, packed, scales, zeros = seeded_layer(1, 4096, 4096, seed=3, device=cuda_ops)
    first, taken = _ops.linear_forced(x, packed, scales, zeros, _ops.PATH_GEMV_SPLITK, op=0)
    assert taken == _ops.PATH_GEMV_SPLITK
    for _ in range(5):
        again, _ = _ops.linear_forced(x, packed, scales, zeros, _ops.PATH_GEMV_SPLITK, op=0)
        assert torch.equal(first, again)
    unsplit, _ = _ops.linear_forced(x, packed, scales, zeros, _ops.PATH_GEMV, op=0)
    torch.testing.assert_close(first, unsplit, atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("name,n,k,seed", [("qkv", 6144, 4096, 0), ("o", 4096, 4096, 1),
                                           ("gate_up", 24576, 4096, 2), ("down", 4096, 12288, 3)])
def test_decode_shapes_meet_the_benchmark_tolerance(name, n, k, seed, cuda_ops):
    """Benchmark config 2 at full size: W ~ N(0, 0.02), x ~ N(0, 1), quantised on CPU."""
    from lowbitlinear_b200 import QuantizedLinear

    x, packed, scales, zeros = seeded_layer(1, n, k, seed=seed, device=cuda_ops)
    layer = QuantizedLinear(packed, scales, zeros, in_features=k)
    y = layer(x)
    assert_north_star_parity(y, torch_fp32_linear(x, packed, scales, zeros))
    if name in ("o", "down"):  # sizes the numpy oracle finishes in seconds
        assert_north_star_parity(y, oracle_linear(x, packed, scales, zeros))
    # Size-independent property, linearity in x: f(2x) = 2 f(x) up to the last FP16 bit
    # (activations below 2^-10 lose a bit in the operand scaled by 1/16, nothing else rounds
    # differently under a factor of two).
    torch.testing.assert_close(layer(x * 2), y * 2, atol=1e-3, rtol=1e-3)


def test_programmatic_dependent_launch_gives_identical_results(cuda_ops):
    from lowbitlinear_b200 import _ops

    layers = [seeded_layer(1, 4096, 4096, seed=s, device=cuda_ops) for s in range(4)]
    plain = [torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(*args, 64) for args in layers]
    _ops.set_programmatic_dependent_launch(True)
    try:
        for _ in range(3):
            chained = [torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(*args, 64) for args in layers]
    finally:
        _ops.set_programmatic_dependent_launch(False)
    for a, b in zip(plain, chained):
        assert torch.equal(a, b)


@pytest.mark.parametrize("bad,match", [
    ("x_dtype", "FP16"), ("x_rank", "shape"), ("m", "shape"), ("k_tail", "divisible"),
    ("empty_k", "divisible"), ("packed_dtype", "int32"), ("packed_rank", "2D"),
    ("packed_shape", "packed weight shape"), ("scales_dtype", "FP32"),
    ("scales_shape", "scales or zeros shape"), ("zeros_dtype", "int32"),
    ("zeros_shape", "scales or zeros shape"), ("cpu_metadata", "CUDA"),
    ("group_size", "group_size=64"), ("empty_n", "Invalid N or K"),
    ("noncontiguous_x", "contiguous"), ("noncontiguous_packed", "contiguous"),
    ("noncontiguous_scales", "contiguous"), ("noncontiguous_zeros", "contiguous"),
])
def test_rejects_invalid_inputs(bad, match, gemv_inputs):
    args = list(gemv_inputs())
    group_size = 64
    if bad == "x_dtype":
        args[0] = args[0].float()
    elif bad == "x_rank":
        args[0] = args[0].squeeze(0)
    elif bad == "m":
        args[0] = args[0].repeat(2, 1)
    elif bad == "k_tail":
        args[0] = args[0][:, :65].contiguous()
    elif bad == "empty_k":
        args[0] = args[0][:, :0]
    elif bad == "packed_dtype":
        args[1] = args[1].long()
    elif bad == "packed_rank":
        args[1] = args[1].flatten()
    elif bad == "packed_shape":
        args[1] = args[1][:, :-1].contiguous()
    elif bad == "scales_dtype":
        args[2] = args[2].half()
    elif bad == "scales_shape":
        args[2] = args[2][:, :-1].contiguous()
    elif bad == "zeros_dtype":
        args[3] = args[3].long()
    elif bad == "zeros_shape":
        args[3] = args[3][:, :-1].contiguous()
    elif bad == "cpu_metadata":
        args[2] = args[2].cpu()
    elif bad == "group_size":
        group_size = 32
    elif bad == "empty_n":
        args[1:] = [t[:0] for t in args[1:]]
    elif bad.startswith("noncontiguous_"):
        index = ["noncontiguous_x", "noncontiguous_packed", "noncontiguous_scales", "noncontiguous_zeros"].index(bad)
        t = args[index]
        args[index] = torch.zeros(t.shape[0], t.shape[1] * 2, device=t.device, dtype=t.dtype)[:, ::2]
        assert not args[index].is_contiguous()
    with pytest.raises(RuntimeError, match=match):
        torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(*args, group_size)


def test_rejects_cpu_input(gemv_inputs):
    args = [t.cpu() for t in gemv_inputs()]
    with pytest.raises(NotImplementedError, match="CPU"):
        torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(*args, 64)


def test_rejects_misaligned_contiguous_input(gemv_inputs):
    x, packed, scales, zeros = gemv_inputs()
    storage = torch.empty(x.numel() + 1, device=x.device, dtype=x.dtype)
    misaligned = storage[1:].view_as(x).copy_(x)
    assert misaligned.is_contiguous() and misaligned.data_ptr() % 16 != 0
    with pytest.raises(RuntimeError, match="16-byte aligned"):
        torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(misaligned, packed, scales, zeros, 64)


@pytest.mark.parametrize("n,k", [(129, 256), (512, 4096)])
def test_uses_current_stream(n, k, gemv_inputs):
    args = gemv_inputs(n, k)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        x = args[0] * 2
        actual = torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(x, *args[1:], 64)
        consumed = actual + 1
    torch.cuda.current_stream().wait_stream(stream)
    expected = oracle_linear(x, *args[1:]) + 1
    torch.testing.assert_close(consumed.cpu(), expected, atol=ATOL, rtol=RTOL)


def test_cuda_graph_capture_and_replay(cuda_ops):
    """The whole call is capturable: no allocation by the library, no host synchronisation."""
    x, packed, scales, zeros = seeded_layer(1, 4096, 4096, seed=11, device=cuda_ops)
    expected = torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(x, packed, scales, zeros, 64)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(x, packed, scales, zeros, 64)  # warm the scratch cache
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph, stream=side):
        out = torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(x, packed, scales, zeros, 64)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, expected)
