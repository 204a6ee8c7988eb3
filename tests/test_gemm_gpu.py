"""Any-shape operator on the GPU, through the C ABI: masked tails, empty dimensions, exactness
and operand-policy cases, the tensor-core path at prefill sizes, error contract, streams.
Adapted from NanjinLin/LowBitLinear tests/test_cute_w4a16_gemm.py (MIT): the shape grid, the
exactness and operand-policy cases and the error tables follow that file; the oracle, the forced
kernel paths and the full-size benchmark shapes are this repository's."""
import pytest
import torch

from conftest import (ATOL, RTOL, assert_north_star_parity, expected_for_operator, oracle_linear, seeded_layer,
                      torch_fp32_linear)
from lowbitlinear_b200.quantization import pack_int4, quantize_int4

pytestmark = pytest.mark.gpu

SHAPES = [
    (1, 1, 1), (4, 9, 7), (4, 8, 8), (4, 8, 63), (32, 32, 64), (17, 23, 65), (5, 9, 70),
    (6, 10, 71), (31, 33, 127), (6, 10, 128), (33, 37, 129), (64, 65, 130), (79, 70, 192),
    (32, 64, 512), (7, 35, 4096),
    # both sides of 64-wide tile boundaries, with K tails
    (63, 63, 63), (65, 63, 64), (63, 65, 65), (65, 65, 129), (127, 129, 192),
    # shapes the streaming kernel serves under this operator (K % 256 == 0, M <= 32)
    (2, 100, 256), (8, 129, 512), (16, 257, 1024), (31, 48, 768),
]


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("real_quant", [False, True], ids=["synthetic-int4", "real-quantization"])
def test_gemm_against_oracle(m, n, k, real_quant, cuda_ops):
    x = torch.randn(m, k, device=cuda_ops, dtype=torch.float16)
    if real_quant:
        q, scales, zeros = quantize_int4(torch.randn(n, k, device=cuda_ops, dtype=torch.float16))
    else:
        q = torch.randint(0, 16, (n, k), device=cuda_ops, dtype=torch.uint8)
        q[:, 7::8] = 15  # top nibble set: negative packed words
        groups = (k + 63) // 64
        scales = torch.rand(n, groups, device=cuda_ops) * .08 + .01
        zeros = torch.randint(0, 16, (n, groups), device=cuda_ops, dtype=torch.int32)
    args = x, pack_int4(q), scales, zeros
    actual = torch.ops.lowbitlinear_cute_w4a16.gemm(*args)
    assert actual.shape == (m, n) and actual.dtype == torch.float16
    assert actual.device == x.device and torch.isfinite(actual).all()
    torch.testing.assert_close(actual.cpu(), expected_for_operator(*args), atol=ATOL, rtol=RTOL)
    # Whatever the kernel, the result is within the benchmark tolerance of the FP32 reference
    # path (a relative L2 norm needs more than a handful of outputs to be meaningful).
    if m * n >= 256:
        assert_north_star_parity(actual, oracle_linear(*args))


@pytest.mark.parametrize("m,n,k", [(32, 32, 64), (17, 23, 129), (65, 65, 129), (4, 64, 512), (130, 256, 512)])
def test_exact_multistage_accumulation(m, n, k, cuda_ops):
    x = torch.ones(m, k, device=cuda_ops, dtype=torch.float16)
    packed = pack_int4(torch.full((n, k), 5, device=cuda_ops, dtype=torch.uint8))
    scales = torch.full((n, (k + 63) // 64), .25, device=cuda_ops)
    zeros = torch.full_like(scales, 3, dtype=torch.int32)
    actual = torch.ops.lowbitlinear_cute_w4a16.gemm(x, packed, scales, zeros)
    torch.testing.assert_close(actual, torch.full_like(actual, k * .5), rtol=0, atol=0)


@pytest.mark.parametrize("m,n,k", [(33, 65, 129), (65, 129, 129), (5, 64, 256), (200, 256, 256)])
def test_one_hot_mapping(m, n, k, cuda_ops):
    """Each weight row selects one column of X: checks the (row, column) mapping of every path,
    including the swizzled shared-memory tiles of the tensor-core kernel."""
    x = (torch.arange(m * k, device=cuda_ops).reshape(m, k) % 101).half()
    q = torch.zeros(n, k, dtype=torch.uint8, device=cuda_ops)
    positions = (torch.arange(n, device=cuda_ops) * 2) % k
    q[torch.arange(n, device=cuda_ops), positions] = 1
    scales = torch.ones(n, (k + 63) // 64, device=cuda_ops)
    zeros = torch.zeros_like(scales, dtype=torch.int32)
    actual = torch.ops.lowbitlinear_cute_w4a16.gemm(x, pack_int4(q), scales, zeros)
    torch.testing.assert_close(actual, x[:, positions], rtol=0, atol=0)


def test_fp16_operand_policy_of_the_masked_kernel(cuda_ops):
    """Scales 1.0004 and 1.03 tell FP16-rounded weights from FP32 weights."""
    x = torch.ones(1, 65, device=cuda_ops, dtype=torch.float16)
    q = torch.ones(1, 65, device=cuda_ops, dtype=torch.uint8)
    scales = torch.tensor([[1.0004, 1.03]], device=cuda_ops)
    zeros = torch.zeros(1, 2, device=cuda_ops, dtype=torch.int32)
    args = x, pack_int4(q), scales, zeros
    expected = oracle_linear(*args, mma=True)
    assert not torch.equal(expected, oracle_linear(*args))
    torch.testing.assert_close(torch.ops.lowbitlinear_cute_w4a16.gemm(*args).cpu(), expected, rtol=0, atol=0)


def test_fp16_operand_policy_of_the_tensor_core_kernel(cuda_ops):
    """Same distinction at a shape the tcgen05 kernel serves: every product is exact, so the
    result must equal the FP16-rounded-weight oracle bit for bit."""
    from lowbitlinear_b200 import _ops

    m, n, k = 130, 256, 256
    x = torch.zeros(m, k, device=cuda_ops, dtype=torch.float16)
    x[torch.arange(m), torch.arange(m) % k] = 1.0  # one-hot rows pick single weights
    q = torch.randint(0, 16, (n, k), device=cuda_ops, dtype=torch.uint8)
    scales = torch.rand(n, k // 64, device=cuda_ops) * 0.1 + 1.0
    zeros = torch.randint(0, 16, (n, k // 64), device=cuda_ops, dtype=torch.int32)
    args = x, pack_int4(q), scales, zeros
    y, taken = _ops.linear_forced(*args, _ops.PATH_GEMM_TC)
    assert taken == _ops.PATH_GEMM_TC
    assert torch.equal(y.cpu(), oracle_linear(*args, mma=True))


@pytest.mark.parametrize("m,n,k", [(1, 256, 256), (127, 256, 512), (128, 512, 256), (129, 256, 1024),
                                   (256, 256, 2048), (257, 768, 768), (300, 512, 4096), (513, 256, 1536)])
def test_tensor_core_path_against_oracle(m, n, k, cuda_ops):
    from lowbitlinear_b200 import _ops

    x, packed, scales, zeros = seeded_layer(m, n, k, seed=m + n + k, std=1.0, device=cuda_ops)
    y, taken = _ops.linear_forced(x, packed, scales, zeros, _ops.PATH_GEMM_TC)
    assert taken == _ops.PATH_GEMM_TC
    torch.testing.assert_close(y.cpu(), oracle_linear(x, packed, scales, zeros, mma=True), atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("m,n,k", [(1, 128, 256), (9, 128, 512), (16, 256, 1024), (17, 384, 2048), (33, 4096, 4096),
                                   (64, 1024, 12288), (100, 640, 768), (128, 2048, 4096)])
def test_small_m_tensor_core_path_against_oracle(m, n, k, cuda_ops):
    """tcgen05 GEMM with the weights on the M side of the MMA (M <= 128): FP16-rounded weights as
    in the reference GEMM; K cut into slices that meet in the scratch, bit-reproducible; without
    scratch one CTA per row block gives the same answer within the tolerance."""
    import ctypes

    from lowbitlinear_b200 import _ops
    from lowbitlinear_b200._extension import native

    x, packed, scales, zeros = seeded_layer(m, n, k, seed=m + n + k, std=1.0, device=cuda_ops)
    expected = oracle_linear(x, packed, scales, zeros, mma=True)
    # Unit-variance weights: outputs of magnitude sqrt(K), where one FP16 step is 2e-3 .. 8e-3 and
    # the order of the FP32 additions decides the last bit; the absolute tolerance follows.
    atol = ATOL * (4 if k > 4096 else 1)
    runs = [_ops.linear_forced(x, packed, scales, zeros, _ops.PATH_GEMM_TC_SMALL) for _ in range(3)]
    assert all(taken == _ops.PATH_GEMM_TC_SMALL for _, taken in runs)
    assert torch.equal(runs[0][0], runs[1][0]) and torch.equal(runs[0][0], runs[2][0])
    torch.testing.assert_close(runs[0][0].cpu(), expected, atol=atol, rtol=RTOL)
    y = torch.empty(m, n, dtype=torch.float16, device=cuda_ops)
    rc = native().lbl_w4a16_linear(x.data_ptr(), packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                   y.data_ptr(), m, n, k, 1, _ops.PATH_GEMM_TC_SMALL, None, 0, 0,
                                   cuda_ops.index, torch.cuda.current_stream().cuda_stream, None)
    assert rc == 0
    torch.testing.assert_close(y.cpu(), expected, atol=atol, rtol=RTOL)


@pytest.mark.parametrize("m,n,k", [(1, 128, 256), (16, 256, 256), (130, 256, 512), (192, 512, 1024), (200, 256, 256),
                                   (64, 4096, 4096), (500, 768, 2048), (385, 384, 4096), (1024, 1024, 1024)])
def test_tensor_memory_path_against_oracle(m, n, k, cuda_ops):
    """tcgen05 GEMM with the weights handed to the MMA through tensor memory: FP16-rounded weights as
    in the reference GEMM, any M (tiles of up to 192 tokens), N % 128 == 0 with a half-empty last
    row block, K cut into slices that meet in the scratch when there is one token tile."""
    from lowbitlinear_b200 import _ops

    x, packed, scales, zeros = seeded_layer(m, n, k, seed=m + n + k, std=1.0, device=cuda_ops)
    expected = oracle_linear(x, packed, scales, zeros, mma=True)
    atol = ATOL * (4 if k > 2048 else 1)  # unit-variance weights: an FP16 step of the outputs is up to 8e-3
    scratch = torch.zeros(max(16, _ops.workspace_bytes(m, n, k, _ops.PATH_GEMM_WT)), dtype=torch.uint8, device=cuda_ops)
    runs = [_ops.linear_forced(x, packed, scales, zeros, _ops.PATH_GEMM_WT, workspace=scratch) for _ in range(3)]
    assert all(taken == _ops.PATH_GEMM_WT for _, taken in runs)
    assert torch.equal(runs[0][0], runs[1][0]) and torch.equal(runs[0][0], runs[2][0])
    torch.testing.assert_close(runs[0][0].cpu(), expected, atol=atol, rtol=RTOL)
    unsliced, _ = _ops.linear_forced(x, packed, scales, zeros, _ops.PATH_GEMM_WT,
                                     workspace=torch.zeros(16, dtype=torch.uint8, device=cuda_ops))
    torch.testing.assert_close(unsliced.cpu(), expected, atol=atol, rtol=RTOL)


@pytest.mark.parametrize("m,n,k", [(1, 256, 256), (16, 512, 256), (130, 256, 512), (512, 1024, 1024), (300, 512, 256),
                                   (700, 1536, 2048), (1100, 768, 1024), (513, 256, 4096)])
def test_paired_tensor_core_path_against_oracle(m, n, k, cuda_ops):
    """tcgen05 GEMM on pairs of CTAs (cta_group::2): 512 tokens x 256 weight rows per pair, each CTA
    dequantising half of the weight rows; token tails, several tiles, bit-reproducible."""
    from lowbitlinear_b200 import _ops

    x, packed, scales, zeros = seeded_layer(m, n, k, seed=m + n + k, std=1.0, device=cuda_ops)
    runs = [_ops.linear_forced(x, packed, scales, zeros, _ops.PATH_GEMM_TC_PAIR) for _ in range(3)]
    assert all(taken == _ops.PATH_GEMM_TC_PAIR for _, taken in runs)
    assert torch.equal(runs[0][0], runs[1][0]) and torch.equal(runs[0][0], runs[2][0])
    atol = ATOL * (4 if k > 2048 else 1)
    torch.testing.assert_close(runs[0][0].cpu(), oracle_linear(x, packed, scales, zeros, mma=True), atol=atol, rtol=RTOL)
    # Same arithmetic as the single-CTA kernel (FP16-rounded weights, FP32 accumulation in K order).
    single, _ = _ops.linear_forced(x, packed, scales, zeros, _ops.PATH_GEMM_TC)
    assert torch.equal(single, runs[0][0])


def test_fp16_operand_policy_of_the_tensor_memory_kernel(cuda_ops):
    """One-hot activations pick single weights: the result must equal the FP16-rounded-weight oracle
    bit for bit (and differ from the FP32-weight one)."""
    from lowbitlinear_b200 import _ops

    m, n, k = 200, 256, 256
    x = torch.zeros(m, k, device=cuda_ops, dtype=torch.float16)
    x[torch.arange(m), torch.arange(m) % k] = 1.0
    q = torch.randint(0, 16, (n, k), device=cuda_ops, dtype=torch.uint8)
    scales = torch.rand(n, k // 64, device=cuda_ops) * 0.1 + 1.0
    zeros = torch.randint(0, 16, (n, k // 64), device=cuda_ops, dtype=torch.int32)
    args = x, pack_int4(q), scales, zeros
    y, taken = _ops.linear_forced(*args, _ops.PATH_GEMM_WT)
    assert taken == _ops.PATH_GEMM_WT
    assert torch.equal(y.cpu(), oracle_linear(*args, mma=True))


def test_small_m_tensor_core_path_rejects_other_shapes(cuda_ops):
    from lowbitlinear_b200 import _ops

    for m, n, k in ((129, 256, 256), (8, 192, 256), (8, 256, 320)):
        x, packed, scales, zeros = seeded_layer(m, n, k, seed=1, device=cuda_ops)
        with pytest.raises(RuntimeError, match="small-M tensor-core GEMM cannot serve"):
            _ops.linear_forced(x, packed, scales, zeros, _ops.PATH_GEMM_TC_SMALL)


@pytest.mark.parametrize("name,n,k,seed", [("gate_up", 24576, 4096, 2), ("down", 4096, 12288, 3)])
@pytest.mark.parametrize("m", [16, 64, 128, 2048])
def test_prefill_shapes_meet_the_benchmark_tolerance(name, n, k, seed, m, cuda_ops):
    """Benchmark config 4 at full size, checked against an FP32 evaluation on the GPU
    (TF32 off) and, on a slice of rows, against the numpy oracle."""
    from lowbitlinear_b200 import QuantizedLinear, _ops

    x, packed, scales, zeros = seeded_layer(m, n, k, seed=seed, device=cuda_ops)
    small = m <= 32 or (m <= 128 and n < 16384)
    large = _ops.PATH_GEMM_TC_PAIR if m >= 512 else _ops.PATH_GEMM_TC
    # A wide shape whose whole activation operand fits the streaming kernel's shared memory still
    # streams at 16 rows.
    streams = m <= 16 and n >= 16384 and m * k * 2 <= 128 * 1024
    assert _ops.select_path(m, n, k) == (_ops.PATH_GEMV if streams else _ops.PATH_GEMM_TC_SMALL if small else large)
    layer = QuantizedLinear(packed, scales, zeros, in_features=k)
    y = layer(x)
    assert_north_star_parity(y, torch_fp32_linear(x, packed, scales, zeros))
    rows = slice(0, 512)
    assert_north_star_parity(y[:8, rows], oracle_linear(x[:8], packed[rows], scales[rows], zeros[rows]))
    # Size-independent properties: doubling X doubles Y (to the last FP16 bit), and a zero X
    # gives a zero Y.
    torch.testing.assert_close(layer(x * 2), y * 2, atol=1e-3, rtol=1e-3)
    assert torch.count_nonzero(layer(torch.zeros_like(x))) == 0


DECODE_SHAPES = {"qkv": (6144, 4096, 0), "o": (4096, 4096, 1), "gate_up": (24576, 4096, 2), "down": (4096, 12288, 3)}
CROSSOVER = [(name, m) for name in DECODE_SHAPES for m in (2, 4, 8, 32)] + \
            [(name, m) for name in ("qkv", "o") for m in (16, 64)] + [("gate_up", 12), ("gate_up", 16)]


@pytest.mark.parametrize("name,m", CROSSOVER)
def test_crossover_shapes_meet_the_benchmark_tolerance_on_every_path(name, m, cuda_ops):
    """Benchmark config 3 at full size: 2 <= M <= 64 on the four decode shapes, through
    QuantizedLinear.forward (the dispatcher's pick) and with each kernel that can serve the shape
    forced -- the streaming kernel, the small-M tcgen05 GEMM and the large tcgen05 GEMM -- every
    result against an FP32 evaluation on the GPU and, on a slice of rows, the numpy oracle."""
    from lowbitlinear_b200 import QuantizedLinear, _ops

    n, k, seed = DECODE_SHAPES[name]
    x, packed, scales, zeros = seeded_layer(m, n, k, seed=seed, device=cuda_ops)
    expected = torch_fp32_linear(x, packed, scales, zeros)
    rows = slice(n - 256, n)
    oracle_rows = oracle_linear(x, packed[rows], scales[rows], zeros[rows])
    layer = QuantizedLinear(packed, scales, zeros, in_features=k)
    results = {"forward": layer(x)}
    paths = [_ops.PATH_GEMM_TC_SMALL, _ops.PATH_GEMM_TC]
    if m <= 32:
        paths.append(_ops.PATH_GEMV)
    for path in paths:
        y, taken = _ops.linear_forced(x, packed, scales, zeros, path)
        assert taken in ((_ops.PATH_GEMV, _ops.PATH_GEMV_SPLITK) if path == _ops.PATH_GEMV else (path,))
        results[_ops.PATH_NAMES[path]] = y
    for label, y in results.items():
        assert y.shape == (m, n), label
        assert_north_star_parity(y, expected)
        assert_north_star_parity(y[:, rows], oracle_rows)
    picked = _ops.PATH_NAMES[_ops.select_path(m, n, k)]
    picked = "gemv" if picked == "gemv_splitk" else picked
    if picked == "gemv" and _ops.select_path(m, n, k) == _ops.PATH_GEMV_SPLITK:
        # Forced and automatic plans may split K differently: same value up to the last bit.
        torch.testing.assert_close(results["forward"], results[picked], atol=ATOL, rtol=RTOL)
    else:
        assert torch.equal(results["forward"], results[picked])


@pytest.mark.parametrize("name", ["gate_up", "down"])
@pytest.mark.parametrize("m", [512, 8192])
def test_prefill_sweep_ends_meet_the_benchmark_tolerance(name, m, cuda_ops):
    """Benchmark config 4 at the sizes with 2 and 32 tiles of 256 rows (M = 128 and 2048 are above)."""
    from lowbitlinear_b200 import QuantizedLinear, _ops

    n, k, seed = DECODE_SHAPES[name]
    x, packed, scales, zeros = seeded_layer(m, n, k, seed=seed + 10, device=cuda_ops)
    # Down at M = 512 is 32 tiles of 256 x 256 for 148 SMs: the tensor-memory GEMM with K cut into
    # slices takes it; everything else here fills the SMs with the large tiles.
    tiles = (n // 256) * ((m + 255) // 256)
    few_tiles = 3 * tiles <= 148 or (2 * tiles <= 148 and k >= 8192)
    assert _ops.select_path(m, n, k) == (_ops.PATH_GEMM_WT if few_tiles else _ops.PATH_GEMM_TC_PAIR)
    layer = QuantizedLinear(packed, scales, zeros, in_features=k)
    y = layer(x)
    assert_north_star_parity(y, torch_fp32_linear(x, packed, scales, zeros))
    rows = slice(n - 256, n)
    picks = torch.tensor([0, 1, 255, 256, m // 2 + 3, m - 129, m - 2, m - 1], device=cuda_ops)
    assert_north_star_parity(y[picks][:, rows], oracle_linear(x[picks], packed[rows], scales[rows], zeros[rows]))
    assert torch.count_nonzero(layer(torch.zeros_like(x))) == 0


@pytest.mark.parametrize("m,n,k", [(32, 32, 0), (0, 32, 65), (32, 0, 65), (0, 0, 0)])
def test_empty_dimensions(m, n, k, cuda_ops):
    x = torch.empty(m, k, device=cuda_ops, dtype=torch.float16)
    packed = torch.empty(n, (k + 7) // 8, device=cuda_ops, dtype=torch.int32)
    scales = torch.empty(n, (k + 63) // 64, device=cuda_ops)
    zeros = torch.empty_like(scales, dtype=torch.int32)
    actual = torch.ops.lowbitlinear_cute_w4a16.gemm(x, packed, scales, zeros)
    assert actual.shape == (m, n) and actual.dtype == x.dtype and actual.device == x.device
    assert torch.count_nonzero(actual) == 0


@pytest.fixture
def small_inputs(cuda_ops):
    def make(n=129, k=256, seed=42):
        g = torch.Generator(device=cuda_ops).manual_seed(seed)
        x = torch.randn(1, k, device=cuda_ops, dtype=torch.float16, generator=g)
        w = torch.randn(n, k, device=cuda_ops, dtype=torch.float16, generator=g)
        q, scales, zeros = quantize_int4(w)
        return x, pack_int4(q), scales, zeros
    return make


@pytest.mark.parametrize("index", range(4), ids=["x", "packed", "scales", "zeros"])
@pytest.mark.parametrize("bad", ["dtype", "rank", "noncontiguous", "cpu"])
def test_invalid_tensor_contract(index, bad, small_inputs):
    args = list(small_inputs())
    tensor = args[index]
    if bad == "dtype":
        args[index] = tensor.double()
        match = ["float16", "int32", "float32", "int32"][index]
    elif bad == "rank":
        args[index] = tensor.flatten()
        match = "2D"
    elif bad == "noncontiguous":
        args[index] = torch.zeros(tensor.shape[0], tensor.shape[1] * 2, device=tensor.device, dtype=tensor.dtype)[:, ::2]
        assert not args[index].is_contiguous()
        match = "contiguous"
    else:
        args[index] = tensor.cpu()
        match = "CUDA"
    with pytest.raises(RuntimeError, match=match):
        torch.ops.lowbitlinear_cute_w4a16.gemm(*args)


@pytest.mark.parametrize("index,match", [(1, "packed_w must have shape"), (2, "scales must have shape"), (3, "zeros must have shape")])
def test_invalid_metadata_shape(index, match, small_inputs):
    args = list(small_inputs())
    args[index] = args[index][:, :-1].contiguous()
    with pytest.raises(RuntimeError, match=match):
        torch.ops.lowbitlinear_cute_w4a16.gemm(*args)


@pytest.mark.parametrize("m,n,k", [(1, 37, 256), (200, 256, 512)])
def test_uses_current_stream(m, n, k, cuda_ops):
    x, packed, scales, zeros = seeded_layer(m, n, k, seed=5, std=1.0, device=cuda_ops)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        x2 = x * 2
        actual = torch.ops.lowbitlinear_cute_w4a16.gemm(x2, packed, scales, zeros)
        consumed = actual + 1
    torch.cuda.current_stream().wait_stream(stream)
    expected = expected_for_operator(x2, packed, scales, zeros) + 1
    torch.testing.assert_close(consumed.cpu(), expected, atol=ATOL, rtol=RTOL)


def test_misaligned_views_fall_back_to_the_masked_kernel(cuda_ops):
    """Vector loads need 16-byte alignment; an offset view must still give the right answer."""
    x, packed, scales, zeros = seeded_layer(4, 64, 512, seed=9, std=1.0, device=cuda_ops)
    storage = torch.empty(x.numel() + 1, device=x.device, dtype=x.dtype)
    shifted = storage[1:].view_as(x).copy_(x)
    assert shifted.data_ptr() % 16 != 0
    actual = torch.ops.lowbitlinear_cute_w4a16.gemm(shifted, packed, scales, zeros)
    torch.testing.assert_close(actual.cpu(), oracle_linear(x, packed, scales, zeros, mma=True), atol=ATOL, rtol=RTOL)
