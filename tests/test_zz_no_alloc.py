"""The allocation-free GEMV entry point (`lbl_w4a16_gemv_noalloc`), called through the C ABI.

It exists for callers that cannot obtain device memory themselves -- a plugin that only receives
input and output pointers, or code running where cudaMalloc is forbidden -- so its split-K scratch
is a fixed array inside the library.  The test checks it against the regular entry point
(`lbl_w4a16_gemv`, caller-provided workspace) on two consecutive calls, because the second call
finds the scratch as the first one left it.  This file is collected last on purpose.
"""
import ctypes

import pytest
import torch

from conftest import ATOL, RTOL, oracle_linear, seeded_layer

pytestmark = pytest.mark.gpu


def _bind():
    from lowbitlinear_b200 import _ops
    from lowbitlinear_b200._extension import load_cuda_extension

    load_cuda_extension(required=True)
    lib = _ops._lib
    p, i64, i32, u32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_uint
    lib.lbl_w4a16_gemv_noalloc.restype = i32
    lib.lbl_w4a16_gemv_noalloc.argtypes = [p, p, p, p, p, i64, i64, i32, u32, i32, p]
    lib.lbl_w4a16_gemv_noalloc_scratch_bytes.restype = ctypes.c_size_t
    lib.lbl_w4a16_gemv_noalloc_scratch_bytes.argtypes = []
    return lib


def _call_noalloc(lib, x, packed, scales, zeros, flags=0):
    n, k = packed.shape[0], x.shape[1]
    y = torch.empty((1, n), dtype=torch.float16, device=x.device)  # outputs belong to the caller
    stream = torch.cuda.current_stream(x.device).cuda_stream
    rc = lib.lbl_w4a16_gemv_noalloc(x.data_ptr(), packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                    y.data_ptr(), n, k, 64, flags, x.device.index, stream)
    assert rc == 0, lib.lbl_last_error().decode()
    return y


@pytest.mark.parametrize("n,k", [(4096, 4096), (1000, 2048), (4096, 12288)])
def test_noalloc_gemv_matches_the_regular_entry_point_twice(n, k, cuda_ops):
    lib = _bind()
    assert lib.lbl_w4a16_gemv_noalloc_scratch_bytes() == 1 << 20
    x, packed, scales, zeros = seeded_layer(1, n, k, seed=n + k, device=cuda_ops)
    regular = torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(x, packed, scales, zeros, 64)
    first = _call_noalloc(lib, x, packed, scales, zeros)
    # Second call with other activations: the scratch still holds the first call's partial sums.
    x2 = (x * 0.5 + 0.25).half()
    regular2 = torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(x2, packed, scales, zeros, 64)
    second = _call_noalloc(lib, x2, packed, scales, zeros)
    torch.cuda.synchronize()
    torch.testing.assert_close(first, regular, atol=ATOL, rtol=RTOL)
    torch.testing.assert_close(second, regular2, atol=ATOL, rtol=RTOL)
    torch.testing.assert_close(first.cpu(), oracle_linear(x, packed, scales, zeros), atol=ATOL, rtol=RTOL)
    # Same inputs again give the same bits: the counters were left at zero.
    assert torch.equal(_call_noalloc(lib, x, packed, scales, zeros), first)


def test_noalloc_gemv_chain_with_programmatic_dependent_launch(cuda_ops):
    """With LBL_FLAG_PDL consecutive calls overlap in time on the GPU: a call starts fetching its
    weights while the previous one is still finishing, yet both use the one built-in scratch.
    What keeps that correct is that no call touches the scratch before the previous kernel has
    completed.  Eight calls back to back, two shapes alternating, no host synchronisation in
    between, three rounds; every output must equal that of the same call made alone."""
    lib = _bind()
    cases = [seeded_layer(1, 4096, 4096, seed=71, device=cuda_ops), seeded_layer(1, 1000, 2048, seed=72, device=cuda_ops)]
    alone = [_call_noalloc(lib, *case) for case in cases]
    torch.cuda.synchronize()
    for _ in range(3):
        chained = [_call_noalloc(lib, *cases[i % 2], flags=1) for i in range(8)]
        torch.cuda.synchronize()
        for i, y in enumerate(chained):
            assert torch.equal(y, alone[i % 2]), i


def test_noalloc_gemv_rejects_what_does_not_fit(cuda_ops):
    lib = _bind()
    n, k = 131072, 1024  # 64 KiB + 2 * N * 4 bytes is more than the built-in megabyte
    x = torch.zeros(1, k, dtype=torch.float16, device=cuda_ops)
    packed = torch.zeros(n, k // 8, dtype=torch.int32, device=cuda_ops)
    scales = torch.ones(n, k // 64, device=cuda_ops)
    zeros = torch.zeros(n, k // 64, dtype=torch.int32, device=cuda_ops)
    y = torch.empty(1, n, dtype=torch.float16, device=cuda_ops)
    rc = lib.lbl_w4a16_gemv_noalloc(x.data_ptr(), packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                    y.data_ptr(), n, k, 64, 0, cuda_ops.index, None)
    assert rc == -3 and b"built-in scratch" in lib.lbl_last_error()
    rc = lib.lbl_w4a16_gemv_noalloc(x.data_ptr(), packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                    y.data_ptr(), n, 192, 64, 0, cuda_ops.index, None)
    assert rc == -4  # K must be a multiple of 256 for the streaming kernel
