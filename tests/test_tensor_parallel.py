"""N-split and K-split sharding.  The host logic runs as two gloo ranks on CPU; the GPU case
runs the same check on two NCCL ranks when two GPUs are present."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from lowbitlinear_b200 import QuantizedLinear  # noqa: E402
from lowbitlinear_b200.quantization import pack_int4, quantize_int4  # noqa: E402
from lowbitlinear_b200.tensor_parallel import (  # noqa: E402
    ColumnParallelLinear, RowParallelLinear, shard_column_parallel, shard_row_parallel)


def _layer(n, k, seed, std=1.0):
    g = torch.Generator("cpu").manual_seed(seed)
    weight = (torch.randn(n, k, generator=g) * std).half()
    x = torch.randn(3, k, generator=g).half()
    return weight, x


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shards_equal_quantising_the_cut_weight(world):
    """quantize(W)[shard] == quantize(W[shard]) bit for bit, for row cuts and for column cuts
    on group boundaries."""
    weight, _ = _layer(64, 1024, seed=1)
    full = QuantizedLinear.from_float(weight)
    for rank in range(world):
        rows = slice(rank * 64 // world, (rank + 1) * 64 // world)
        cols = slice(rank * 1024 // world, (rank + 1) * 1024 // world)
        for shard, cut in ((shard_column_parallel(full, rank, world), weight[rows]),
                           (shard_row_parallel(full, rank, world), weight[:, cols])):
            direct = QuantizedLinear.from_float(cut.contiguous())
            assert torch.equal(shard.packed_weight, direct.packed_weight)
            assert torch.equal(shard.zeros, direct.zeros)
            assert torch.equal(shard.scales, direct.scales)
            assert shard.packed_weight.is_contiguous() and shard.scales.is_contiguous()


def test_single_process_sharded_sum_matches_full():
    weight, x = _layer(48, 512, seed=2)
    full = QuantizedLinear.from_float(weight)
    expected = full(x).float()
    world = 4
    column_blocks = [shard_column_parallel(full, r, world)(x) for r in range(world)]
    assert torch.equal(torch.cat(column_blocks, dim=1), full(x))
    partial = sum(shard_row_parallel(full, r, world)(x[:, r * 128:(r + 1) * 128].contiguous()).float()
                  for r in range(world))
    torch.testing.assert_close(partial, expected, atol=2e-2, rtol=2e-3)


def test_invalid_splits():
    full = QuantizedLinear.from_float(torch.randn(6, 192))
    with pytest.raises(ValueError):
        shard_column_parallel(full, 0, 4)
    with pytest.raises(ValueError):
        shard_row_parallel(full, 0, 2)  # 96 columns per rank is not a whole number of groups
    shard_row_parallel(full, 0, 3)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, backend, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    device = torch.device("cpu")
    if backend == "nccl":
        torch.cuda.set_device(rank)
        device = torch.device("cuda", rank)
    dist.init_process_group(backend, rank=rank, world_size=world)
    try:
        weight, x = _layer(256, 1024, seed=5, std=0.05)
        full = QuantizedLinear.from_float(weight).to(device)
        x = x.to(device)
        expected = QuantizedLinear.from_float(weight)(x.cpu()).float()  # CPU reference path

        column = ColumnParallelLinear.from_full(full, gather_output=True)
        gathered = column(x)
        local = ColumnParallelLinear.from_full(full)(x)
        row = RowParallelLinear.from_full(full, input_is_parallel=False)
        reduced = row(x)
        part = 1024 // world
        reduced_local = RowParallelLinear.from_full(full)(x[:, rank * part:(rank + 1) * part].contiguous())
        np.savez(Path(result_dir) / f"rank{rank}.npz", gathered=gathered.float().cpu().numpy(),
                 local=local.float().cpu().numpy(), reduced=reduced.float().cpu().numpy(),
                 reduced_local=reduced_local.float().cpu().numpy(), expected=expected.numpy())
    finally:
        dist.destroy_process_group()


def _check(result_dir, world):
    for rank in range(world):
        r = np.load(Path(result_dir) / f"rank{rank}.npz")
        expected = r["expected"]
        n_part = expected.shape[1] // world
        np.testing.assert_allclose(r["gathered"], expected, atol=2e-3, rtol=1e-3)
        np.testing.assert_allclose(r["local"], expected[:, rank * n_part:(rank + 1) * n_part], atol=2e-3, rtol=1e-3)
        # FP16 partial sums are added across ranks: one extra FP16 rounding per rank.
        np.testing.assert_allclose(r["reduced"], expected, atol=4e-3, rtol=2e-3)
        np.testing.assert_allclose(r["reduced_local"], r["reduced"], atol=0, rtol=0)


def test_two_gloo_ranks_on_cpu(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), "gloo", str(tmp_path)), nprocs=world, join=True)
    _check(tmp_path, world)


@pytest.mark.gpu
def test_two_nccl_ranks_on_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), "nccl", str(tmp_path)), nprocs=world, join=True)
    _check(tmp_path, world)


def _fused_worker(rank, world, port, result_dir):
    """K-split decode GEMV with the all-reduce fused into the kernel (peer exchange buffers)."""
    from lowbitlinear_b200 import _ops
    from lowbitlinear_b200.tensor_parallel import PeerExchange

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        n, k = 512, 2048 * world
        weight, x = _layer(n, k, seed=9, std=0.05)
        full = QuantizedLinear.from_float(weight)
        exchange = PeerExchange(max_n=n, device=device)
        on_gpu = QuantizedLinear.from_float(weight).to(device)  # Module.to moves buffers in place
        row = RowParallelLinear.from_full(on_gpu, exchange=exchange)
        part = k // world
        outputs, expected = [], []
        for i in range(6):  # consecutive calls alternate between the two exchange vectors
            xi = (x[:1] * (1.0 + 0.25 * i)).half()
            outputs.append(row(xi[:, rank * part:(rank + 1) * part].contiguous().to(device)))
            expected.append(full(xi).float())
        torch.cuda.synchronize()
        assert _ops.device_status(device) == 0, "a bounded wait expired"
        dist.barrier()
        exchange.close()
        np.savez(Path(result_dir) / f"fused{rank}.npz",
                 outputs=torch.cat(outputs).float().cpu().numpy(), expected=torch.cat(expected).numpy())
    finally:
        dist.destroy_process_group()


def _check_fused(result_dir, world):
    first = None
    for rank in range(world):
        r = np.load(Path(result_dir) / f"fused{rank}.npz")
        # FP32 partial sums are added across ranks, one FP16 rounding at the end.
        np.testing.assert_allclose(r["outputs"], r["expected"], atol=2e-3, rtol=1e-3)
        if first is None:
            first = r["outputs"]
        assert np.array_equal(r["outputs"], first), "ranks must agree bit for bit"


@pytest.mark.gpu
def test_fused_allreduce_single_rank(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA GPU")
    mp.spawn(_fused_worker, args=(1, _free_port(), str(tmp_path)), nprocs=1, join=True)
    _check_fused(tmp_path, 1)


@pytest.mark.gpu
def test_fused_allreduce_two_ranks(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_fused_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    _check_fused(tmp_path, 2)


def _fused_gemm_worker(rank, world, port, result_dir):
    """K-split GEMM (large M) whose epilogue scatters the partial tiles to the owners of their
    columns, followed by the two-kernel reduce + gather over peer memory."""
    from lowbitlinear_b200 import _ops
    from lowbitlinear_b200.graph import GraphedLinears
    from lowbitlinear_b200.tensor_parallel import PeerExchange, shard_row_parallel

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        n, k = 1024, 512 * world
        weight, _ = _layer(n, k, seed=11, std=0.05)
        full = QuantizedLinear.from_float(weight)
        exchange = PeerExchange.for_gemm(640, n, device)
        on_gpu = QuantizedLinear.from_float(weight).to(device)
        row = RowParallelLinear.from_full(on_gpu, gemm_exchange=exchange)
        part = k // world
        g = torch.Generator().manual_seed(5)
        outputs, expected = [], []
        for m in (640, 300, 512, 640):  # ragged last tile, a smaller call in between, reuse of the buffers
            xi = torch.randn(m, k, generator=g).half()
            outputs.append(row(xi[:, rank * part:(rank + 1) * part].contiguous().to(device)))
            expected.append(full(xi).float())
        # The same through the graph runner: the finish kernels run on a side stream.
        shard = shard_row_parallel(on_gpu, rank, world)
        runner = GraphedLinears([shard, shard], m=512, reduce=[True, True], gemm_exchange=exchange)
        assert runner.fused == [True, True]
        xa, xb = torch.randn(512, k, generator=g).half(), torch.randn(512, k, generator=g).half()
        for _ in range(3):
            runner.xs[0].copy_(xa[:, rank * part:(rank + 1) * part])
            runner.xs[1].copy_(xb[:, rank * part:(rank + 1) * part])
            runner.replay()
        torch.cuda.synchronize()
        outputs += [runner.ys[0].clone(), runner.ys[1].clone()]
        expected += [full(xa).float(), full(xb).float()]
        assert _ops.device_status(device) == 0, "a bounded wait expired"
        dist.barrier()
        exchange.close()
        np.savez(Path(result_dir) / f"fused_gemm{rank}.npz",
                 outputs=torch.cat(outputs).float().cpu().numpy(), expected=torch.cat(expected).numpy())
    finally:
        dist.destroy_process_group()


def _check_fused_gemm(result_dir, world):
    first = None
    for rank in range(world):
        r = np.load(Path(result_dir) / f"fused_gemm{rank}.npz")
        # FP16 partial outputs (weights rounded to FP16, as the reference GEMM), FP32 sums over the
        # ranks, one more FP16 rounding.
        np.testing.assert_allclose(r["outputs"], r["expected"], atol=6e-3, rtol=2e-3)
        if first is None:
            first = r["outputs"]
        assert np.array_equal(r["outputs"], first), "ranks must agree bit for bit"


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_fused_gemm_allreduce(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_fused_gemm_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    _check_fused_gemm(tmp_path, world)
