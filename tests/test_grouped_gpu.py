"""Grouped decode GEMV (`lbl_w4a16_group_*`): many independent linears in one persistent launch.

Checked through the C ABI against the numpy oracle, against the per-linear operator (same
arithmetic in the same order, so the bits must agree), on ragged N and mixed K, repeatedly, inside
a CUDA graph, and -- when two GPUs are present -- tensor parallel with the all-reduce kernel over
peer memory.  The reference has no counterpart: it launches one kernel per linear
(csrc/w4a16_gemv_warp_vec.cu:171-187)."""
import os
import socket
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ATOL, RTOL, assert_north_star_parity, oracle_linear, seeded_layer, torch_fp32_linear

pytestmark = pytest.mark.gpu

MIXED = [(1, 512, 1024), (1, 100, 256), (2, 130, 2048), (1, 4096, 4096), (1, 48, 12288), (2, 16, 512),
         (1, 1, 256), (1, 1000, 768), (1, 33, 4096)]


def _problems(shapes, device, seed=0):
    problems = []
    for i, (m, n, k) in enumerate(shapes):
        x, packed, scales, zeros = seeded_layer(m, n, k, seed=seed + 17 * i + m + n + k, std=0.05, device=device)
        problems.append((x, packed, scales, zeros, torch.zeros(m, n, dtype=torch.float16, device=device)))
    return problems


def test_group_matches_oracle_and_the_per_linear_operator(cuda_ops):
    from lowbitlinear_b200 import _ops

    problems = _problems(MIXED, cuda_ops)
    group = _ops.LinearGroup(problems)
    group.run()
    torch.cuda.synchronize()
    for (m, n, k), (x, packed, scales, zeros, y) in zip(MIXED, problems):
        torch.testing.assert_close(y.cpu(), oracle_linear(x, packed, scales, zeros), atol=ATOL, rtol=RTOL)
        single, taken = _ops.linear_forced(x, packed, scales, zeros, _ops.PATH_GEMV, op=0)
        assert taken == _ops.PATH_GEMV
        assert torch.equal(single, y), (m, n, k)
    assert group.algorithmic_bytes == sum(n * k // 2 + 8 * n * (k // 64) + 2 * m * k + 2 * m * n for m, n, k in MIXED)
    # New activations in the same static buffers, twice: same plan, new results, same bits.
    for x, *_ in problems:
        x.mul_(0.5).add_(0.125)
    group.run()
    torch.cuda.synchronize()
    first = [q[4].clone() for q in problems]
    for q in problems:
        q[4].zero_()
    group.run()
    torch.cuda.synchronize()
    for (x, packed, scales, zeros, y), before in zip(problems, first):
        assert torch.equal(y, before)
        torch.testing.assert_close(y.cpu(), oracle_linear(x, packed, scales, zeros), atol=ATOL, rtol=RTOL)
    group.close()


def test_group_of_one_and_more_ctas_than_units(cuda_ops):
    from lowbitlinear_b200 import _ops

    for shapes in ([(1, 16, 256)], [(2, 40, 512), (1, 8, 256)]):
        problems = _problems(shapes, cuda_ops, seed=3)
        group = _ops.LinearGroup(problems)
        group.run()
        torch.cuda.synchronize()
        for x, packed, scales, zeros, y in problems:
            torch.testing.assert_close(y.cpu(), oracle_linear(x, packed, scales, zeros), atol=ATOL, rtol=RTOL)


def test_decode_layers_at_full_size_in_one_launch(cuda_ops):
    """Two layers of the benchmark stack (QKV, O, Gate/Up, Down each) as one group."""
    from lowbitlinear_b200 import _ops

    shapes = [(1, 6144, 4096), (1, 4096, 4096), (1, 24576, 4096), (1, 4096, 12288)] * 2
    problems = []
    for i, (m, n, k) in enumerate(shapes):
        x, packed, scales, zeros = seeded_layer(m, n, k, seed=1000 * (i // 4) + i % 4, device=cuda_ops)
        problems.append((x, packed, scales, zeros, torch.empty(m, n, dtype=torch.float16, device=cuda_ops)))
    group = _ops.LinearGroup(problems)
    for _ in range(3):
        group.run()
    torch.cuda.synchronize()
    for x, packed, scales, zeros, y in problems:
        assert_north_star_parity(y, torch_fp32_linear(x, packed, scales, zeros))
        single = torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(x, packed, scales, zeros, 64)
        assert torch.equal(single, y)
    x, packed, scales, zeros, y = problems[1]
    assert_north_star_parity(y, oracle_linear(x, packed, scales, zeros))


def test_group_inside_a_cuda_graph_with_dependent_launch(cuda_ops):
    from lowbitlinear_b200 import QuantizedLinear, _ops
    from lowbitlinear_b200.graph import GraphedLinears

    layers = []
    for i, (n, k) in enumerate([(512, 1024), (256, 4096), (1024, 2048), (128, 12288)] * 3):
        _, packed, scales, zeros = seeded_layer(1, n, k, seed=40 + i, std=0.05, device=cuda_ops)
        layers.append(QuantizedLinear(packed, scales, zeros, in_features=k))
    runner = GraphedLinears(layers, m=1)
    assert runner.grouped
    host_x = torch.randn(runner.x_flat.numel()).half().pin_memory()
    host_y = torch.zeros(runner.y_flat.numel(), dtype=torch.float16).pin_memory()
    for _ in range(3):
        runner.run(host_x, host_y)
    for layer, xo, yo in zip(layers, runner.x_offsets, runner.y_offsets):
        x = host_x[xo:xo + layer.in_features].view(1, -1).to(cuda_ops)
        want, _ = _ops.linear_forced(x, layer.packed_weight, layer.scales, layer.zeros, _ops.PATH_GEMV, op=0)
        assert torch.equal(host_y[yo:yo + layer.out_features].view(1, -1), want.cpu())
    # The per-layer form of the runner (one launch per layer, its own scratch; small N is split
    # along K there, so the last bit may differ).
    plain = GraphedLinears(layers, m=1, grouped=False)
    other = torch.zeros_like(host_y)
    plain.run(host_x, other)
    torch.testing.assert_close(other, host_y, atol=ATOL, rtol=RTOL)


def test_two_deep_pipeline_matches_the_serial_runner(cuda_ops):
    """PipelinedLinears overlaps the copies of neighbouring steps with the compute; every step's
    outputs must equal those of the serial copy-compute-copy runner on the same activations."""
    from lowbitlinear_b200 import QuantizedLinear
    from lowbitlinear_b200.graph import GraphedLinears, PipelinedLinears

    layers = []
    for i, (n, k) in enumerate([(512, 1024), (256, 4096), (1024, 2048), (128, 12288)] * 2):
        _, packed, scales, zeros = seeded_layer(1, n, k, seed=60 + i, std=0.05, device=cuda_ops)
        layers.append(QuantizedLinear(packed, scales, zeros, in_features=k))
    serial = GraphedLinears(layers, m=1)
    pipe = PipelinedLinears(layers, m=1)
    steps = 7
    host_xs = [torch.randn(serial.x_flat.numel()).half().pin_memory() for _ in range(steps)]
    want = []
    for hx in host_xs:
        out = torch.zeros(serial.y_flat.numel(), dtype=torch.float16).pin_memory()
        want.append(serial.run(hx, out).clone())
    got = [torch.zeros(serial.y_flat.numel(), dtype=torch.float16).pin_memory() for _ in range(steps)]
    for hx, hy in zip(host_xs, got):
        pipe.submit(hx, hy)
    pipe.drain()
    for i, (a, b) in enumerate(zip(got, want)):
        assert torch.equal(a, b), i


def test_group_rejects_what_it_cannot_serve(cuda_ops):
    from lowbitlinear_b200 import _ops

    for m, n, k in ((3, 64, 256), (1, 64, 320), (2, 64, 32768)):
        x = torch.zeros(m, k, dtype=torch.float16, device=cuda_ops)
        packed = torch.zeros(n, k // 8, dtype=torch.int32, device=cuda_ops)
        scales = torch.ones(n, k // 64, device=cuda_ops)
        zeros = torch.zeros(n, k // 64, dtype=torch.int32, device=cuda_ops)
        y = torch.zeros(m, n, dtype=torch.float16, device=cuda_ops)
        with pytest.raises(RuntimeError, match="grouped GEMV serves"):
            _ops.LinearGroup([(x, packed, scales, zeros, y)])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank, world, port, result_dir):
    """Every rank runs a group of N-split and K-split shards; the K-split outputs are summed by the
    all-reduce kernel over peer memory.  Six runs in a row alternate the two exchange vectors."""
    from lowbitlinear_b200 import QuantizedLinear, _ops
    from lowbitlinear_b200.tensor_parallel import PeerExchange, shard_column_parallel, shard_row_parallel

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        shapes = [("col", 512, 1024), ("row", 256, 2048 * world), ("row", 1024, 1024 * world), ("col", 128 * world, 4096)]
        fulls, shards, xs_full = [], [], []
        for i, (kind, n, k) in enumerate(shapes):
            g = torch.Generator("cpu").manual_seed(100 + i)
            weight = (torch.randn(n, k, generator=g) * 0.05).half()
            xs_full.append(torch.randn(1, k, generator=g).half())
            full = QuantizedLinear.from_float(weight)
            fulls.append(full)
            cut = shard_column_parallel if kind == "col" else shard_row_parallel
            shards.append(cut(full, rank, world).to(device))
        exchange = PeerExchange(max_n=sum(n for kind, n, _ in shapes if kind == "row"), device=device)
        problems = []
        for (kind, n, k), shard in zip(shapes, shards):
            x = torch.zeros(1, shard.in_features, dtype=torch.float16, device=device)
            y = torch.zeros(1, shard.out_features, dtype=torch.float16, device=device)
            problems.append((x, shard.packed_weight, shard.scales, shard.zeros, y, kind == "row"))
        group = _ops.LinearGroup(problems, exchange=exchange)
        outputs, expected = [], []
        for step in range(6):
            for (kind, n, k), x_full, q in zip(shapes, xs_full, problems):
                xi = (x_full * (1.0 + 0.25 * step)).half()
                part = q[0].shape[1]
                q[0].copy_(xi[:, rank * part:(rank + 1) * part] if kind == "row" else xi)
            group.run()
            torch.cuda.synchronize()
            for (kind, n, k), x_full, full, q in zip(shapes, xs_full, fulls, problems):
                xi = (x_full * (1.0 + 0.25 * step)).half()
                want = full(xi).float()
                if kind == "col":
                    cols = n // world
                    want = want[:, rank * cols:(rank + 1) * cols]
                outputs.append(q[4].float().cpu().flatten())
                expected.append(want.flatten())
        assert _ops.device_status(device) == 0, "a bounded wait expired"
        exchange.close()
        np.savez(Path(result_dir) / f"group{rank}.npz", outputs=torch.cat(outputs).numpy(),
                 expected=torch.cat(expected).numpy(),
                 reduced=torch.cat([o for i, o in enumerate(outputs) if shapes[i % 4][0] == "row"]).numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2])
def test_tensor_parallel_group_with_the_peer_allreduce(world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_tp_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    first = None
    for rank in range(world):
        r = np.load(tmp_path / f"group{rank}.npz")
        np.testing.assert_allclose(r["outputs"], r["expected"], atol=2e-3, rtol=1e-3)
        if first is None:
            first = r["reduced"]
        assert np.array_equal(r["reduced"], first), "ranks must agree bit for bit on the reduced outputs"
