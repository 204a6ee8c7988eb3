"""Profiling target for Nsight Compute: a few launches of one kernel on rotating weights.

    python -m lowbitlinear_b200.profile --operator gemv  --shape 1x24576x4096 [--copies 4] [--launches 12]
    python -m lowbitlinear_b200.profile --operator gemm  --shape 2048x24576x4096 --copies 1 --launches 3
    python -m lowbitlinear_b200.profile --operator gemm  --shape 16x4096x4096 --path gemm_tc_small
    python -m lowbitlinear_b200.profile --operator group --layers 2 --launches 3
    python -m lowbitlinear_b200.profile --operator quantize --shape 1x8192x4096 --launches 3
    torchrun --nproc-per-node 2 -m lowbitlinear_b200.profile --operator exchange_trace --layers 36

Plays the role of the reference's ``benchmarks/profile_w4a16.py``: inputs are prepared and the
result is checked against an FP32 evaluation first, then the kernel is launched ``--launches``
times, cycling through ``--copies`` distinct copies of the weights (so that a decode GEMV reads
HBM rather than the L2).  ``--path`` forces one kernel of the dispatcher (generic, gemv,
gemv_splitk, gemm_tc, gemm_tc_small); ``--operator group`` runs the grouped decode launch over
``--layers`` Qwen3-8B-shaped layers (four linears each, 120 MB of weights per layer);
``--operator quantize`` runs the device quantiser on an FP16 weight of the given N x K.
``--operator exchange_trace`` (one process per GPU under torchrun; library built with
``python -m lowbitlinear_b200.build --force -D LBL_TRACE_EXCHANGE``) replays the tensor-parallel
decode step of ``--layers`` layers and prints, per replay, the %globaltimer stamps that the grouped
GEMV and the all-reduce kernel leave in the exchange buffer's control block -- a timeline of the
step, not run under a profiler.
The other operators report no latency: timing under a profiler means nothing.  Keep the case small (one kernel,
a few launches, a few hundred MB) when capturing with
``ncu --set full --clock-control none -k regex:<kernel> -s <skip> -c <count>``.
"""
import argparse

import torch

from . import QuantizedLinear, _ops
from ._extension import load_cuda_extension

LAYER_SHAPES = ((6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288))


def fp32_linear(x, layer):
    n, k = layer.out_features, layer.in_features
    shifts = torch.arange(8, device=x.device) * 4
    q = ((layer.packed_weight.to(torch.int64)[..., None] >> shifts) & 15).reshape(n, -1)[:, :k]
    groups = torch.arange(k, device=x.device) // 64
    weight = (q.float() - layer.zeros[:, groups].float()) * layer.scales[:, groups]
    return (x.float() @ weight.T).half()


def rel_l2(actual, expected):
    return ((actual.float() - expected.float()).norm() / expected.float().norm()).item()


def exchange_trace(args):
    """Timeline of the tensor-parallel decode step from the stamps of a trace build."""
    import ctypes
    import os

    import torch.distributed as dist

    from .graph import GraphedLinears
    from .tensor_parallel import PeerExchange

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl")
    g = torch.Generator(device=device).manual_seed(args.seed + rank)
    layers, reduce = [], []
    for _ in range(args.layers):
        for i, (n, k) in enumerate(LAYER_SHAPES):
            rows, cols = (n, k // world) if i == 3 else (n // world, k)  # Down is cut along K, the others along N
            layers.append(QuantizedLinear.from_float((torch.randn(rows, cols, device=device, generator=g) * 0.02).half()))
            reduce.append(i == 3)
    exchange = PeerExchange(max_n=args.layers * LAYER_SHAPES[3][0], device=device)
    runner = GraphedLinears(layers, m=1, reduce=reduce, exchange=exchange)
    runner.x_flat.copy_(torch.randn(runner.x_flat.numel(), device=device, generator=g).half())
    for _ in range(10):
        runner.replay()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    for _ in range(max(8, args.launches)):
        runner.replay()
    torch.cuda.synchronize()
    stamps = (ctypes.c_ulonglong * 64)()
    rc = _ops._lib.lbl_peer_buffer_peek(exchange.pointers[rank], 1536, stamps, 512, local)
    records = sorted(([stamps[i * 8 + j] for j in range(8)] for i in range(8)), key=lambda q: q[0])
    names = ("gemv_end", "allreduce_entered", "gemv_complete_seen", "flags_complete", "sums_complete", "epoch_updated")
    lines = []
    for i, q in enumerate(records):
        if q[0] == 0:
            continue
        parts = [f"{name} {(q[j + 1] - q[0]) / 1e3:.1f}" for j, name in enumerate(names)]
        if i + 1 < len(records):
            parts.append(f"next_step_starts {(records[i + 1][0] - q[0]) / 1e3:.1f}")
        lines.append("  ".join(parts))
    gathered = [None] * world
    dist.all_gather_object(gathered, (rc, lines))
    if rank == 0:
        print(f"decode step of {args.layers} layers on {world} GPUs; microseconds after the start of the grouped GEMV")
        for r, (code, rows) in enumerate(gathered):
            if code != 0 or not rows:
                print(f"rank {r}: no stamps (library not built with -D LBL_TRACE_EXCHANGE?)")
            for row in rows:
                print(f"rank {r}: {row}")
    torch.cuda.synchronize()
    dist.barrier()
    exchange.close()
    dist.destroy_process_group()


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--operator", choices=("gemv", "gemm", "group", "quantize", "exchange_trace"), required=True)
    parser.add_argument("--shape", default=None, help="MxNxK")
    parser.add_argument("--path", choices=tuple(v for v in _ops.PATH_NAMES.values() if v != "auto"), default=None)
    parser.add_argument("--layers", type=int, default=2)
    parser.add_argument("--copies", type=int, default=4)
    parser.add_argument("--launches", type=int, default=12)
    parser.add_argument("--seed", type=int, default=42)
    args = parser.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA GPU")
    load_cuda_extension(required=True)
    torch.backends.cuda.matmul.allow_tf32 = False
    if args.operator == "exchange_trace":
        return exchange_trace(args)
    device = torch.device("cuda", 0)
    g = torch.Generator(device=device).manual_seed(args.seed)

    if args.operator == "group":
        problems, layers = [], []
        for _ in range(args.layers):
            for n, k in LAYER_SHAPES:
                layer = QuantizedLinear.from_float((torch.randn(n, k, device=device, generator=g) * 0.02).half())
                x = torch.randn(1, k, device=device, generator=g).half()
                y = torch.zeros(1, n, dtype=torch.float16, device=device)
                layers.append(layer)
                problems.append((x, layer.packed_weight, layer.scales, layer.zeros, y))
        group = _ops.LinearGroup(problems)
        group.run()
        torch.cuda.synchronize()
        worst = max(rel_l2(q[4], fp32_linear(q[0], layer)) for q, layer in zip(problems, layers))
        assert worst <= 1e-3, f"relative L2 error {worst:.3e}"
        for _ in range(args.launches):
            group.run()
        torch.cuda.synchronize()
        print(f"PASS group layers={args.layers} problems={len(problems)} algorithmic_bytes={group.algorithmic_bytes} "
              f"launches={args.launches} rel_l2={worst:.3e}; no latency is reported here")
        return

    m, n, k = (int(v) for v in args.shape.lower().split("x"))
    if args.operator == "quantize":
        weight = (torch.randn(n, k, device=device, generator=g) * 0.02).half()
        from .quantization import pack_int4, quantize_int4
        packed, scales, zeros = _ops.quantize_pack(weight)
        q, s_ref, z_ref = quantize_int4(weight[:256].cpu(), 64)
        assert torch.equal(packed[:256].cpu(), pack_int4(q)) and torch.equal(zeros[:256].cpu(), z_ref)
        assert torch.equal(scales[:256].cpu(), s_ref)
        for _ in range(args.launches):
            packed, scales, zeros = _ops.quantize_pack(weight)
        torch.cuda.synchronize()
        print(f"PASS quantize shape={n}x{k} launches={args.launches} bit-exact on 256 rows; no latency is reported here")
        return

    x = torch.randn(m, k, device=device, generator=g).half()
    base = QuantizedLinear.from_float((torch.randn(n, k, device=device, generator=g) * 0.02).half())
    copies = [(base.packed_weight.clone(), base.scales.clone(), base.zeros.clone())
              for _ in range(max(1, args.copies))]
    forced = None if args.path is None else {v: c for c, v in _ops.PATH_NAMES.items()}[args.path]

    def run(w):
        if forced is not None:
            return _ops.linear_forced(x, *w, forced, op=0 if args.operator == "gemv" else 1)[0]
        if args.operator == "gemv":
            return torch.ops.lowbitlinear_ext.w4a16_gemv_warp_vec(x, *w, 64)
        return torch.ops.lowbitlinear_cute_w4a16.gemm(x, *w)

    rel = rel_l2(run(copies[0]), fp32_linear(x, base))
    assert rel <= 1e-3, f"relative L2 error {rel:.3e}"
    for i in range(args.launches):
        out = run(copies[i % len(copies)])
    torch.cuda.synchronize()
    print(f"PASS {args.operator} shape={m}x{n}x{k} path={args.path or 'dispatcher'} copies={len(copies)} "
          f"launches={args.launches} rel_l2={rel:.3e} checksum={float(out.float().abs().sum()):.4f}; "
          "no latency is reported here")


if __name__ == "__main__":
    main()
