#!/usr/bin/env python
"""Benchmark of the W4A16 linear forward at Qwen3-8B linear shapes on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode|prefill] [--pdl 0|1]

Workload (synthetic, random-init, no checkpoint): the 36 decoder layers of a Qwen3-8B-shaped
model, four linears per layer -- QKV 6144x4096, O 4096x4096, Gate/Up 24576x4096,
Down 4096x12288 -- with group-64 asymmetric INT4 weights from N(0, 0.02) and FP16 activations
from N(0, 1).  One step is one pass over all 144 linears, each with its own activation:

  decode  (default)  M = 1.     Metric: achieved HBM GB/s = algorithmic bytes / time, where the
                                bytes of one linear are N K / 2 + 8 N K / 64 + 2 M K + 2 M N.
  prefill            M = 2048.  Metric: achieved TFLOP/s = 2 M N K / time.

The 144 weight sets total 4.3 GB, far more than the 126 MB L2, so every step streams from HBM.
The device-timed value replays a CUDA graph of the 144 launches (inputs resident in HBM); the
`e2e` value goes through the public Python API (QuantizedLinear.forward) from pinned host
activations to host outputs, copies included.  With N > 1 (torchrun) the stack is tensor
parallel: QKV, O and Gate/Up are split along N, Down along K with an NCCL all-reduce; the
total work is fixed (strong scaling) and the time is the maximum over ranks.

`--impl reference` times the reference algorithm's CPU path (the numpy oracle under oracle/,
a restatement of lowbitlinear/linear.py:43-70 of NanjinLin/LowBitLinear) on the host cores.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 24576, 4096), ("down", 4096, 12288)]
LAYERS = 36
WEIGHT_STD = 0.02


def linear_bytes(m, n, k):
    return n * k // 2 + 2 * 4 * n * k // 64 + 2 * m * k + 2 * m * n


def linear_flops(m, n, k):
    return 2 * m * n * k


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return {"hbm_gbs": data["hbm_gbs"], "tflops_burst": data["bf16_tflops"],
                "tflops_sustained": data["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
# Clock sampling during the timed region
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.rows = []
        self.proc = None
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", uuid, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except (OSError, RuntimeError, AttributeError):
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        inside = [r for t, r in self.rows if t0 <= t <= t1 + 0.1] or [r for _, r in self.rows[-3:]]
        sm, sm_max, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in inside:
            parts = [p.strip() for p in row.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                sm_max.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(sm_max) if sm_max else None,
                "power_w": statistics.median(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
# Synthetic stack
# ------------------------------------------------------------------------------------------------
def cpu_layer_inputs(m, shape_index, layer=0):
    """Seeded CPU tensors of one linear (the recipe the parity tests use): returns
    (x, weight) FP16 from torch.Generator('cpu').manual_seed(1000 * layer + shape_index)."""
    _, n, k = SHAPES[shape_index]
    g = torch.Generator("cpu").manual_seed(1000 * layer + shape_index)
    weight = (torch.randn(n, k, generator=g) * WEIGHT_STD).half()
    x = torch.randn(m, k, generator=g).half()
    return x, weight


def shard_dims(name, n, k, world):
    """Tensor-parallel shard of one linear: Down is split along K, the others along N."""
    if name == "down":
        return n, k // world
    return n // world, k


def build_stack(m, device, rank, world, host_layer0):
    """Quantised layers and activations resident on `device`.  Layer 0 comes from the seeded CPU
    tensors in `host_layer0` (so that CPU baseline and GPU see identical bits, at world 1);
    the other layers are drawn and quantised on the GPU from per-linear seeds."""
    from lowbitlinear_b200 import QuantizedLinear

    layers, xs = [], []
    for layer in range(LAYERS):
        for idx, (name, n, k) in enumerate(SHAPES):
            ns, ks = shard_dims(name, n, k, world)
            if layer == 0 and world == 1 and host_layer0 is not None:
                x, packed, scales, zeros = host_layer0[idx]
                q_layer = QuantizedLinear(packed.to(device), scales.to(device), zeros.to(device), in_features=k)
                x = x.to(device)
            else:
                g = torch.Generator(device=device).manual_seed(100003 * rank + 1000 * layer + idx)
                weight = (torch.randn(ns, ks, device=device, generator=g) * WEIGHT_STD).half()
                x = torch.randn(m, ks, device=device, generator=g).half()
                q_layer = QuantizedLinear.from_float(weight)
                del weight
            layers.append((name, q_layer))
            xs.append(x)
    return layers, xs


EXCHANGE = None  # PeerExchange of a tensor-parallel decode run: all-reduce fused into the GEMV


def run_stack(layers, xs, world):
    """One pass over the stack through the public operators; returns the outputs.  Between
    tensor-parallel ranks the K-split Down projection ends in an all-reduce: fused into the
    decode kernel over peer memory when an exchange is set up, NCCL otherwise."""
    import torch.distributed as dist

    from lowbitlinear_b200 import _ops

    outs = []
    for (name, layer), x in zip(layers, xs):
        if world > 1 and name == "down":
            if EXCHANGE is not None and x.shape[0] == 1:
                y = _ops.gemv_allreduce(x, layer.packed_weight, layer.scales, layer.zeros, EXCHANGE)
            else:
                y = layer(x)
                dist.all_reduce(y)
        else:
            y = layer(x)
        outs.append(y)
    return outs


# ------------------------------------------------------------------------------------------------
# CPU baseline (oracle) -- checker and reported baseline, never the product path
# ------------------------------------------------------------------------------------------------
def oracle_sample(m, shape_indices, repeats=1):
    """Times the numpy oracle on the given linears of layer 0; returns (seconds per pass,
    per-linear inputs and oracle outputs as torch CPU tensors)."""
    from oracle import w4a16_oracle as oracle

    prepared = []
    for idx in shape_indices:
        x, weight = cpu_layer_inputs(m, idx)
        q, scales, zeros = oracle.quantize_int4(weight.numpy(), 64)
        prepared.append((idx, x.numpy(), oracle.pack_int4(q), scales, zeros))
    times, outputs = [], None
    for _ in range(repeats):
        t0 = time.perf_counter()
        outputs = [oracle.linear_int4_reference(x, p, s, z) for _, x, p, s, z in prepared]
        times.append(time.perf_counter() - t0)
    tensors = {idx: (torch.from_numpy(x), torch.from_numpy(p), torch.from_numpy(s), torch.from_numpy(z))
               for idx, x, p, s, z in prepared}
    return statistics.median(times), tensors, {idx: torch.from_numpy(y) for (idx, *_), y in zip(prepared, outputs)}


def blas_threads():
    try:
        from threadpoolctl import threadpool_info
        counts = [info.get("num_threads", 1) for info in threadpool_info()]
        return max(counts) if counts else os.cpu_count()
    except Exception:  # noqa: BLE001
        return os.cpu_count()


def unit_and_amount(workload, m, shape_indices):
    if workload == "decode":
        return "GB/s", sum(linear_bytes(m, SHAPES[i][1], SHAPES[i][2]) for i in shape_indices) / 1e9
    return "TFLOP/s", sum(linear_flops(m, SHAPES[i][1], SHAPES[i][2]) for i in shape_indices) / 1e12


def metric_name(workload):
    if workload == "decode":
        return "W4A16 decode GEMV achieved HBM GB/s, Qwen3-8B linear shapes (36-layer stack, M=1)"
    return "W4A16 prefill GEMM achieved TFLOP/s, Qwen3-8B linear shapes (36-layer stack, M=2048)"


def config_of(workload, m, world, pdl):
    return {"workload": f"qwen3_8b_linear_stack_{workload}_m{m}",
            "layers": LAYERS, "linears_per_layer": [f"{n}:{N}x{K}" for n, N, K in SHAPES],
            "M": m, "group_size": 64, "weights": "int4 asymmetric, N(0,0.02)", "activations": "fp16 N(0,1)",
            "parallelism": f"tp{world}" if world > 1 else "single",
            "l2": "inputs (4.3 GB of weights per step) are larger than the 126 MB L2",
            "launch": "CUDA graph replay of 144 linears per step", "pdl": bool(pdl)}


# ------------------------------------------------------------------------------------------------
# Reference arm: the reference algorithm's CPU path on the host cores
# ------------------------------------------------------------------------------------------------
def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    m = 1 if args.workload == "decode" else 2048
    budget_s = 150.0
    # Pick a sample that keeps (warmup + steps) passes inside the budget.
    t_o, _, _ = oracle_sample(m, [1])
    passes = args.warmup + args.steps
    indices = [0, 1, 2, 3] if passes * t_o * 12.0 <= budget_s else [1]
    for _ in range(args.warmup):
        oracle_sample(m, indices)
    times = []
    for _ in range(args.steps):
        t, _, _ = oracle_sample(m, indices)
        times.append(t)
    per_step = sum(times) / len(times)
    unit, amount = unit_and_amount(args.workload, m, indices)
    value = amount / per_step
    sample = ("one layer (QKV, O, Gate/Up, Down)" if len(indices) == 4 else "the O projection 4096x4096") + f" at M={m} per step"
    cores = blas_threads()
    line = {"impl": "reference", "metric": metric_name(args.workload), "value": value, "unit": unit,
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": config_of(args.workload, m, 1, 0),
            "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# Our arm
# ------------------------------------------------------------------------------------------------
def check_parity(actual, expected, what):
    a, e = actual.float().cpu(), expected.float().cpu()
    rel = ((a - e).norm() / e.norm().clamp_min(1e-30)).item()
    worst = ((a - e).abs() - (1e-2 + 1e-2 * e.abs())).max().item()
    if not (rel <= 1e-3 and worst <= 0):
        raise SystemExit(f"parity failure on {what}: rel L2 {rel:.3e}, element excess {worst:.3e}")
    return rel


def note(message):
    """Progress line on stderr (only with BENCH_VERBOSE=1): shows where a multi-rank run is."""
    if os.environ.get("BENCH_VERBOSE"):
        print(f"[bench rank {os.environ.get('RANK', '0')} {time.strftime('%H:%M:%S')}] {message}",
              file=sys.stderr, flush=True)


def leave_process_group(world):
    """End a multi-rank run.  Tearing down an NCCL communicator whose collectives live in a
    captured CUDA graph can block for minutes, so the ranks meet at a barrier, flush their
    output and leave without running the destructors."""
    if world <= 1:
        return
    import torch.distributed as dist

    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def run_ours(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU; there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=180))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torchrun for N > 1")

    from lowbitlinear_b200 import _ops
    from lowbitlinear_b200._extension import load_cuda_extension

    load_cuda_extension(required=True)  # fail loudly without the native library
    torch.backends.cuda.matmul.allow_tf32 = False
    m = 1 if args.workload == "decode" else 2048
    peaks = measured_peaks()

    # ---- CPU baseline and identical-input parity (rank 0, single GPU) -------------------------
    cpu_baseline, host_layer0, oracle_out = None, None, None
    if rank == 0 and world == 1:
        indices = [0, 1, 2, 3] if args.workload == "decode" else [1]
        seconds, host_layer0_map, oracle_out = oracle_sample(m, indices)
        unit, amount = unit_and_amount(args.workload, m, indices)
        cpu_baseline = {"value": amount / seconds, "unit": unit, "cores": blas_threads(), "kind": "port",
                        "sample": ("layer 0 (QKV, O, Gate/Up, Down)" if len(indices) == 4 else "layer 0 O projection")
                        + f" at M={m}, one pass, {seconds:.2f} s of numpy oracle"}
        if len(indices) == 4:
            host_layer0 = [host_layer0_map[i] for i in range(4)]

    with torch.inference_mode():
        global EXCHANGE
        if world > 1 and args.workload == "decode" and args.fused_allreduce:
            from lowbitlinear_b200.tensor_parallel import PeerExchange
            EXCHANGE = PeerExchange(max_n=4096, device=device)
        note("building the stack")
        layers, xs = build_stack(m, device, rank, world, host_layer0)
        torch.cuda.synchronize()

        # ---- correctness before timing -----------------------------------------------------------
        _ops.set_programmatic_dependent_launch(False)
        note("eager pass")
        eager = run_stack(layers, xs, world)
        torch.cuda.synchronize()
        parity = {}
        if oracle_out is not None:
            for idx, expected in oracle_out.items():
                if host_layer0 is not None:
                    parity[SHAPES[idx][0]] = check_parity(eager[idx], expected, f"layer 0 {SHAPES[idx][0]} vs oracle")
            if host_layer0 is not None:
                # Packed weights and zero points: the package's quantiser against the oracle's, bit exact.
                from lowbitlinear_b200.quantization import pack_int4, quantize_int4
                x_o, w_o = cpu_layer_inputs(m, 1)
                q, s, z = quantize_int4(w_o, 64)
                assert torch.equal(pack_int4(q), host_layer0[1][1]) and torch.equal(z, host_layer0[1][3])
                assert torch.equal(s, host_layer0[1][2])
        if world == 1:
            # A few linears of other layers against an FP32 evaluation on the GPU.
            for i in (5, 70, 143):
                name, layer = layers[i]
                kk = layer.in_features
                shifts = torch.arange(8, device=device) * 4
                q = ((layer.packed_weight.to(torch.int64)[..., None] >> shifts) & 15).reshape(layer.out_features, -1)[:, :kk]
                groups = torch.arange(kk, device=device) // 64
                w = (q.float() - layer.zeros[:, groups].float()) * layer.scales[:, groups]
                check_parity(eager[i], (xs[i].float() @ w.T).half(), f"linear {i} ({name}) vs FP32 torch")
                del q, w

        # ---- capture one step as a CUDA graph ---------------------------------------------------
        note("capturing the step")
        # When tensor-parallel ranks use NCCL, the kernels alternate with NCCL kernels; a
        # dependent launch that holds SM resources while it waits for a collective could starve
        # it, so programmatic dependent launch is used only when no NCCL kernel is in the graph.
        use_pdl = bool(args.pdl) and (world == 1 or EXCHANGE is not None)
        _ops.set_programmatic_dependent_launch(use_pdl)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                run_stack(layers, xs, world)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            graph_out = run_stack(layers, xs, world)
        note("first replay")
        graph.replay()
        torch.cuda.synchronize()
        for i, (a, b) in enumerate(zip(graph_out, eager)):
            if not torch.equal(a, b):
                if world > 1 and layers[i][0] == "down":
                    continue  # all-reduce order may differ between eager and captured runs
                raise SystemExit(f"graph replay differs from eager run on linear {i}")

        note("timed region")

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        # ---- device-timed region ------------------------------------------------------------------
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        barrier()
        sampler = ClockSampler(local_rank) if rank == 0 else None
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t0 = time.perf_counter()
        start.record()
        for _ in range(args.steps):
            graph.replay()
        end.record()
        barrier()
        t1 = time.perf_counter()
        elapsed_ms = start.elapsed_time(end)
        if world > 1:
            t = torch.tensor([elapsed_ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            elapsed_ms = t.item()
        if elapsed_ms < 1500.0:
            # The timed region was too short for nvidia-smi to sample: hold the same load a
            # little longer, for the clock record only.  Every rank replays the same number of
            # times (the count derives from the reduced time), since the graph holds collectives.
            hold_replays = int(1500.0 / max(elapsed_ms / args.steps, 1e-3)) + 1
            for _ in range(hold_replays):
                graph.replay()
            torch.cuda.synchronize()
            t1 = time.perf_counter()
        clocks = sampler.stop(t0, t1) if sampler is not None else None
        ms_per_step = elapsed_ms / args.steps

        note("end-to-end region")
        # ---- end to end through the public API, host buffers ---------------------------------------
        _ops.set_programmatic_dependent_launch(False)
        # Decode: the whole stack's activations go up in one pinned copy and all outputs come
        # back in one.  Prefill: one layer at a time through the same pinned buffers (the
        # activations of a step would not fit pinned memory comfortably), so every layer sees
        # layer 0's activation values; the work per step is unchanged.
        chunk = len(layers) if args.workload == "decode" else len(SHAPES)
        x_sizes = [x.numel() for x in xs[:chunk]]
        host_x = torch.empty(sum(x_sizes), dtype=torch.float16).pin_memory()
        offset = 0
        for x, size in zip(xs[:chunk], x_sizes):
            host_x[offset:offset + size].copy_(x.reshape(-1).cpu())
            offset += size
        dev_x = torch.empty_like(host_x, device=device)
        out_elems = sum(m * layer.out_features for _, layer in layers[:chunk])
        host_y = torch.empty(out_elems, dtype=torch.float16).pin_memory()
        chunks_per_step = len(layers) // chunk

        def e2e_step():
            for c in range(chunks_per_step):
                dev_x.copy_(host_x, non_blocking=True)
                views, off = [], 0
                for x, size in zip(xs[:chunk], x_sizes):
                    views.append(dev_x[off:off + size].view_as(x))
                    off += size
                outs = run_stack(layers[c * chunk:(c + 1) * chunk], views, world)
                host_y.copy_(torch.cat([o.reshape(-1) for o in outs]), non_blocking=True)
            torch.cuda.current_stream().synchronize()

        e2e_api = "QuantizedLinear.forward, eager, pinned host activations in, host outputs out"
        e2e_eager_ms = None
        if args.workload == "decode" and world == 1:
            # Eager first (kept as a secondary figure), then the CUDA-graph runner of the package:
            # one pinned host-to-device copy, one replay of the captured operators, one copy back.
            for _ in range(2):
                e2e_step()
            t_eager = time.perf_counter()
            for _ in range(5):
                e2e_step()
            e2e_eager_ms = (time.perf_counter() - t_eager) * 1e3 / 5
            from lowbitlinear_b200.graph import GraphedLinears
            runner = GraphedLinears([layer for _, layer in layers], m=m,
                                    programmatic_dependent_launch=bool(args.pdl))
            host_x = torch.zeros(runner.x_flat.numel(), dtype=torch.float16).pin_memory()
            host_y = torch.zeros(runner.y_flat.numel(), dtype=torch.float16).pin_memory()
            for offset, x in zip(runner.x_offsets, xs):
                host_x[offset:offset + x.numel()] = x.reshape(-1).cpu()
            runner.run(host_x, host_y)
            for offset, want in zip(runner.y_offsets, eager):
                if not torch.equal(host_y[offset:offset + want.numel()].view_as(want), want.cpu()):
                    raise SystemExit("graph runner output differs from the eager forward")
            chunks_per_step = 1

            def e2e_step():  # noqa: F811
                runner.run(host_x, host_y)

            e2e_api = ("lowbitlinear_b200.graph.GraphedLinears.run: pinned host activations in, one CUDA-graph "
                       "replay of the public operators, host outputs out")

        e2e_steps = max(3, min(args.steps, 20))
        for _ in range(3):
            e2e_step()
        barrier()
        e0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        e2e_ms = (time.perf_counter() - e0) * 1e3 / e2e_steps
        if world > 1:
            t = torch.tensor([e2e_ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = t.item()

        status = _ops.device_status(device)
        if status != 0:
            raise SystemExit(f"device status {status}: a bounded wait expired inside a kernel")

    # ---- report -------------------------------------------------------------------------------------
    all_idx = [0, 1, 2, 3]
    unit, per_layer = unit_and_amount(args.workload, m, all_idx)
    amount = per_layer * LAYERS  # whole job, all ranks together
    value = amount / (ms_per_step * 1e-3)
    launches_per_step = len(layers)
    # DRAM bytes per launch: ratio of (dram read + write) to algorithmic bytes from the committed
    # ncu captures of one Gate/Up launch (profiles/), applied to this rank's average launch;
    # traffic follows the weights in proportion, there are no re-reads.
    algorithmic_bytes_per_launch = sum(linear_bytes(m, SHAPES[i][1], SHAPES[i][2]) for i in all_idx) / 4.0 / world
    traffic_ratio = 1.006 if args.workload == "decode" else 0.750
    traffic = traffic_ratio * algorithmic_bytes_per_launch
    if args.workload == "decode":
        roofline = {"bound": "hbm", "achieved": value / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": value / world / peaks["hbm_gbs"], "traffic": traffic,
                    "traffic_unit": "bytes per launch (ncu dram read+write of one Gate/Up launch, scaled)",
                    "kernel": "w4a16_gemv_decode_kernel", "peak_source": peaks["source"],
                    "per_launch": "per-GPU algorithmic bytes of the step / 144 launches, over the step's CUDA-event time / 144"}
    else:
        roofline = {"bound": "tensor", "achieved": value / world, "peak": peaks["tflops_sustained"], "unit": "TFLOP/s",
                    "frac": value / world / peaks["tflops_sustained"], "traffic": traffic,
                    "traffic_unit": "bytes per launch (ncu dram read+write of one Gate/Up launch, scaled)",
                    "kernel": "w4a16_gemm_tc_kernel", "peak_source": peaks["source"] + " (sustained bf16)",
                    "per_launch": "per-GPU flops of the step / 144 launches, over the step's CUDA-event time / 144"}
    if rank != 0:
        leave_process_group(world)
        return
    line = {
        "metric": metric_name(args.workload), "value": value, "unit": unit, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 activations x int4 weights, f32 accumulate", "data": "synthetic",
        "config": dict(config_of(args.workload, m, world, args.pdl and (world == 1 or EXCHANGE is not None)),
                       allreduce=("none" if world == 1 else
                                  "fused into the Down GEMV over NVLink peer memory" if EXCHANGE is not None
                                  else "NCCL")),
        "roofline": roofline, "cpu_baseline": cpu_baseline, "clocks": clocks,
        "e2e": {"value": amount / (e2e_ms * 1e-3), "unit": unit, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": int(host_x.numel() * 2 * chunks_per_step),
                "d2h_bytes_per_step": int(host_y.numel() * 2 * chunks_per_step),
                "api": e2e_api,
                "eager_forward_ms_per_step": e2e_eager_ms},
        "gpu_launches": launches_per_step * args.steps,
        "parity": {"rel_l2_vs_oracle": parity, "tolerance": "rel L2 <= 1e-3, |a-b| <= 1e-2 + 1e-2|b|"},
        "fraction_of_nominal": value / world / (8000.0 if args.workload == "decode" else 2250.0),
    }
    print(json.dumps(line), flush=True)
    leave_process_group(world)


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--workload", choices=("decode", "prefill"), default="decode")
    parser.add_argument("--pdl", type=int, default=1)
    parser.add_argument("--fused-allreduce", type=int, default=1,
                        help="tensor-parallel decode: fuse the K-split all-reduce into the GEMV (0: NCCL)")
    args = parser.parse_args()
    if args.impl == "reference":
        if args.steps == 200:
            args.steps = 3
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
