#!/usr/bin/env python
"""Benchmark of the W4A16 linear forward at Qwen3-8B linear shapes on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference_gpu]
                    [--workload stack|decode|prefill|crossover|prefill_sweep]

Workload (synthetic, random-init, no checkpoint): the 36 decoder layers of a Qwen3-8B-shaped
model, four linears per layer -- QKV 6144x4096, O 4096x4096, Gate/Up 24576x4096,
Down 4096x12288 -- with group-64 asymmetric INT4 weights from N(0, 0.02) and FP16 activations
from N(0, 1).  One step is one pass over all 144 linears, each with its own activation:

  decode   M = 1.     Metric: achieved HBM GB/s = algorithmic bytes / time, where the bytes of one
                      linear are N K / 2 + 8 N K / 64 + 2 M K + 2 M N.  The 144 independent
                      linears run as ONE grouped launch (lbl_w4a16_group_run).
  prefill  M = 2048.  Metric: achieved TFLOP/s = 2 M N K / time, one launch per linear.
  stack    (default)  both: the JSON line's `value` is the decode figure, its `gemm` block the
                      prefill figure.
  crossover      benchmark config 3: the four shapes at M in {2..64}, every kernel path forced
                 plus the dispatcher's pick, weights rotating through more than the L2.
  prefill_sweep  benchmark config 4: Gate/Up and Down at M in {128, 512, 2048, 8192}.

The 144 weight sets total 4.3 GB, far more than the 126 MB L2, so every step streams from HBM.
Device-timed values replay a CUDA graph of the step (inputs resident in HBM), each step between
its own pair of CUDA events; `e2e` goes through the package's public runner from pinned host
activations to host outputs, copies included.  With N > 1 (torchrun) the stack is tensor
parallel: QKV, O and Gate/Up are split along N, Down along K with an all-reduce over NVLink (peer
memory kernel for decode, NCCL for prefill); total work is fixed (strong scaling), time is the
maximum over ranks, and every rank's layer-0 outputs are checked against the CPU reference.

`--impl reference` times the reference's own CPU path, `linear_int4_reference` of
NanjinLin/LowBitLinear (lowbitlinear/linear.py:43-70), imported from oracle/_ref when that
install exists (oracle/make_ref.py) and restated by the numpy oracle otherwise.
`--impl reference_gpu` (crossover / prefill_sweep only) times the reference's own CUDA operators,
compiled for sm_100a by the same install, in a process that never loads this library.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
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
PREFILL_M = 2048
REF_DIR = ROOT / "oracle" / "_ref"
TOLERANCE = "rel L2 <= 1e-3, |a-b| <= 1e-2 + 1e-2|b|"


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


def traffic_ratio(kernel):
    """DRAM bytes (read + write) per algorithmic byte of one launch of `kernel`, from the ncu
    capture summarised under profiles/ (profiles/traffic.json); None when there is no capture."""
    path = ROOT / "profiles" / "traffic.json"
    if not path.is_file():
        return None, None
    entry = json.loads(path.read_text()).get(kernel)
    if not entry:
        return None, None
    return entry.get("dram_bytes_per_algorithmic_byte"), entry.get("source")


def summary(samples_ms):
    """Median / P90 / min / max of per-step times, as the reference's harness reports them
    (benchmarks/_common.py:175-181)."""
    ordered = sorted(samples_ms)
    p90 = ordered[min(len(ordered) - 1, int(round(0.9 * (len(ordered) - 1))))]
    return {"median_ms": statistics.median(ordered), "p90_ms": p90, "min_ms": ordered[0], "max_ms": ordered[-1],
            "samples": len(ordered)}


# ------------------------------------------------------------------------------------------------
# Clock sampling during the timed region (read-only NVML queries from a thread)
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20}

    def __init__(self, device_index, period_s=0.002):
        self.rows = []
        self.period = period_s
        self.stop_flag = False
        self.handle = None
        self.thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001  (no NVML: the line says so)
            self.handle = None

    def _loop(self):
        nv = self.nvml
        while not self.stop_flag:
            try:
                sm = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                power = nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                self.rows.append((time.perf_counter(), sm, reasons, power))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def window(self, t0, t1):
        """Clock record of [t0, t1]; when the region was too short for three samples, the
        samples of the warm-up right before it (same load) are included and that is stated."""
        if self.handle is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["NVML unavailable"]}
        inside = [r for r in self.rows if t0 <= r[0] <= t1]
        note = "sampled inside the timed region"
        if len(inside) < 3:
            inside = [r for r in self.rows if t0 - 0.25 <= r[0] <= t1 + 0.005]
            note = "timed region shorter than three samples: includes the warm-up replays just before it"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": float(self.max_sm), "reasons": ["no samples"], "samples": 0}
        reasons = set()
        for _, _, mask, _ in inside:
            for name, bit in self.REASONS.items():
                if mask & bit:
                    reasons.add(name)
        return {"sm_mhz": statistics.median(r[1] for r in inside), "sm_max_mhz": float(self.max_sm),
                "power_w": statistics.median(r[3] for r in inside), "samples": len(inside),
                "reasons": sorted(reasons), "window": note}

    def close(self):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=1.0)


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


def shard_of(name, tensor_nk, rank, world, per_k):
    """Rank's slice of a [N, K / per_k] buffer of a full linear (rows, or columns for Down)."""
    if world == 1:
        return tensor_nk
    if name == "down":
        cols = tensor_nk.shape[1] // world
        return tensor_nk[:, rank * cols:(rank + 1) * cols].contiguous()
    rows = tensor_nk.shape[0] // world
    return tensor_nk[rank * rows:(rank + 1) * rows].contiguous()


def build_layers(device, rank, world, host_layer0):
    """Quantised (sharded) layers resident on `device`.  Layer 0 is cut from the seeded CPU tensors
    in `host_layer0` (packed, scales, zeros per linear), so that the CPU reference and every rank
    see identical bits; the other layers are drawn and quantised on the GPU from per-linear seeds."""
    from lowbitlinear_b200 import QuantizedLinear

    layers = []
    for layer in range(LAYERS):
        for idx, (name, n, k) in enumerate(SHAPES):
            ns, ks = shard_dims(name, n, k, world)
            if layer == 0 and host_layer0 is not None:
                packed, scales, zeros = host_layer0[idx]
                q_layer = QuantizedLinear(shard_of(name, packed, rank, world, 8).to(device),
                                          shard_of(name, scales, rank, world, 64).to(device),
                                          shard_of(name, zeros, rank, world, 64).to(device), in_features=ks)
            else:
                g = torch.Generator(device=device).manual_seed(100003 * rank + 1000 * layer + idx)
                weight = (torch.randn(ns, ks, device=device, generator=g) * WEIGHT_STD).half()
                q_layer = QuantizedLinear.from_float(weight)
                del weight
            layers.append((name, q_layer))
    return layers


def fill_activations(runner, layers, m, device, rank, world, host_x0):
    """Seeded activations into the runner's static buffer; layer 0 gets the CPU reference's x."""
    for i, ((name, layer), x_view) in enumerate(zip(layers, runner.xs)):
        if i < len(SHAPES) and host_x0 is not None:
            x = host_x0[i]
            if world > 1 and name == "down":
                part = layer.in_features
                x = x[:, rank * part:(rank + 1) * part]
            x_view.copy_(x.to(device))
        else:
            g = torch.Generator(device=device).manual_seed(7 + 100003 * rank + i + 1009 * m)
            x_view.copy_(torch.randn(m, layer.in_features, device=device, generator=g).half())


# ------------------------------------------------------------------------------------------------
# Reference arm: the reference's own CPU path on the host cores (own process, never this library)
# ------------------------------------------------------------------------------------------------
def reference_functions():
    """(linear_int4_reference, quantize, kind): from the reference install when present."""
    if (REF_DIR / "lowbitlinear" / "linear.py").is_file():
        sys.path.insert(0, str(REF_DIR))
        from lowbitlinear.linear import linear_int4_reference
        from lowbitlinear.quantization import pack_int4, quantize_int4

        def quantize(weight):
            q, scales, zeros = quantize_int4(weight, 64)
            return pack_int4(q), scales, zeros

        return linear_int4_reference, quantize, "reference"
    from oracle import w4a16_oracle as oracle

    def quantize(weight):
        q, scales, zeros = oracle.quantize_int4(weight.numpy(), 64)
        return torch.from_numpy(oracle.pack_int4(q)), torch.from_numpy(scales), torch.from_numpy(zeros)

    def linear(x, packed, scales, zeros, group_size=64):
        return torch.from_numpy(oracle.linear_int4_reference(x.numpy(), packed.numpy(), scales.numpy(), zeros.numpy()))

    return linear, quantize, "port"


def cpu_description(kind):
    model = ""
    try:
        for line in Path("/proc/cpuinfo").read_text().splitlines():
            if line.startswith("model name"):
                model = line.split(":", 1)[1].strip()
                break
    except OSError:
        pass
    return {"kind": kind, "cores": torch.get_num_threads(), "cpu_count": os.cpu_count(), "cpu_model": model,
            "implementation": ("lowbitlinear.linear.linear_int4_reference of the unmodified reference (oracle/_ref)"
                               if kind == "reference" else "numpy restatement (oracle/w4a16_oracle.py); oracle/_ref absent")}


def reference_sample(m, shape_indices, passes, warmup, emit=None):
    """Times `passes` evaluations of the given layer-0 linears on the host cores.  Returns
    (seconds per pass, per-pass list, kind); with `emit` also saves inputs and outputs."""
    linear, quantize, kind = reference_functions()
    prepared = []
    for idx in shape_indices:
        x, weight = cpu_layer_inputs(m, idx)
        packed, scales, zeros = quantize(weight)
        prepared.append((idx, x, packed, scales, zeros))
    outputs = None
    times = []
    with torch.inference_mode():
        for it in range(warmup + passes):
            t0 = time.perf_counter()
            outputs = [linear(x, p, s, z, 64) for _, x, p, s, z in prepared]
            if it >= warmup:
                times.append(time.perf_counter() - t0)
    if emit is not None:
        arrays = {}
        for (idx, x, p, s, z), y in zip(prepared, outputs):
            arrays.update({f"x{idx}": x.numpy(), f"packed{idx}": p.numpy(), f"scales{idx}": s.numpy(),
                           f"zeros{idx}": z.numpy(), f"y{idx}": y.numpy()})
        np.savez(emit, **arrays)
    return sum(times) / len(times), times, kind


def unit_and_amount(workload, m, shape_indices):
    if workload == "decode":
        return "GB/s", sum(linear_bytes(m, SHAPES[i][1], SHAPES[i][2]) for i in shape_indices) / 1e9
    return "TFLOP/s", sum(linear_flops(m, SHAPES[i][1], SHAPES[i][2]) for i in shape_indices) / 1e12


def metric_name(workload):
    decode = "W4A16 decode GEMV achieved HBM GB/s, Qwen3-8B linear shapes (36-layer stack, M=1)"
    prefill = f"W4A16 prefill GEMM achieved TFLOP/s, Qwen3-8B linear shapes (36-layer stack, M={PREFILL_M})"
    if workload == "decode":
        return decode
    if workload == "prefill":
        return prefill
    return decode + "; `gemm` block: " + prefill


def config_of(workload, world):
    """Identical for both arms of a run (the reference arm measures a bounded sample of it)."""
    return {"workload": {"stack": f"qwen3_8b_linear_stack_decode_m1+prefill_m{PREFILL_M}",
                         "decode": "qwen3_8b_linear_stack_decode_m1",
                         "prefill": f"qwen3_8b_linear_stack_prefill_m{PREFILL_M}"}[workload],
            "layers": LAYERS, "linears_per_layer": [f"{n}:{N}x{K}" for n, N, K in SHAPES],
            "M": {"stack": [1, PREFILL_M], "decode": [1], "prefill": [PREFILL_M]}[workload], "group_size": 64,
            "weights": "int4 asymmetric, N(0,0.02)", "activations": "fp16 N(0,1)",
            "parallelism": f"tp{world}" if world > 1 else "single",
            "l2": "inputs (4.3 GB of weights per step) are larger than the 126 MB L2"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # All the host threads there are (torchrun sets OMP_NUM_THREADS=1 for its workers).
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    if args.emit:  # helper mode of our own arm: layer 0 at M = 1, inputs and outputs saved
        seconds, times, kind = reference_sample(1, [0, 1, 2, 3], passes=max(1, args.steps), warmup=min(1, args.warmup),
                                                emit=args.emit)
        print(json.dumps({"seconds_per_pass": seconds, "times": times, **cpu_description(kind)}), flush=True)
        return
    workload = args.workload if args.workload in ("decode", "prefill", "stack") else "stack"
    passes = max(1, args.steps)
    line = {"impl": "reference", "metric": metric_name(workload), "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": config_of(workload, args.gpus), "gpu_launches": 0}
    blocks = {}
    for part in (["decode", "prefill"] if workload == "stack" else [workload]):
        m = 1 if part == "decode" else PREFILL_M
        # Bounded sample: one layer at M = 1 (about a second per pass); the O projection at M = 2048.
        indices = [0, 1, 2, 3] if part == "decode" else [1]
        n_pass = passes if part == "decode" else max(1, min(passes, 5))
        seconds, times, kind = reference_sample(m, indices, passes=n_pass, warmup=min(args.warmup, 2))
        unit, amount = unit_and_amount(part, m, indices)
        sample = (("layer 0 (QKV, O, Gate/Up, Down)" if len(indices) == 4 else "layer 0 O projection 4096x4096")
                  + f" at M={m} per step, {n_pass} timed passes")
        blocks[part] = {"value": amount / seconds, "unit": unit, "ms_per_step": seconds * 1e3,
                        "stats": summary([t * 1e3 for t in times]),
                        "cpu_baseline": {"value": amount / seconds, "unit": unit, "sample": sample,
                                         **cpu_description(kind)},
                        "e2e": {"value": amount / seconds, "unit": unit, "h2d_bytes_per_step": 0,
                                "d2h_bytes_per_step": 0}}
    head = blocks.get("decode") or blocks["prefill"]
    line.update({"value": head["value"], "unit": head["unit"], "ms_per_step": head["ms_per_step"],
                 "stats": head["stats"], "cpu_baseline": head["cpu_baseline"], "e2e": head["e2e"]})
    if workload == "stack":
        line["gemm"] = blocks["prefill"]
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# Our arm
# ------------------------------------------------------------------------------------------------
def parity_numbers(actual, expected):
    a, e = actual.float().cpu(), expected.float().cpu()
    rel = ((a - e).norm() / e.norm().clamp_min(1e-30)).item()
    worst = ((a - e).abs() - (1e-2 + 1e-2 * e.abs())).max().item()
    return rel, worst


def check_parity(actual, expected, what):
    rel, worst = parity_numbers(actual, expected)
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


class Context:
    """What every workload of our arm needs: ranks, device, peaks, the clock sampler."""

    def __init__(self, args):
        import torch.distributed as dist

        self.args = args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA GPU; there is no CPU fallback")
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        if self.world > 1:
            import datetime
            dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=300))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}; launch with torchrun for N > 1")
        from lowbitlinear_b200._extension import load_cuda_extension

        load_cuda_extension(required=True)  # fail loudly without the native library
        torch.backends.cuda.matmul.allow_tf32 = False
        self.peaks = measured_peaks()
        self.dist = dist
        self.sampler = ClockSampler(self.local_rank) if self.rank == 0 else None

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, value):
        if self.world == 1:
            return value
        t = torch.tensor([value], device=self.device, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.item()

    def timed_replays(self, replay, steps, warmup):
        """`warmup` untimed replays, then exactly `steps` replays, each between its own CUDA events
        on the launching stream, bracketed by barrier + synchronize.  Returns (total ms as the
        maximum over ranks, this rank's per-step ms, clock record of the region)."""
        for _ in range(max(warmup, 3)):
            replay()
        self.barrier()
        events = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        self.barrier()
        t0 = time.perf_counter()
        events[0].record()
        for i in range(steps):
            replay()
            events[i + 1].record()
        self.barrier()
        t1 = time.perf_counter()
        total = self.max_over_ranks(events[0].elapsed_time(events[-1]))
        per_step = [events[i].elapsed_time(events[i + 1]) for i in range(steps)]
        clocks = self.sampler.window(t0, t1) if self.sampler is not None else None
        return total, per_step, clocks

    def wall_steps(self, step, steps):
        """End-to-end timing by the host clock (copies included), maximum over ranks."""
        for _ in range(3):
            step()
        self.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        self.barrier()
        return self.max_over_ranks((time.perf_counter() - t0) * 1e3 / steps)


def reference_layer0(ctx):
    """Rank 0 runs the reference's CPU path on layer 0 (M = 1) in a process of its own -- the
    reference install registers the same operator names as this library, so the two never share
    a process -- and every rank receives its inputs and outputs."""
    payload = [None]
    if ctx.rank == 0:
        with tempfile.TemporaryDirectory() as tmp:
            emit = str(Path(tmp) / "layer0.npz")
            env = {k: v for k, v in os.environ.items() if k != "OMP_NUM_THREADS"}
            env.update(RANK="0", WORLD_SIZE="1")
            timed = ctx.world == 1  # the timed CPU baseline is reported at N = 1 only
            result = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--emit", emit,
                                     "--steps", "3" if timed else "1", "--warmup", "1" if timed else "0"],
                                    capture_output=True, text=True, env=env)
            if result.returncode != 0:
                raise SystemExit("the CPU reference leg failed:\n" + result.stdout[-2000:] + result.stderr[-2000:])
            info = json.loads(result.stdout.strip().splitlines()[-1])
            data = np.load(emit)
            payload[0] = (info, {key: data[key] for key in data.files})
    if ctx.world > 1:
        ctx.dist.broadcast_object_list(payload, src=0)
    info, arrays = payload[0]
    tensors = {key: torch.from_numpy(value) for key, value in arrays.items()}
    host_layer0 = [(tensors[f"packed{i}"], tensors[f"scales{i}"], tensors[f"zeros{i}"]) for i in range(4)]
    host_x0 = [tensors[f"x{i}"] for i in range(4)]
    expected = [tensors[f"y{i}"] for i in range(4)]
    return info, host_layer0, host_x0, expected


def check_layer0(ctx, layers, runner, expected, m_label):
    """Every rank compares its layer-0 outputs of `runner` with the CPU reference (its own
    column block for the N-split linears, the whole all-reduced vector for Down), and the ranks
    compare their Down outputs bit for bit.  Returns {name: worst relative L2 over the ranks}."""
    result = {}
    for idx, (name, n, k) in enumerate(SHAPES):
        got = runner.ys[idx]
        want = expected[idx]
        if ctx.world > 1 and name != "down":
            cols = n // ctx.world
            want = want[:, ctx.rank * cols:(ctx.rank + 1) * cols]
        rel = check_parity(got, want, f"layer 0 {name} ({m_label}) vs the CPU reference, rank {ctx.rank}")
        result[name] = ctx.max_over_ranks(rel)
        if ctx.world > 1 and name == "down":
            gathered = [torch.empty_like(got) for _ in range(ctx.world)]
            ctx.dist.all_gather(gathered, got.contiguous())
            if not all(torch.equal(gathered[0], other) for other in gathered[1:]):
                raise SystemExit("ranks disagree on an all-reduced Down output")
            result["down_bit_identical_across_ranks"] = True
    return result


def run_decode(ctx, layers, reference):
    """M = 1: the whole stack as one grouped launch (plus the all-reduce kernel between ranks)."""
    from lowbitlinear_b200 import _ops
    from lowbitlinear_b200.graph import GraphedLinears

    args, world, device = ctx.args, ctx.world, ctx.device
    info, _, host_x0, expected = reference
    exchange = None
    if world > 1:
        from lowbitlinear_b200.tensor_parallel import PeerExchange
        exchange = PeerExchange(max_n=LAYERS * SHAPES[3][1], device=device)
    reduce = [name == "down" for name, _ in layers]
    modules = [layer for _, layer in layers]
    runner = GraphedLinears(modules, m=1, reduce=reduce, exchange=exchange)
    assert runner.grouped
    fill_activations(runner, layers, 1, device, ctx.rank, world, host_x0)
    note("decode: correctness")
    runner.replay()
    torch.cuda.synchronize()
    parity = check_layer0(ctx, layers, runner, expected, "M=1, grouped launch")
    # The public per-call API on the same inputs: identical arithmetic, so identical bits wherever
    # that call does not split K; other layers against an FP32 evaluation on the GPU.
    for i in (1, 5, 70, 143):
        name, layer = layers[i]
        if world > 1 and name == "down":
            continue
        eager = layer(runner.xs[i])
        if _ops.select_path(1, layer.out_features, layer.in_features, 0) == _ops.PATH_GEMV:
            if not torch.equal(eager, runner.ys[i]):
                raise SystemExit(f"grouped launch differs from QuantizedLinear.forward on linear {i}")
        kk = layer.in_features
        shifts = torch.arange(8, device=device) * 4
        q = ((layer.packed_weight.to(torch.int64)[..., None] >> shifts) & 15).reshape(layer.out_features, -1)[:, :kk]
        groups = torch.arange(kk, device=device) // 64
        w = (q.float() - layer.zeros[:, groups].float()) * layer.scales[:, groups]
        check_parity(runner.ys[i], (runner.xs[i].float() @ w.T).half(), f"linear {i} ({name}) vs FP32 torch")
        del q, w

    note("decode: timed region")
    total_ms, per_step, clocks = ctx.timed_replays(runner.replay, args.steps, args.warmup)
    ms_per_step = total_ms / args.steps
    after = runner.y_flat.clone()
    runner.replay()
    torch.cuda.synchronize()
    if not torch.equal(after, runner.y_flat):
        raise SystemExit("the grouped launch is not bit-reproducible")

    # ---- end to end: every step copies its activations up from pinned host memory, runs one replay
    # and copies its outputs down; a two-deep pipeline (PipelinedLinears) overlaps the copies of
    # neighbouring steps with the compute.  The serial form (copy, compute, copy, wait) is reported too.
    from lowbitlinear_b200.graph import PipelinedLinears

    host_x = runner.x_flat.cpu().pin_memory()
    host_y = torch.zeros(runner.y_flat.numel(), dtype=torch.float16).pin_memory()
    serial_ms = ctx.wall_steps(lambda: runner.run(host_x, host_y), max(5, min(args.steps, 50)))
    if not torch.equal(host_y, after.cpu()):
        raise SystemExit("end-to-end outputs differ from the device-timed ones")
    pipe = PipelinedLinears(modules, m=1, reduce=reduce, exchange=exchange)
    host_ys = [torch.zeros_like(host_y).pin_memory() for _ in range(3)]
    e2e_steps = max(10, min(args.steps, 50))

    def pipelined_pass(steps):
        for i in range(steps):
            pipe.submit(host_x, host_ys[i % 3])
        pipe.drain()

    pipelined_pass(6)
    ctx.barrier()
    t0 = time.perf_counter()
    pipelined_pass(e2e_steps)
    ctx.barrier()
    e2e_ms = ctx.max_over_ranks((time.perf_counter() - t0) * 1e3 / e2e_steps)
    for buf in host_ys:
        if not torch.equal(buf, after.cpu()):
            raise SystemExit("pipelined end-to-end outputs differ from the device-timed ones")
    del pipe

    # ---- secondary: one launch per linear (what a model with dependent layers would do) -----------
    per_linear = None
    if world == 1:
        plain = GraphedLinears(modules, m=1, grouped=False)
        plain.x_flat.copy_(runner.x_flat)
        plain_total, plain_steps, _ = ctx.timed_replays(plain.replay, min(args.steps, 20), 3)
        plain_ms = plain_total / min(args.steps, 20)
        eager_ms = None
        steps = 3
        xs = plain.xs
        for _ in range(2):
            for layer, x in zip(modules, xs):
                layer(x)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            for layer, x in zip(modules, xs):
                layer(x)
        torch.cuda.synchronize()
        eager_ms = (time.perf_counter() - t0) * 1e3 / steps
        per_linear = {"ms_per_step": plain_ms, "launches_per_step": len(modules),
                      "how": "CUDA graph of 144 launches with programmatic dependent launch",
                      "eager_forward_ms_per_step": eager_ms}
        del plain

    # ---- secondary at N > 1: the same step without the all-reduce kernel (not a valid result, the
    # Down outputs stay partial): what the collective adds to the step.
    without_collective = None
    if world > 1:
        bare = GraphedLinears(modules, m=1)
        bare.x_flat.copy_(runner.x_flat)
        bare_total, _, _ = ctx.timed_replays(bare.replay, args.steps, 3)
        without_collective = {"ms_per_step": bare_total / args.steps,
                              "what": "the grouped launch alone, no all-reduce kernel (partial Down outputs)"}
        del bare

    status = _ops.device_status(device)
    if status != 0:
        raise SystemExit(f"device status {status}: a bounded wait expired inside a kernel")

    unit, per_layer = unit_and_amount("decode", 1, [0, 1, 2, 3])
    amount = per_layer * LAYERS  # whole job, all ranks together
    value = amount / (ms_per_step * 1e-3)
    if per_linear is not None:
        per_linear["value"] = amount / (per_linear["ms_per_step"] * 1e-3)
        per_linear["unit"] = unit
    launches = 1 if world == 1 else 2
    algorithmic_per_launch = amount * 1e9 / world
    ratio, source = traffic_ratio("w4a16_gemv_grouped_kernel")
    roofline = {"bound": "hbm", "achieved": value / world, "peak": ctx.peaks["hbm_gbs"], "unit": "GB/s",
                "frac": value / world / ctx.peaks["hbm_gbs"],
                "traffic": None if ratio is None else ratio * algorithmic_per_launch,
                "traffic_unit": "DRAM bytes (read + write) per launch", "traffic_source": source,
                "kernel": "w4a16_gemv_grouped_kernel", "peak_source": ctx.peaks["source"],
                "algorithmic_bytes_per_launch": algorithmic_per_launch,
                "per_launch": "one launch per step: this GPU's algorithmic bytes of the step over the step's CUDA-event time",
                "fraction_of_nominal_8tbs": value / world / 8000.0}
    block = {"value": value, "unit": unit, "ms_per_step": ms_per_step, "stats": summary(per_step),
             "roofline": roofline, "clocks": clocks,
             "e2e": {"value": amount / (e2e_ms * 1e-3), "unit": unit, "ms_per_step": e2e_ms,
                     "h2d_bytes_per_step": int(host_x.numel() * 2), "d2h_bytes_per_step": int(host_y.numel() * 2),
                     "api": "lowbitlinear_b200.graph.PipelinedLinears.submit: per step pinned host activations in, one "
                            "CUDA-graph replay (one grouped launch), host outputs out; two steps in flight",
                     "serial_ms_per_step": serial_ms,
                     "serial_api": "GraphedLinears.run: copy in, replay, copy out, wait -- one step at a time"},
             "gpu_launches": launches * args.steps,
             "launch": ("one grouped launch (lbl_w4a16_group_run) over the 144 independent linears"
                        + ("" if world == 1 else " + one all-reduce kernel over NVLink peer memory for the 36 Down outputs")),
             "per_linear_launch": per_linear, "without_collective": without_collective,
             "parity": {"rel_l2_vs_cpu_reference": parity, "tolerance": TOLERANCE, "checker": info["kind"]}}
    return block, runner, exchange


def run_prefill(ctx, layers, reference):
    """M = 2048: one launch per linear (TMA + tcgen05 GEMM); NCCL all-reduce of Down between ranks."""
    from lowbitlinear_b200 import _ops
    from lowbitlinear_b200.graph import GraphedLinears

    args, world, device = ctx.args, ctx.world, ctx.device
    m = PREFILL_M
    reduce = [name == "down" for name, _ in layers]
    modules = [layer for _, layer in layers]
    gemm_exchange = None
    if world > 1 and args.allreduce == "fused":
        from lowbitlinear_b200.tensor_parallel import PeerExchange
        gemm_exchange = PeerExchange.for_gemm(m, SHAPES[3][1], device)
    runner = GraphedLinears(modules, m=m, reduce=reduce, gemm_exchange=gemm_exchange)
    fused = gemm_exchange is not None and any(runner.fused)
    fill_activations(runner, layers, m, device, ctx.rank, world, None)
    # Layer 0: rows 0..3 of every activation are the CPU reference's M = 1 activations, so the
    # reference outputs of the decode leg check the GEMM as well.
    _, _, host_x0, expected = reference
    for idx, (name, n, k) in enumerate(SHAPES):
        x = host_x0[idx]
        if world > 1 and name == "down":
            part = layers[idx][1].in_features
            x = x[:, ctx.rank * part:(ctx.rank + 1) * part]
        runner.xs[idx][0:1].copy_(x.to(device))
    note("prefill: correctness")
    runner.replay()
    torch.cuda.synchronize()
    parity = {}
    for idx, (name, n, k) in enumerate(SHAPES):
        got = runner.ys[idx][0:1]
        want = expected[idx]
        if world > 1 and name != "down":
            cols = n // world
            want = want[:, ctx.rank * cols:(ctx.rank + 1) * cols]
        parity[name] = ctx.max_over_ranks(check_parity(got, want, f"layer 0 {name} (M={m}, row 0) vs the CPU reference"))
    if world > 1:
        # The all-reduced Down output (all 2048 rows) must be the same bits on every rank.
        mine = runner.ys[3].clone()
        theirs = mine.clone()
        ctx.dist.broadcast(theirs, src=0)
        same = torch.tensor([1.0 if torch.equal(mine, theirs) else 0.0], device=device)
        ctx.dist.all_reduce(same, op=ctx.dist.ReduceOp.MIN)
        parity["down_bit_identical_across_ranks"] = bool(same.item() == 1.0)
        if not parity["down_bit_identical_across_ranks"]:
            raise SystemExit("prefill: the all-reduced Down output differs between ranks")
        del mine, theirs
    for i in (6, 75):  # whole outputs of two other linears against an FP32 evaluation on the GPU
        name, layer = layers[i]
        if world > 1 and name == "down":
            continue
        kk = layer.in_features
        shifts = torch.arange(8, device=device) * 4
        q = ((layer.packed_weight.to(torch.int64)[..., None] >> shifts) & 15).reshape(layer.out_features, -1)[:, :kk]
        groups = torch.arange(kk, device=device) // 64
        w = (q.float() - layer.zeros[:, groups].float()) * layer.scales[:, groups]
        check_parity(runner.ys[i], (runner.xs[i].float() @ w.T).half(), f"linear {i} ({name}, M={m}) vs FP32 torch")
        del q, w

    note("prefill: timed region")
    total_ms, per_step, clocks = ctx.timed_replays(runner.replay, args.steps, args.warmup)
    ms_per_step = total_ms / args.steps
    without_collective = None
    if world > 1:
        # Secondary: the same 144 launches without the all-reduces (partial Down outputs, not a
        # valid result): what the collective adds to the step.
        saved = runner.x_flat.clone()
        del runner
        bare = GraphedLinears(modules, m=m)
        bare.x_flat.copy_(saved)
        bare_total, _, _ = ctx.timed_replays(bare.replay, args.steps, 3)
        without_collective = {"ms_per_step": bare_total / args.steps,
                              "what": "the 144 GEMM launches alone, no all-reduce (partial Down outputs)"}
        runner = bare  # the end-to-end leg below only needs its buffers' shapes and scratch
        del saved

    # ---- end to end: one layer at a time through the same pinned buffers (the activations of a
    # whole step would need 9 GB of pinned memory), so every layer is fed layer 0's activation
    # values; work and bytes moved per step are unchanged.
    chunk = len(SHAPES)
    x_elems = sum(runner.xs[i].numel() for i in range(chunk))
    y_elems = sum(runner.ys[i].numel() for i in range(chunk))
    host_x = torch.empty(x_elems, dtype=torch.float16).pin_memory()
    host_x.copy_(torch.cat([runner.xs[i].reshape(-1) for i in range(chunk)]).cpu())
    host_y = torch.empty(y_elems, dtype=torch.float16).pin_memory()
    # Two sets of device buffers and three streams: while layer c computes, the activations of layer
    # c + 1 come up and the outputs of layer c - 1 go down.  Every layer still makes its own copies.
    up, compute, down = (torch.cuda.Stream(device=device) for _ in range(3))
    sets = []
    for _ in range(2):
        dev_x = torch.empty(x_elems, dtype=torch.float16, device=device)
        dev_y = torch.empty(y_elems, dtype=torch.float16, device=device)
        x_views, y_views, xo, yo = [], [], 0, 0
        for i in range(chunk):
            x_views.append(dev_x[xo:xo + runner.xs[i].numel()].view_as(runner.xs[i]))
            y_views.append(dev_y[yo:yo + runner.ys[i].numel()].view_as(runner.ys[i]))
            xo += runner.xs[i].numel()
            yo += runner.ys[i].numel()
        sets.append({"x": dev_x, "y": dev_y, "xv": x_views, "yv": y_views, "uploaded": torch.cuda.Event(),
                     "computed": torch.cuda.Event(), "downloaded": torch.cuda.Event()})
    scratch = runner.scratch

    def e2e_step():
        for c in range(LAYERS):
            b = sets[c & 1]
            with torch.cuda.stream(up):
                if c >= 2:
                    up.wait_event(b["computed"])  # layer c - 2 has read this buffer
                b["x"].copy_(host_x, non_blocking=True)
                b["uploaded"].record(up)
            with torch.cuda.stream(compute):
                compute.wait_event(b["uploaded"])
                if c >= 2:
                    compute.wait_event(b["downloaded"])  # the outputs of layer c - 2 have left
                for j in range(chunk):
                    name, layer = layers[c * chunk + j]
                    if fused and name == "down":
                        _ops.gemm_allreduce(b["xv"][j], layer.packed_weight, layer.scales, layer.zeros, gemm_exchange,
                                            out=b["yv"][j])
                        continue
                    _ops.linear_out(b["xv"][j], layer.packed_weight, layer.scales, layer.zeros, b["yv"][j],
                                    workspace=scratch)
                    if world > 1 and name == "down":
                        ctx.dist.all_reduce(b["yv"][j])
                b["computed"].record(compute)
            with torch.cuda.stream(down):
                down.wait_event(b["computed"])
                host_y.copy_(b["y"], non_blocking=True)
                b["downloaded"].record(down)
        down.synchronize()
        compute.synchronize()

    e2e_ms = ctx.wall_steps(e2e_step, max(2, min(args.steps, 5)))
    status = _ops.device_status(device)
    if status != 0:
        raise SystemExit(f"device status {status}: a bounded wait expired inside a kernel")

    unit, per_layer = unit_and_amount("prefill", m, [0, 1, 2, 3])
    amount = per_layer * LAYERS
    value = amount / (ms_per_step * 1e-3)
    ratio, source = traffic_ratio("w4a16_gemm_tc_pair_kernel")
    algorithmic_per_launch = sum(linear_bytes(m, n, k) for _, n, k in SHAPES) / 4.0 / world
    roofline = {"bound": "tensor", "achieved": value / world, "peak": ctx.peaks["tflops_sustained"], "unit": "TFLOP/s",
                "frac": value / world / ctx.peaks["tflops_sustained"],
                "traffic": None if ratio is None else ratio * algorithmic_per_launch,
                "traffic_unit": "DRAM bytes (read + write) per average launch", "traffic_source": source,
                "kernel": "w4a16_gemm_tc_pair_kernel", "peak_source": ctx.peaks["source"] + " (sustained bf16 GEMM)",
                "per_launch": "this GPU's flops of the step / 144 launches over the step's CUDA-event time / 144",
                "fraction_of_nominal_2250": value / world / 2250.0}
    block = {"metric": metric_name("prefill"), "value": value, "unit": unit, "ms_per_step": ms_per_step,
             "stats": summary(per_step), "roofline": roofline, "clocks": clocks,
             "e2e": {"value": amount / (e2e_ms * 1e-3), "unit": unit, "ms_per_step": e2e_ms,
                     "h2d_bytes_per_step": int(x_elems * 2 * LAYERS), "d2h_bytes_per_step": int(y_elems * 2 * LAYERS),
                     "api": "lowbitlinear_b200._ops.linear_out per linear, eager; per layer its pinned host activations "
                            "in and its host outputs out, on upload / compute / download streams with two sets of "
                            "device buffers (the copies of neighbouring layers overlap the GEMMs)"},
             "gpu_launches": (len(layers) + (2 * LAYERS if fused else 0)) * args.steps,
             "launch": "CUDA graph of 144 launches" + (
                 "" if world == 1 else
                 " (Down: GEMM whose epilogue scatters its partial tiles to the owner ranks over NVLink) + 2 x 36 "
                 "reduce / gather kernels over peer memory on a side stream" if fused else
                 " with 36 NCCL all-reduces, issued asynchronously"),
             "without_collective": without_collective,
             "parity": {"rel_l2_vs_cpu_reference": parity, "tolerance": TOLERANCE}}
    if gemm_exchange is not None:
        del runner
        gemm_exchange.close()
    return block


def run_stack(args):
    ctx = Context(args)
    with torch.inference_mode():
        note("CPU reference leg")
        reference = reference_layer0(ctx)
        info = reference[0]
        note("building the stack")
        layers = build_layers(ctx.device, ctx.rank, ctx.world, reference[1])
        torch.cuda.synchronize()
        decode = prefill = None
        if args.workload in ("stack", "decode"):
            decode, runner, exchange = run_decode(ctx, layers, reference)
            del runner
        if args.workload in ("stack", "prefill"):
            prefill = run_prefill(ctx, layers, reference)
    if ctx.sampler is not None:
        ctx.sampler.close()
    if ctx.rank != 0:
        leave_process_group(ctx.world)
        return
    head = decode if decode is not None else prefill
    unit, amount = unit_and_amount("decode", 1, [0, 1, 2, 3])
    cpu_baseline = {"value": amount / info["seconds_per_pass"], "unit": unit,
                    "sample": f"layer 0 (QKV, O, Gate/Up, Down) at M=1, {len(info['times'])} passes of "
                              f"{info['seconds_per_pass']:.2f} s", **{k: info[k] for k in
                                                                     ("kind", "cores", "cpu_count", "cpu_model", "implementation")}}
    line = {"metric": metric_name(args.workload), "value": head["value"], "unit": head["unit"], "n_gpus": ctx.world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 activations x int4 weights, f32 accumulate", "data": "synthetic",
            "config": config_of(args.workload, ctx.world)}
    for key in ("stats", "roofline", "clocks", "e2e", "gpu_launches", "launch", "per_linear_launch",
                "without_collective", "parity"):
        if key in head:
            line[key] = head[key]
    line["cpu_baseline"] = cpu_baseline if ctx.world == 1 else None
    if decode is not None and prefill is not None:
        line["gemm"] = prefill
    print(json.dumps(line), flush=True)
    leave_process_group(ctx.world)


# ------------------------------------------------------------------------------------------------
# Kernel tables: crossover (config 3) and prefill sweep (config 4), single GPU
# ------------------------------------------------------------------------------------------------
def time_rotating(call, copies, replays, device):
    """µs per call of `call(i)` for i over `copies` distinct weight sets, captured back to back
    in one CUDA graph (programmatic dependent launch on), median over `replays` replays."""
    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        for i in range(copies):
            call(i)
    torch.cuda.current_stream(device).wait_stream(side)
    torch.cuda.synchronize(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(copies):
            call(i)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize(device)
    samples = []
    for _ in range(replays):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize(device)
        samples.append(start.elapsed_time(end) * 1e3 / copies)
    del graph
    return statistics.median(samples), min(samples)


def rotating_weights(n, k, copies, device, seed):
    from lowbitlinear_b200 import QuantizedLinear

    g = torch.Generator(device=device).manual_seed(seed)
    base = QuantizedLinear.from_float((torch.randn(n, k, device=device, generator=g) * WEIGHT_STD).half())
    sets = [(base.packed_weight, base.scales, base.zeros)]
    for _ in range(copies - 1):
        sets.append((base.packed_weight.clone(), base.scales.clone(), base.zeros.clone()))
    return sets


def reference_gpu_table(workload):
    """The reference's own CUDA operators on this GPU, timed in a process of their own."""
    if not any((REF_DIR / "lowbitlinear").glob("_C*")):
        return None
    result = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference_gpu", "--workload", workload],
                            capture_output=True, text=True)
    if result.returncode != 0:
        return {"unavailable": (result.stderr.strip().splitlines() or ["failed"])[-1][:300]}
    return json.loads(result.stdout.strip().splitlines()[-1])["rows"]


def run_tables(args):
    from lowbitlinear_b200 import _ops
    from lowbitlinear_b200._extension import load_cuda_extension

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU; there is no CPU fallback")
    load_cuda_extension(required=True)
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peaks = measured_peaks()
    sampler = ClockSampler(0, period_s=0.02)
    t_start = time.perf_counter()
    rows = []
    _ops.set_programmatic_dependent_launch(True)
    with torch.inference_mode():
        if args.workload == "crossover":
            paths = [("gemv", _ops.PATH_GEMV), ("gemm_tc_small", _ops.PATH_GEMM_TC_SMALL),
                     ("gemm_tc", _ops.PATH_GEMM_TC), ("dispatcher", _ops.PATH_AUTO)]
            for idx, (name, n, k) in enumerate(SHAPES):
                copies = max(3, -(-(300 << 20) // linear_bytes(1, n, k)))  # > 2 x L2 of weights in rotation
                sets = rotating_weights(n, k, copies, device, seed=idx)
                for m in (1, 2, 4, 8, 16, 32, 64):
                    g = torch.Generator(device=device).manual_seed(100 + m)
                    x = torch.randn(m, k, device=device, generator=g).half()
                    row = {"shape": name, "N": n, "K": k, "M": m, "algorithmic_bytes": linear_bytes(m, n, k),
                           "hbm_ideal_us": linear_bytes(m, n, k) / peaks["hbm_gbs"] / 1e3}
                    for label, path in paths:
                        if path == _ops.PATH_GEMV and m > 32:
                            continue
                        taken = []
                        # Scratch of exactly the size this path asks for, owned by this measurement.
                        need = max(_ops.workspace_bytes(m, n, k, path), _ops.workspace_bytes(m, n, k, _ops.PATH_GEMV_SPLITK))
                        scratch = torch.zeros(max(16, need), dtype=torch.uint8, device=device)

                        def call(i, path=path, taken=taken, scratch=scratch):
                            y, t = _ops.linear_forced(x, *sets[i], path, op=0 if m == 1 else 1, workspace=scratch)
                            taken.append(t)
                        us, best = time_rotating(call, copies, args.steps if args.steps != 200 else 30, device)
                        row[label] = {"us": us, "min_us": best, "gbs": linear_bytes(m, n, k) / us / 1e3,
                                      "frac_of_hbm": linear_bytes(m, n, k) / us / 1e3 / peaks["hbm_gbs"],
                                      "path": _ops.PATH_NAMES[taken[0]]}
                    if m <= 2:
                        # The same `copies` calls as ONE grouped launch (lbl_w4a16_group_run).
                        outs = [torch.empty(m, n, dtype=torch.float16, device=device) for _ in range(copies)]
                        group = _ops.LinearGroup([(x, *sets[i], outs[i]) for i in range(copies)])
                        us, best = time_rotating(lambda i: group.run() if i == 0 else None, copies,
                                                 args.steps if args.steps != 200 else 30, device)
                        row["grouped_launch"] = {"us": us, "min_us": best, "gbs": linear_bytes(m, n, k) / us / 1e3,
                                                 "frac_of_hbm": linear_bytes(m, n, k) / us / 1e3 / peaks["hbm_gbs"],
                                                 "path": f"one launch over the {copies} rotating weight sets"}
                        group.close()
                        del outs
                    forced = {k2: v["us"] for k2, v in row.items()
                              if isinstance(v, dict) and k2 not in ("dispatcher", "grouped_launch")}
                    row["dispatcher_is_fastest"] = row["dispatcher"]["us"] <= 1.03 * min(forced.values())
                    rows.append(row)
                del sets
        else:
            for idx, (name, n, k) in ((2, SHAPES[2]), (3, SHAPES[3])):
                sets = rotating_weights(n, k, 3, device, seed=idx)
                for m in (128, 512, 2048, 8192):
                    g = torch.Generator(device=device).manual_seed(100 + m)
                    x = torch.randn(m, k, device=device, generator=g).half()
                    out = torch.empty(m, n, dtype=torch.float16, device=device)
                    scratch = torch.zeros(max(16, _ops._lib.lbl_w4a16_workspace_bytes(m, n, k, _ops.PATH_AUTO)),
                                          dtype=torch.uint8, device=device)

                    def call(i):
                        _ops.linear_out(x, *sets[i], out, op=1, workspace=scratch)
                    us, best = time_rotating(call, 3, args.steps if args.steps != 200 else 30, device)
                    flops = linear_flops(m, n, k)
                    rows.append({"shape": name, "N": n, "K": k, "M": m, "us": us, "min_us": best,
                                 "tflops": flops / us / 1e6, "frac_of_sustained_bf16": flops / us / 1e6 / peaks["tflops_sustained"],
                                 "frac_of_nominal_2250": flops / us / 1e6 / 2250.0,
                                 "path": _ops.PATH_NAMES[_ops.select_path(m, n, k)]})
                    del out
                del sets
    _ops.set_programmatic_dependent_launch(False)
    status = _ops.device_status(device)
    if status != 0:
        raise SystemExit(f"device status {status}: a bounded wait expired inside a kernel")
    clocks = sampler.window(t_start, time.perf_counter())
    sampler.close()
    line = {"workload": args.workload, "n_gpus": 1, "rows": rows, "clocks": clocks, "peaks": peaks,
            "timing": "CUDA graph of back-to-back launches over rotating weight copies (> 2 x L2), programmatic "
                      "dependent launch, CUDA events around a replay, median of the replays",
            "reference_kernels_on_this_gpu": reference_gpu_table(args.workload)}
    print(json.dumps(line), flush=True)


def run_reference_gpu(args):
    """The reference's two CUDA operators (oracle/_ref, compiled for sm_100a) on the table shapes.
    This process imports the reference package only."""
    sys.path.insert(0, str(REF_DIR))
    import lowbitlinear  # noqa: F401  (loads the reference's own extension)
    from lowbitlinear import QuantizedLinear

    device = torch.device("cuda", 0)
    rows = []
    with torch.inference_mode():
        if args.workload == "crossover":
            cases = [(name, n, k, m) for name, n, k in SHAPES for m in (1, 2, 4, 8, 16, 32, 64)]
        else:
            cases = [(name, n, k, m) for name, n, k in SHAPES[2:] for m in (128, 512, 2048)]
        cache = {}
        for name, n, k, m in cases:
            if (n, k) not in cache:
                cache.clear()
                g = torch.Generator(device=device).manual_seed(n + k)
                base = QuantizedLinear.from_float((torch.randn(n, k, device=device, generator=g) * WEIGHT_STD).half())
                copies = max(3, -(-(300 << 20) // linear_bytes(1, n, k)))
                cache[(n, k)] = [base] + [QuantizedLinear(base.packed_weight.clone(), base.scales.clone(),
                                                          base.zeros.clone(), in_features=k) for _ in range(copies - 1)]
            layers = cache[(n, k)]
            x = torch.randn(m, k, device=device).half()
            us, best = time_rotating(lambda i: layers[i](x), len(layers), 10, device)
            rows.append({"shape": name, "M": m, "us": us, "min_us": best,
                         "operator": "w4a16_gemv_warp_vec" if m == 1 else "cute_w4a16 gemm"})
    print(json.dumps({"impl": "reference_gpu", "rows": rows}), flush=True)


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference", "reference_gpu"), default="ours")
    parser.add_argument("--workload", choices=("stack", "decode", "prefill", "crossover", "prefill_sweep"),
                        default="stack")
    parser.add_argument("--allreduce", choices=("fused", "nccl"), default="nccl",
                        help="prefill at N > 1: asynchronous NCCL all-reduces of the Down output (the faster of the "
                             "two on two GPUs, equal on four) or the all-reduce fused into the GEMM over peer memory")
    parser.add_argument("--emit", default=None, help=argparse.SUPPRESS)
    args = parser.parse_args()
    if args.impl == "reference":
        if args.steps == 200:
            args.steps = 5
        run_reference_arm(args)
    elif args.impl == "reference_gpu":
        run_reference_gpu(args)
    elif args.workload in ("crossover", "prefill_sweep"):
        run_tables(args)
    else:
        if args.steps == 200:
            args.steps = 50
        run_stack(args)


if __name__ == "__main__":
    main()
