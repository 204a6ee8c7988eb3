"""CUDA-graph runner for a set of quantised linears with static buffers.

``QuantizedLinear.forward`` re-validates its state and allocates its output on every call
(as the reference does, ``lowbitlinear/linear.py:95-129``); at decode sizes that host work costs
more than the kernels.  ``GraphedLinears`` validates once, captures the work of every layer into
one CUDA graph (``torch.cuda.CUDAGraph``: streams and graphs, no tracing compiler), and replays
it on demand:

    runner = GraphedLinears(layers, m=1)            # layers: list of QuantizedLinear on one GPU
    runner.run(host_x, host_y)                      # pinned flat FP16 buffers in, out

Each layer has its own activation ``[m, in_features]`` (views of one flat device buffer, in
layer order) and writes its ``[m, out_features]`` result into a flat output buffer, so one
host-to-device copy feeds a replay and one device-to-host copy returns everything.  The layers
are independent of each other.  For decode (``m <= 2``) the whole set is ONE persistent launch
(``_ops.LinearGroup``); otherwise one launch per layer with programmatic dependent launch.

Tensor parallel: give every rank its shards, flag the K-split (row-parallel) ones in ``reduce``
and pass the ranks' ``PeerExchange``; the flagged outputs are summed over the ranks by the
group's second kernel (decode) or by NCCL all-reduces captured in the graph (larger ``m``), issued
asynchronously so that they overlap the launches that follow.
"""
import torch

from . import _ops
from ._extension import load_cuda_extension
from .linear import _validate_packed_weight


class GraphedLinears:
    def __init__(self, layers, m=1, programmatic_dependent_launch=True, reduce=None, exchange=None,
                 group=None, grouped=None, gemm_exchange=None):
        load_cuda_extension(required=True)
        layers = list(layers)
        if not layers:
            raise ValueError("no layers")
        device = layers[0].packed_weight.device
        for layer in layers:
            _validate_packed_weight(layer.packed_weight, layer.scales, layer.zeros, layer.group_size,
                                    layer.in_features)
            if layer.group_size != 64 or not layer.packed_weight.is_cuda or layer.packed_weight.device != device:
                raise ValueError("GraphedLinears needs CUDA layers with group_size 64 on one device")
        self.layers = layers
        self.m = m
        self.device = device
        self.reduce = [False] * len(layers) if reduce is None else [bool(r) for r in reduce]
        if len(self.reduce) != len(layers):
            raise ValueError("reduce needs one entry per layer")
        self.process_group = group
        world = 1
        if any(self.reduce):
            import torch.distributed as dist

            if dist.is_available() and dist.is_initialized():
                world = dist.get_world_size(group)
        self.world = world
        # Offsets are multiples of 8 elements so that every view stays 16-byte aligned.
        pad = lambda v: (v + 7) // 8 * 8
        self.x_offsets, self.y_offsets = [], []
        x_total = y_total = 0
        for layer in layers:
            self.x_offsets.append(x_total)
            self.y_offsets.append(y_total)
            x_total += pad(m * layer.in_features)
            y_total += pad(m * layer.out_features)
        self.x_flat = torch.zeros(x_total, dtype=torch.float16, device=device)
        self.y_flat = torch.zeros(y_total, dtype=torch.float16, device=device)
        self.xs = [self.x_flat[o:o + m * l.in_features].view(m, l.in_features)
                   for o, l in zip(self.x_offsets, layers)]
        self.ys = [self.y_flat[o:o + m * l.out_features].view(m, l.out_features)
                   for o, l in zip(self.y_offsets, layers)]
        can_group = m <= 2 and all(l.in_features % 256 == 0 and m * l.in_features <= 32768 for l in layers)
        if grouped is None:
            grouped = can_group
        elif grouped and not can_group:
            raise ValueError("the grouped launch needs m <= 2, in_features % 256 == 0 and m * in_features <= 32768")
        self.grouped = grouped
        self.linear_group = None
        self.scratch = None
        if grouped:
            self.linear_group = _ops.LinearGroup(
                [(x, l.packed_weight, l.scales, l.zeros, y, r and world > 1)
                 for l, x, y, r in zip(layers, self.xs, self.ys, self.reduce)],
                exchange=exchange if world > 1 else None)
        else:
            # The runner owns its split-K scratch: the captured graph holds the raw pointer, so the
            # buffer must live exactly as long as the graph does.
            need = max(_ops._lib.lbl_w4a16_workspace_bytes(m, l.out_features, l.in_features, _ops.PATH_AUTO)
                       for l in layers)
            self.scratch = torch.zeros(max(need, 16), dtype=torch.uint8, device=device)
        # Large M, K-split layers: with a ``PeerExchange.for_gemm`` the partial outputs leave the GEMM's
        # epilogue for their owners over NVLink and the rest of the all-reduce (two small kernels)
        # runs on a side stream beside the following GEMMs; without one NCCL sums the outputs.
        self.gemm_exchange = gemm_exchange if (world > 1 and not grouped) else None
        self.fused = [False] * len(layers)
        if self.gemm_exchange is not None:
            ex = self.gemm_exchange
            for i, (layer, r) in enumerate(zip(layers, self.reduce)):
                need = ex._lib.lbl_peer_gemm_buffer_bytes(m, layer.out_features, ex.world)
                self.fused[i] = bool(r and m >= 256 and layer.in_features % 256 == 0
                                     and layer.out_features % (256 * ex.world) == 0 and 0 < need <= ex.bytes)
        self.side_stream = torch.cuda.Stream(device=device) if any(self.fused) else None
        self.stream = torch.cuda.Stream(device=device)
        self.graph = torch.cuda.CUDAGraph()
        previous = _ops._flags
        # Without the grouped launch the K-split outputs are summed by NCCL.  The all-reduces are
        # issued asynchronously (NCCL's own stream) and waited for at the end of the step, so they
        # overlap the launches that follow; programmatic dependent launch stays on between the
        # library's own kernels.
        _ops.set_programmatic_dependent_launch(programmatic_dependent_launch)
        # The layers of a runner are independent of each other (own activations, own outputs), so a
        # launch need not wait for the one before it: the tensor-core GEMMs fill each other's tails.
        _ops.set_independent_launches(programmatic_dependent_launch)
        try:
            self.stream.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(self.stream):
                self._forward()  # warm-up outside the capture
            torch.cuda.current_stream(device).wait_stream(self.stream)
            torch.cuda.synchronize(device)
            with torch.cuda.graph(self.graph, stream=self.stream):
                self._forward()
        finally:
            _ops._flags = previous

    def _forward(self):
        if self.grouped:
            self.linear_group.run()
            return
        pending = []
        main = torch.cuda.current_stream(self.device)
        exchanged = None  # event: the side stream has finished the previous fused all-reduce
        for layer, x, y, reduce, fused in zip(self.layers, self.xs, self.ys, self.reduce, self.fused):
            if fused:
                # One all-reduce per exchange at a time: the scattering GEMM follows the previous finish.
                if exchanged is not None:
                    main.wait_event(exchanged)
                _ops.gemm_scatter(x, layer.packed_weight, layer.scales, layer.zeros, self.gemm_exchange)
                scattered = torch.cuda.Event()
                scattered.record(main)
                self.side_stream.wait_event(scattered)
                with torch.cuda.stream(self.side_stream):
                    _ops.gemm_allreduce_finish(y, self.gemm_exchange)
                    exchanged = torch.cuda.Event()
                    exchanged.record(self.side_stream)
                continue
            _ops.linear_out(x, layer.packed_weight, layer.scales, layer.zeros, y, workspace=self.scratch)
            if reduce and self.world > 1:
                import torch.distributed as dist

                pending.append(dist.all_reduce(y, group=self.process_group, async_op=True))
        if exchanged is not None:
            main.wait_event(exchanged)
        for work in pending:
            work.wait()

    def replay(self):
        """Replay on the current stream with whatever ``x_flat`` holds; results in ``y_flat``."""
        self.graph.replay()

    def run(self, host_x, host_y):
        """``host_x`` -> device, replay, device -> ``host_y`` (flat FP16 tensors, ideally pinned),
        then wait for the copy.  Layout: ``x_offsets`` / ``y_offsets`` in elements."""
        self.x_flat.copy_(host_x, non_blocking=True)
        self.graph.replay()
        host_y.copy_(self.y_flat, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return host_y


class PipelinedLinears:
    """Two ``GraphedLinears`` over the same layers with separate static buffers, driven as a
    two-deep pipeline: while step *i* computes, the activations of step *i + 1* are copied up and
    the outputs of step *i - 1* are copied down, on a copy stream of their own.

        pipe = PipelinedLinears(layers, m=1)
        for host_x, host_y in steps:            # pinned flat FP16 buffers, two or more pairs in rotation
            pipe.submit(host_x, host_y)         # returns once step i is queued; step i - 2 has landed
        pipe.drain()                            # every submitted host_y is complete

    Every step still does its own host-to-device and device-to-host copy; only the waiting
    overlaps.  A ``host_y`` may be read after the second ``submit`` that follows its own, or after
    ``drain``.  Weights are shared between the two runners; the extra cost is a second set of
    activation and output buffers."""

    def __init__(self, layers, m=1, **kwargs):
        self.runners = [GraphedLinears(layers, m=m, **kwargs) for _ in range(2)]
        self.device = self.runners[0].device
        self.up_stream = torch.cuda.Stream(device=self.device)
        self.down_stream = torch.cuda.Stream(device=self.device)
        self.compute_stream = torch.cuda.Stream(device=self.device)
        self.uploaded = [torch.cuda.Event() for _ in range(2)]
        self.computed = [torch.cuda.Event() for _ in range(2)]
        self.downloaded = [torch.cuda.Event() for _ in range(2)]
        self.steps = 0

    def submit(self, host_x, host_y):
        slot = self.steps & 1
        runner = self.runners[slot]
        reused = self.steps >= 2
        if reused:
            # Bound the queue: the host runs at most two steps ahead of the copies coming back.
            self.downloaded[slot].synchronize()
        with torch.cuda.stream(self.up_stream):
            if reused:
                self.up_stream.wait_event(self.computed[slot])  # the slot's activations have been read
            runner.x_flat.copy_(host_x, non_blocking=True)
            self.uploaded[slot].record(self.up_stream)
        with torch.cuda.stream(self.compute_stream):
            self.compute_stream.wait_event(self.uploaded[slot])
            if reused:
                self.compute_stream.wait_event(self.downloaded[slot])  # the slot's outputs have left
            runner.graph.replay()
            self.computed[slot].record(self.compute_stream)
        with torch.cuda.stream(self.down_stream):
            self.down_stream.wait_event(self.computed[slot])
            host_y.copy_(runner.y_flat, non_blocking=True)
            self.downloaded[slot].record(self.down_stream)
        self.steps += 1

    def drain(self):
        self.up_stream.synchronize()
        self.compute_stream.synchronize()
        self.down_stream.synchronize()
