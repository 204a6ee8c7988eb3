"""Sharding a quantised linear across GPUs: N-split (column parallel) and K-split (row parallel).

The reference has no multi-GPU code; these helpers sit on top of ``QuantizedLinear`` and do
not change it.  Quantisation is independent per (row, 64-column group), so cutting the packed
tensors gives exactly the bits that quantising the cut weight would give:

* column parallel -- rank r keeps rows ``[r N / g, (r + 1) N / g)`` of packed words, scales and
  zero points (contiguous row slices); the activation is replicated; outputs are the rank's
  column block of Y, optionally all-gathered along N.  No communication on the data path.
* row parallel    -- rank r keeps columns ``[r K / g, (r + 1) K / g)`` (a multiple of 64, so whole
  groups and whole packed words), made contiguous once; it multiplies its slice of the
  activation and the partial outputs are summed with an all-reduce.

One process per GPU; ``torch.distributed`` (NCCL on GPUs, gloo on CPU) carries the collectives.
For decode (M = 1) the K-split all-reduce can be fused into the GEMV kernel instead: each rank
leaves its FP32 partial vector in an exchange buffer that its peers map through CUDA IPC, and
the kernel's last CTA adds the ranks' vectors over NVLink (``PeerExchange``).
"""
import ctypes

import torch
import torch.distributed as dist

from .linear import QuantizedLinear


def _world(group):
    return dist.get_rank(group), dist.get_world_size(group)


def shard_column_parallel(layer, rank, world_size):
    """Rows ``[rank N / g, (rank + 1) N / g)`` of ``layer`` as a new ``QuantizedLinear``."""
    n = layer.out_features
    if n % world_size != 0:
        raise ValueError(f"out_features {n} is not divisible by {world_size} ranks")
    rows = slice(rank * n // world_size, (rank + 1) * n // world_size)
    return QuantizedLinear(
        layer.packed_weight[rows].contiguous(), layer.scales[rows].contiguous(),
        layer.zeros[rows].contiguous(), layer.group_size, in_features=layer.in_features)


def shard_row_parallel(layer, rank, world_size):
    """Columns ``[rank K / g, (rank + 1) K / g)`` of ``layer`` as a new ``QuantizedLinear``.

    The cut must fall on a group boundary that is also a packed-word boundary."""
    k, gs = layer.in_features, layer.group_size
    if k % world_size != 0:
        raise ValueError(f"in_features {k} is not divisible by {world_size} ranks")
    part = k // world_size
    if part % gs != 0 or part % 8 != 0:
        raise ValueError(f"K / ranks = {part} must be a multiple of group_size {gs} and of 8")
    words = slice(rank * part // 8, (rank + 1) * part // 8)
    groups = slice(rank * part // gs, (rank + 1) * part // gs)
    return QuantizedLinear(
        layer.packed_weight[:, words].contiguous(), layer.scales[:, groups].contiguous(),
        layer.zeros[:, groups].contiguous(), gs, in_features=part)


class PeerExchange:
    """Exchange buffers of all ranks of ``group`` for the fused K-split all-reduce (same node,
    one process per GPU).  Creating one is a collective call.  ``max_n`` bounds ``out_features``."""

    def __init__(self, max_n, device, group=None, gemm_shape=None):
        from . import _extension

        lib = _extension.native()
        self._lib = lib
        self.group = group
        self.rank, self.world = _world(group)
        self.capacity_n = int(max_n)
        self.device = torch.device(device)
        if gemm_shape is None:
            size = lib.lbl_peer_buffer_bytes(self.capacity_n)
        else:
            size = lib.lbl_peer_gemm_buffer_bytes(int(gemm_shape[0]), int(gemm_shape[1]), self.world)
            if size == 0:
                raise ValueError(f"no GEMM exchange for shape {tuple(gemm_shape)} on {self.world} ranks")
        self.bytes = int(size)
        self.gemm_shape = None if gemm_shape is None else (int(gemm_shape[0]), int(gemm_shape[1]))
        own = ctypes.c_void_p()
        self._check(lib.lbl_peer_buffer_create(size, self.device.index, ctypes.byref(own)))
        handle = (ctypes.c_ubyte * 64)()
        self._check(lib.lbl_peer_buffer_export(own, handle))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self._own = own
        self._opened = []
        pointers = []
        for r, raw in enumerate(handles):
            if r == self.rank:
                pointers.append(own.value)
                continue
            mapped = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(raw)
            self._check(lib.lbl_peer_buffer_open(buf, self.device.index, ctypes.byref(mapped)))
            self._opened.append(mapped)
            pointers.append(mapped.value)
        self.pointers = (ctypes.c_void_p * self.world)(*pointers)
        dist.barrier(group=group)  # every rank has mapped every buffer before the first kernel

    @classmethod
    def for_gemm(cls, max_m, n, device, group=None):
        """Exchange buffers for the large-M K-split GEMM with fused all-reduce: outputs of up to
        ``max_m`` rows and ``n`` columns (``n`` a multiple of 256 times the number of ranks)."""
        return cls(0, device, group, gemm_shape=(max_m, n))

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError(self._lib.lbl_last_error().decode())

    def close(self):
        """Unmap the peers' buffers and free this rank's.  A collective call: every rank waits for
        its own GPU and then for all the others before anything is unmapped, because a peer's last
        kernel may still be reading this rank's vector when this rank's own kernel has finished.
        Calling it again is a no-op."""
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for mapped in self._opened:
            self._lib.lbl_peer_buffer_close(mapped, self.device.index)
        self._opened = []
        self._lib.lbl_peer_buffer_destroy(self._own, self.device.index)
        self._own = None


class ColumnParallelLinear(torch.nn.Module):
    """N-split linear.  ``forward(x)`` takes the full activation ``[M, K]`` and returns this
    rank's ``[M, N / g]`` block, or the full ``[M, N]`` after an all-gather when
    ``gather_output`` is set."""

    def __init__(self, shard, group=None, gather_output=False):
        super().__init__()
        self.shard = shard
        self.group = group
        self.gather_output = gather_output

    @classmethod
    def from_full(cls, layer, group=None, gather_output=False):
        rank, world = _world(group)
        return cls(shard_column_parallel(layer, rank, world), group, gather_output)

    def forward(self, x):
        y = self.shard(x)
        if not self.gather_output:
            return y
        _, world = _world(self.group)
        if world == 1:
            return y
        # Ranks own column blocks: gather into [g, M, N/g] and interleave the blocks per row.
        m, n_local = y.shape
        gathered = torch.empty((world * m, n_local), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(gathered, y.contiguous(), group=self.group)
        return gathered.view(world, m, n_local).permute(1, 0, 2).reshape(m, world * n_local)


class RowParallelLinear(torch.nn.Module):
    """K-split linear.  ``forward(x_local)`` takes this rank's ``[M, K / g]`` slice of the
    activation (or the full ``[M, K]`` with ``input_is_parallel=False``) and returns the
    all-reduced ``[M, N]``."""

    def __init__(self, shard, group=None, input_is_parallel=True, exchange=None, gemm_exchange=None):
        super().__init__()
        self.shard = shard
        self.group = group
        self.input_is_parallel = input_is_parallel
        self.exchange = exchange  # PeerExchange: fuse the all-reduce into the decode kernel
        self.gemm_exchange = gemm_exchange  # PeerExchange.for_gemm: the same for large M

    @classmethod
    def from_full(cls, layer, group=None, input_is_parallel=True, exchange=None, gemm_exchange=None):
        rank, world = _world(group)
        return cls(shard_row_parallel(layer, rank, world), group, input_is_parallel, exchange, gemm_exchange)

    def _fused_gemm(self, x):
        ex, shard = self.gemm_exchange, self.shard
        if ex is None or not x.is_cuda or x.dtype != torch.float16 or not x.is_contiguous():
            return False
        m, n = x.shape[0], shard.out_features
        return (shard.group_size == 64 and m >= 256 and shard.in_features % 256 == 0
                and n % (256 * ex.world) == 0
                and 0 < ex._lib.lbl_peer_gemm_buffer_bytes(m, n, ex.world) <= ex.bytes)

    def _fused(self, x):
        shard = self.shard
        return (self.exchange is not None and x.is_cuda and x.shape[0] == 1 and shard.group_size == 64
                and shard.in_features % 256 == 0 and shard.out_features <= self.exchange.capacity_n
                and x.dtype == torch.float16 and x.is_contiguous())

    def check_status(self):
        """Synchronises this rank's GPU and raises if a bounded device-side wait expired since the
        last check -- for instance a peer that never reported to the fused all-reduce, whose
        outputs are then NaN."""
        from . import _ops

        status = _ops.device_status(self.shard.packed_weight.device)
        if status != 0:
            raise RuntimeError(f"device status {status}: a bounded wait inside a kernel expired "
                               "(110 = a tensor-parallel peer did not report in time)")

    def forward(self, x):
        rank, world = _world(self.group)
        if not self.input_is_parallel:
            part = self.shard.in_features
            x = x[:, rank * part:(rank + 1) * part].contiguous()
        if self._fused(x):
            from . import _ops

            return _ops.gemv_allreduce(x, self.shard.packed_weight, self.shard.scales,
                                       self.shard.zeros, self.exchange)
        if world > 1 and self._fused_gemm(x):
            from . import _ops

            return _ops.gemm_allreduce(x, self.shard.packed_weight, self.shard.scales, self.shard.zeros,
                                       self.gemm_exchange)
        y = self.shard(x)
        if world > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y
