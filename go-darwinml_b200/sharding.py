"""Batch sharding across GPUs: the path has no exchange step, so N GPUs run N independent shards.

The reference has one device and ignores sharding arguments (mpsgraph/gomlx/function.go:288, 343;
NumDevices() = 1, backend.go:56-57).  Every op on this path is independent along the leading batch
axis (rows of softmax / norms, the batch axis of DotGeneral, sequences of a forward pass), so the
multi-GPU form is: split axis 0, one replica of the executable per device, no collective on the data
path.  Two ways to drive it:

  * one process per GPU (bench.py under torchrun): `shard_bounds` picks this rank's rows and
    `max_over_ranks` / `aggregate_throughput` combine device-measured times over torch.distributed
    (NCCL on GPUs, gloo in the CPU tests);
  * one process, several devices (what a GoMLX program does through deviceNum): `BatchShardedRunner`
    compiles the graph once per device for its shard, places the shards, executes all replicas and
    concatenates the outputs on the host.
"""
from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

import numpy as np


def shard_bounds(total: int, rank: int, world: int) -> Tuple[int, int]:
    """[lo, hi) of `total` items owned by `rank`: an even split, the first total % world ranks get one more."""
    if world < 1 or not (0 <= rank < world) or total < 0:
        raise ValueError(f"bad shard request: total={total} rank={rank} world={world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(array: np.ndarray, rank: int, world: int, axis: int = 0) -> np.ndarray:
    lo, hi = shard_bounds(array.shape[axis], rank, world)
    index = [slice(None)] * array.ndim
    index[axis] = slice(lo, hi)
    return np.ascontiguousarray(array[tuple(index)])


def max_over_ranks(values: Sequence[float], device=None) -> List[float]:
    """Element-wise maximum of `values` over all ranks of the default process group (identity without one)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


def sum_over_ranks(values: Sequence[float], device=None) -> List[float]:
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return [float(v) for v in t]


def aggregate_throughput(units_this_rank: float, elapsed_ms_this_rank: float, device=None) -> Tuple[float, float]:
    """Whole-job throughput: (units of all ranks) / (slowest rank's time).  Returns (units per second, that time in ms)."""
    (total_units,) = sum_over_ranks([units_this_rank], device)
    (worst_ms,) = max_over_ranks([elapsed_ms_this_rank], device)
    return total_units / (worst_ms * 1e-3), worst_ms


class BatchShardedRunner:
    """One replica of a graph per device, inputs split on axis 0 (or replicated), outputs concatenated on axis 0."""

    def __init__(self, pkg, devices: Sequence[int], build: Callable, input_shapes: Sequence[Tuple[Tuple[int, ...], np.dtype]],
                 sharded: Sequence[bool]):
        """`build(f, *params)` builds the graph; input i is split on its axis 0 when sharded[i], else replicated (weights)."""
        self.pkg, self.devices, self.sharded = pkg, list(devices), list(sharded)
        self.replicas = []
        world = len(self.devices)
        for rank, dev in enumerate(self.devices):
            backend = pkg.New(f"device={dev}")
            builder = backend.Builder(f"replica{rank}")
            f = builder.Main()
            params = []
            for i, (shape, dt) in enumerate(input_shapes):
                shape = tuple(shape)
                if self.sharded[i]:
                    lo, hi = shard_bounds(shape[0], rank, world)
                    shape = (hi - lo,) + shape[1:]
                params.append(f.Parameter(f"p{i}", pkg.Shape(pkg.dtypes.from_numpy(np.dtype(dt)), shape)))
            out = build(f, *params)
            f.Return(list(out) if isinstance(out, (list, tuple)) else [out], None)
            self.replicas.append((backend, builder, builder.Compile()))

    def __call__(self, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
        world = len(self.devices)
        pending = []
        for rank, (backend, _, exe) in enumerate(self.replicas):
            dev = self.devices[rank]
            bufs = [backend.FromNumpy(shard_batch(a, rank, world) if self.sharded[i] else a, dev) for i, a in enumerate(inputs)]
            pending.append((backend, bufs, exe.Execute(bufs, None, dev)))   # enqueues and returns: replicas overlap
        per_rank = []
        for backend, bufs, outs in pending:
            per_rank.append([backend.ToNumpy(o) for o in outs])
            for b in bufs + outs:
                backend.BufferFinalize(b)
        return [np.concatenate([r[j] for r in per_rank], axis=0) for j in range(len(per_rank[0]))]

    def close(self):
        for backend, builder, exe in self.replicas:
            exe.Finalize()
            builder.Finalize()


class ColumnShardedMatmul:
    """The one exchange step this path may have: a weight too wide for one GPU is split by columns, every rank
    multiplies the (replicated) activations by its column block, and every rank needs the full result.

    The usual form is GEMM then all-gather.  Here the all-gather is inside the GEMM: each rank's result buffer
    C [m, world * n_local] is exported once to the other ranks of the host (`b200_buffer_ipc_export` / `_import`),
    and `b200_k_gemm_allgather`'s epilogue stores every tile of the local [m, n_local] slab into ALL ranks' buffers,
    its own and the peers' (plain stores over NVLink), while later tiles are still being multiplied.  After the
    kernel each rank synchronises its stream and the ranks meet at a host barrier; nothing else is exchanged.

    `exchange(obj) -> list` must return every rank's `obj` in rank order (torch.distributed.all_gather_object does);
    `barrier()` must return once all ranks have called it.  One process per GPU.
    """

    def __init__(self, backend, device: int, rank: int, world: int, m: int, n_local: int, k: int, np_dtype,
                 exchange: Callable[[bytes], List[bytes]], barrier: Callable[[], None], b_k_major: bool = False):
        import ctypes

        from . import _lib, dtypes
        from .backend import Buffer, _check, _i64

        if world < 1 or world > 8 or not (0 <= rank < world):
            raise ValueError(f"bad rank {rank} of {world}")
        if n_local % 8 != 0:
            raise ValueError("n_local must be a multiple of 8 (16-byte stores)")
        self.backend, self.device, self.rank, self.world = backend, device, rank, world
        self.m, self.n_local, self.k, self.b_k_major = m, n_local, k, bool(b_k_major)
        self._L = _lib.lib()
        self._barrier = barrier
        self.dtype = dtypes.from_numpy(np.dtype(np_dtype))
        shape = (m, n_local * world)
        err = _lib.B200Error()
        handle = self._L.b200_buffer_alloc(device, int(self.dtype), _i64(shape), 2, ctypes.byref(err))
        _check(err, "ColumnShardedMatmul: alloc")
        self.c = Buffer(handle)
        raw = ctypes.create_string_buffer(64)
        self._L.b200_buffer_ipc_export(self.c.handle, raw, ctypes.byref(err))
        _check(err, "ColumnShardedMatmul: export")
        handles = exchange(bytes(raw.raw))
        if len(handles) != world:
            raise ValueError(f"exchange returned {len(handles)} handles for {world} ranks")
        self._imported = []
        self._views = []
        for r in range(world):
            if r == rank:
                self._views.append(self.c)
                continue
            err = _lib.B200Error()
            h = self._L.b200_buffer_ipc_import(device, handles[r], int(self.dtype), _i64(shape), 2, ctypes.byref(err))
            _check(err, f"ColumnShardedMatmul: import from rank {r}")
            buf = Buffer(h)
            self._imported.append(buf)
            self._views.append(buf)
        ptrs = [self._L.b200_buffer_device_ptr(v.handle) for v in self._views]
        self._c_all = (ctypes.c_void_p * world)(*ptrs)
        barrier()   # nobody launches before every rank has mapped every buffer

    def run(self, a, b_local) -> "object":
        """a: Buffer [m, k]; b_local: Buffer [k, n_local] (or [n_local, k] with b_k_major).  Enqueues the kernel, waits
        for this rank's stream and for the other ranks, and returns this rank's full C [m, world * n_local]."""
        import ctypes

        from . import _lib
        from .backend import _check

        err = _lib.B200Error()
        self._L.b200_k_gemm_allgather(self.device, self._L.b200_buffer_device_ptr(a.handle), self._L.b200_buffer_device_ptr(b_local.handle),
                                      self._c_all, self.world, self.rank, self.m, self.n_local, self.k, 1, int(self.b_k_major),
                                      int(self.dtype), ctypes.byref(err))
        _check(err, "ColumnShardedMatmul: gemm_allgather")
        self.backend.Synchronize(self.device)
        self._barrier()
        return self.c

    def launch(self, a, b_local) -> None:
        """Only enqueues the kernel (for timing with device events); the caller synchronises and calls the barrier."""
        import ctypes

        from . import _lib
        from .backend import _check

        err = _lib.B200Error()
        self._L.b200_k_gemm_allgather(self.device, self._L.b200_buffer_device_ptr(a.handle), self._L.b200_buffer_device_ptr(b_local.handle),
                                      self._c_all, self.world, self.rank, self.m, self.n_local, self.k, 1, int(self.b_k_major),
                                      int(self.dtype), ctypes.byref(err))
        _check(err, "ColumnShardedMatmul: gemm_allgather")

    def close(self) -> None:
        """Unmaps the peers' buffers, waits for everybody to have done so, then frees this rank's."""
        self.backend.Synchronize(self.device)
        for buf in self._imported:
            self.backend.BufferFinalize(buf)
        self._imported = []
        self._barrier()
        self.backend.BufferFinalize(self.c)
