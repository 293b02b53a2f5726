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
