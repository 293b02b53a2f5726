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

    Ownership of C: every rank's kernel writes into every rank's C.  `run()` therefore opens with a synchronise and a
    barrier of its own -- a rank enters only when ITS consumers of the previous C have finished, and no rank's kernel
    starts before all have entered -- so a fast rank cannot overwrite a C that a slower rank is still reading.
    `launch()` has no such guard (it exists for back-to-back timing): its caller must make sure that every rank has
    finished reading C before any rank launches again.
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

        self.backend.Synchronize(self.device)   # this rank's readers of the previous C are done ...
        self._barrier()                          # ... and so are everybody else's: C may be overwritten
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


def column_sharded_matmul_check(backend, device: int, rank: int, world: int, gm: int, gn: int, gk: int, iters: int = 10, warmup: int = 3):
    """Runs ColumnShardedMatmul on bf16 A [gm, gk] (replicated) and W [gk, gn] split by columns over the ranks of an
    initialised torch.distributed NCCL group (one process per GPU), compares this rank's full C bit for bit with this
    library's single-GPU GEMM on the whole W, and times (CUDA events on the library's stream, max over ranks) the
    fused kernel beside the two-step form -- the same GEMM into a local slab, then all_gather_into_tensor -- and the
    GEMM alone.  Every rank returns the same dict."""
    import ctypes

    import ml_dtypes
    import torch
    import torch.distributed as dist

    from . import _lib as libmod
    from .backend import Buffer

    L = libmod.lib()
    if gn % (8 * world) != 0:
        raise ValueError("gn must be a multiple of 8 * world")
    n_local = gn // world
    dev = f"cuda:{device}"
    gen = torch.Generator(device=dev).manual_seed(1234)      # the same A and W on every rank
    a = (torch.randn(gm, gk, generator=gen, device=dev) * 0.5).to(torch.bfloat16)
    w = (torch.randn(gk, gn, generator=gen, device=dev) * 0.05).to(torch.bfloat16)
    w_local = w[:, rank * n_local:(rank + 1) * n_local].contiguous()
    code = 6   # BFloat16

    def wrap(t):
        err = libmod.B200Error()
        shape = (ctypes.c_int64 * t.dim())(*t.shape)
        return Buffer(L.b200_buffer_wrap(device, t.data_ptr(), code, shape, t.dim(), ctypes.byref(err)))

    def exchange(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    def gemm(a_t, w_t, out_t, n):
        e = libmod.B200Error()
        if not L.b200_k_gemm(device, a_t.data_ptr(), w_t.data_ptr(), out_t.data_ptr(), 1, gm, n, gk, 1, 0, code, None, 0, ctypes.byref(e)):
            raise RuntimeError(L.take_string(e.message))

    mm = ColumnShardedMatmul(backend, device, rank, world, gm, n_local, gk, np.dtype(ml_dtypes.bfloat16), exchange, dist.barrier)
    a_buf, w_buf = wrap(a), wrap(w_local)
    c_buf = mm.run(a_buf, w_buf)
    ref = torch.empty(gm, gn, device=dev, dtype=torch.bfloat16)
    gemm(a, w, ref, gn)
    backend.Synchronize(device)
    got = backend.ToNumpy(c_buf).view(np.uint16)
    match = bool(np.array_equal(got, ref.view(torch.int16).cpu().numpy().view(np.uint16)))
    del ref

    stream = torch.cuda.ExternalStream(L.b200_device_stream(device, ctypes.byref(libmod.B200Error())), device=device)

    def timed(fn):
        for _ in range(warmup):
            fn()
        backend.Synchronize(device)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            fn()
        e1.record(stream)
        backend.Synchronize(device)
        torch.cuda.synchronize()
        dist.barrier()
        return max_over_ranks([e0.elapsed_time(e1) / iters], device=dev)[0]

    # every launch writes the same values, so back-to-back launches without the guard of run() are safe here
    fused_ms = timed(lambda: mm.launch(a_buf, w_buf))
    slab = torch.empty(gm, n_local, device=dev, dtype=torch.bfloat16)
    gathered = torch.empty(world, gm, n_local, device=dev, dtype=torch.bfloat16)

    def two_step():
        gemm(a, w_local, slab, n_local)
        with torch.cuda.stream(stream):
            dist.all_gather_into_tensor(gathered, slab)     # leaves [world, m, n_local]: a transpose short of C

    two_ms = timed(two_step)
    gemm_only_ms = timed(lambda: gemm(a, w_local, slab, n_local))
    matches = exchange(match)
    mm.close()
    flops = 2.0 * gm * n_local * gk
    nvlink_bytes = (world - 1) * gm * n_local * 2
    return {"what": "column-sharded matmul, all-gather fused into the GEMM epilogue (peer stores over NVLink)", "n_gpus": world,
            "m": gm, "n": gn, "k": gk, "match_single_gpu_gemm_bitwise": all(matches), "fused_ms": fused_ms,
            "gemm_then_nccl_all_gather_ms": two_ms, "gemm_only_ms": gemm_only_ms, "fused_TFLOP/s_per_gpu": flops / (fused_ms * 1e-3) / 1e12,
            "nvlink_GB/s_out_per_gpu": nvlink_bytes / (fused_ms * 1e-3) / 1e9}
