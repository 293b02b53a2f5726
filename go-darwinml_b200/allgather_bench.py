"""Column-sharded matmul with the all-gather fused into the GEMM epilogue, on N GPUs of one host.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29540 \
      go-darwinml_b200/allgather_bench.py --gm 8192 --gn 8192 --gk 4096 [--iters 10]

Every rank holds A [m, k] (replicated) and its column block of W [k, n / world].  The fused kernel
(b200_k_gemm_allgather) writes each rank's [m, n / world] slab into every rank's full C over NVLink from inside the
GEMM.  Checked bit for bit against this library's own single-GPU GEMM on the full W, and timed (CUDA events on the
library's stream, max over ranks) beside the two-step form: the same GEMM into a local slab, then
torch.distributed.all_gather_into_tensor (NCCL).  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gm", type=int, default=8192)
    ap.add_argument("--gn", type=int, default=8192, help="total columns (split evenly over the ranks)")
    ap.add_argument("--gk", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    import go_darwinml_b200 as b200
    from go_darwinml_b200 import _lib as libmod
    from go_darwinml_b200.sharding import ColumnShardedMatmul, max_over_ranks

    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    backend = b200.New(f"device={local}")
    L = b200.lib()
    if args.gn % (8 * world) != 0:
        raise SystemExit("n must be a multiple of 8 * world")
    n_local = args.gn // world
    dev = f"cuda:{local}"
    gen = torch.Generator(device=dev).manual_seed(1234)      # the same A and W on every rank
    a = (torch.randn(args.gm, args.gk, generator=gen, device=dev) * 0.5).to(torch.bfloat16)
    w = (torch.randn(args.gk, args.gn, generator=gen, device=dev) * 0.05).to(torch.bfloat16)
    w_local = w[:, rank * n_local:(rank + 1) * n_local].contiguous()
    code = int(b200.dtypes.BFloat16)

    def wrap(t):
        err = libmod.B200Error()
        shape = (ctypes.c_int64 * t.dim())(*t.shape)
        return b200.Buffer(L.b200_buffer_wrap(local, t.data_ptr(), code, shape, t.dim(), ctypes.byref(err)))

    def exchange(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    import ml_dtypes
    mm = ColumnShardedMatmul(backend, local, rank, world, args.gm, n_local, args.gk, np.dtype(ml_dtypes.bfloat16), exchange, dist.barrier)
    a_buf, w_buf = wrap(a), wrap(w_local)
    c_buf = mm.run(a_buf, w_buf)

    # reference: the single-GPU GEMM of this library on the full weight
    ref = torch.empty(args.gm, args.gn, device=dev, dtype=torch.bfloat16)
    err = libmod.B200Error()
    ok = L.b200_k_gemm(local, a.data_ptr(), w.data_ptr(), ref.data_ptr(), 1, args.gm, args.gn, args.gk, 1, 0, code, None, 0, ctypes.byref(err))
    if not ok:
        raise RuntimeError(L.take_string(err.message))
    backend.Synchronize(local)
    got = backend.ToNumpy(c_buf).view(np.uint16)
    match = bool(np.array_equal(got, ref.view(torch.int16).cpu().numpy().view(np.uint16)))

    stream = torch.cuda.ExternalStream(L.b200_device_stream(local, ctypes.byref(libmod.B200Error())), device=local)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        backend.Synchronize(local)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.iters):
            fn()
        e1.record(stream)
        backend.Synchronize(local)
        torch.cuda.synchronize()
        dist.barrier()
        return max_over_ranks([e0.elapsed_time(e1) / args.iters], device=dev)[0]

    fused_ms = timed(lambda: mm.launch(a_buf, w_buf))

    slab = torch.empty(args.gm, n_local, device=dev, dtype=torch.bfloat16)
    gathered = torch.empty(world, args.gm, n_local, device=dev, dtype=torch.bfloat16)

    def two_step():
        e = libmod.B200Error()
        L.b200_k_gemm(local, a.data_ptr(), w_local.data_ptr(), slab.data_ptr(), 1, args.gm, n_local, args.gk, 1, 0, code, None, 0, ctypes.byref(e))
        with torch.cuda.stream(stream):
            dist.all_gather_into_tensor(gathered, slab)     # leaves [world, m, n_local]: a transpose short of C

    two_ms = timed(two_step)
    gemm_only_ms = timed(lambda: L.b200_k_gemm(local, a.data_ptr(), w_local.data_ptr(), slab.data_ptr(), 1, args.gm, n_local, args.gk, 1, 0, code, None,
                                                0, ctypes.byref(libmod.B200Error())))
    matches = [None] * world
    dist.all_gather_object(matches, match)
    if rank == 0:
        flops = 2.0 * args.gm * n_local * args.gk
        nvlink_bytes = (world - 1) * args.gm * n_local * 2
        print(json.dumps({
            "what": "column-sharded matmul, all-gather fused into the GEMM epilogue", "n_gpus": world, "m": args.gm, "n": args.gn, "k": args.gk,
            "match_single_gpu_gemm_bitwise": all(matches), "fused_ms": fused_ms, "gemm_then_nccl_all_gather_ms": two_ms, "gemm_only_ms": gemm_only_ms,
            "fused_TFLOP/s_per_gpu": flops / (fused_ms * 1e-3) / 1e12, "nvlink_GB/s_out_per_gpu": nvlink_bytes / (fused_ms * 1e-3) / 1e9,
        }), flush=True)
    mm.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
