"""Column-sharded matmul with the all-gather fused into the GEMM epilogue, on N GPUs of one host.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29540 \
      go-darwinml_b200/allgather_bench.py --gm 8192 --gn 8192 --gk 4096 [--iters 10]

Command line over go_darwinml_b200.sharding.column_sharded_matmul_check: every rank holds A [m, k] (replicated) and
its column block of W [k, n / world]; the fused kernel (b200_k_gemm_allgather) writes each rank's [m, n / world] slab
into every rank's full C over NVLink from inside the GEMM.  Checked bit for bit against this library's own single-GPU
GEMM on the full W, and timed beside GEMM + NCCL all-gather.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

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
    from go_darwinml_b200.sharding import column_sharded_matmul_check

    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    backend = b200.New(f"device={local}")
    res = column_sharded_matmul_check(backend, local, rank, world, args.gm, args.gn, args.gk, args.iters, args.warmup)
    if rank == 0:
        print(json.dumps(res), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
