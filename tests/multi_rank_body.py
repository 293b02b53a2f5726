"""Rank body of the multi-GPU tests: launched by torch.distributed.run, one process per GPU.

  python -m torch.distributed.run --nproc-per-node 2 ... tests/multi_rank_body.py column_sharded 1000 1536 512
  python -m torch.distributed.run --nproc-per-node 2 ... tests/multi_rank_body.py peer_copy

Rank 0 prints one JSON line with what the test asserts on.
"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    import numpy as np
    import torch
    import torch.distributed as dist

    import go_darwinml_b200 as b200

    what = sys.argv[1]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    backend = b200.New(f"device={local}")
    if what == "column_sharded":
        from go_darwinml_b200.sharding import column_sharded_matmul_check
        gm, gn, gk = (int(v) for v in sys.argv[2:5])
        res = column_sharded_matmul_check(backend, local, rank, world, gm, gn, gk, iters=2, warmup=1)
    else:
        raise SystemExit(f"unknown body {what}")
    if rank == 0:
        print(json.dumps(res), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
