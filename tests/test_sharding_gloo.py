"""The N>1 path on CPU: two gloo ranks shard a batch, time their shard and aggregate like bench.py does."""
import importlib.util
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _sharding():
    spec = importlib.util.spec_from_file_location("b200_sharding", os.path.join(ROOT, "go-darwinml_b200", "sharding.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["b200_sharding"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_shard_bounds_cover_the_batch_once():
    s = _sharding()
    for total in (0, 1, 7, 64, 65, 1000):
        for world in (1, 2, 3, 8):
            spans = [s.shard_bounds(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        s.shard_bounds(10, 2, 2)


def _free_port():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    s = _sharding()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle.oracle import OracleFunction
    rng = np.random.default_rng(0)
    logits = rng.standard_normal((5, 3, 16, 16)).astype(np.float32)     # ragged over two ranks: 3 + 2
    mine = s.shard_batch(logits, rank, world)
    part = OracleFunction().FusedSoftmaxMasked(mine, 1.0, True, None)    # a rank's shard needs nothing from the others
    np.save(os.path.join(out_dir, f"part{rank}.npy"), part)
    elapsed_ms = 10.0 * (rank + 1)                                       # rank 1 is the slow one
    value, worst = s.aggregate_throughput(float(mine.size), elapsed_ms)
    maxed = s.max_over_ranks([elapsed_ms, 1.0])
    dist.barrier()
    if rank == 0:
        np.save(os.path.join(out_dir, "agg.npy"), np.array([value, worst, maxed[0], maxed[1]]))
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_aggregate(tmp_path):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    from oracle.oracle import OracleFunction
    rng = np.random.default_rng(0)
    logits = rng.standard_normal((5, 3, 16, 16)).astype(np.float32)
    whole = OracleFunction().FusedSoftmaxMasked(logits, 1.0, True, None)
    parts = np.concatenate([np.load(tmp_path / "part0.npy"), np.load(tmp_path / "part1.npy")], axis=0)
    np.testing.assert_array_equal(parts, whole)                          # sharded result == unsharded result, bit for bit
    value, worst, m0, m1 = np.load(tmp_path / "agg.npy")
    assert worst == 20.0 and m0 == 20.0 and m1 == 1.0                     # max over ranks
    assert value == pytest.approx(logits.size / 20e-3)                    # all ranks' units / slowest rank's time


def test_column_sharded_matmul_rejects_bad_arguments_before_touching_a_gpu():
    # the constructor validates the layout first; these never reach the device
    import numpy as np
    import pytest

    from go_darwinml_b200.sharding import ColumnShardedMatmul

    def never(*_a, **_k):
        raise AssertionError("exchange / barrier must not be called for a rejected layout")

    with pytest.raises(ValueError, match="multiple of 8"):
        ColumnShardedMatmul(None, 0, 0, 2, 128, 12, 64, np.float16, never, never)
    with pytest.raises(ValueError, match="bad rank"):
        ColumnShardedMatmul(None, 0, 2, 2, 128, 16, 64, np.float16, never, never)
    with pytest.raises(ValueError, match="bad rank"):
        ColumnShardedMatmul(None, 0, 0, 9, 128, 16, 64, np.float16, never, never)
