"""Tests that need two GPUs of one host (skipped on a one-GPU box)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _need_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")


def test_fused_allgather_matmul_matches_single_gpu_gemm():
    """The column-sharded matmul whose all-gather runs inside the GEMM epilogue (peer stores over NVLink), two ranks."""
    _need_two_gpus()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29547", os.path.join(ROOT, "tests", "multi_rank_body.py"), "column_sharded", "1000", "1536", "512"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-3000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    res = json.loads(line)
    assert res["n_gpus"] == 2 and res["match_single_gpu_gemm_bitwise"] is True, res


def test_peer_copy_survives_freeing_and_reusing_the_source(b200, backend):
    """BufferCopyToDevice across GPUs (ref mpsgraph/gomlx/backend.go:165 returns an error: one device there).  The usual
    caller finalizes the source right after the copy; the source device's allocator hands the block out again at once,
    and new work on the source stream overwrites it.  The copy must still deliver the old contents."""
    _need_two_gpus()
    rng = np.random.default_rng(50)
    for trial in range(4):
        x = rng.standard_normal(48 << 20 >> 2).astype(np.float32)          # 48 MiB: the copy takes a while
        src = backend.FromNumpy(x, 0)
        dst = backend.BufferCopyToDevice(src, 1)
        assert backend.BufferDeviceNum(dst) == 1
        backend.BufferFinalize(src)
        clobber = backend.FromNumpy(np.full(x.shape, float(trial), dtype=np.float32), 0)   # same size: gets the freed block
        np.testing.assert_array_equal(backend.ToNumpy(dst), x)
        backend.BufferFinalize(clobber)
        backend.BufferFinalize(dst)
