"""Helpers shared by the tests: run one graph-building routine on the backend and on the oracle."""
from __future__ import annotations

import numpy as np

from oracle.oracle import OracleFunction, compare


def default_switches():
    """True unless an environment switch (B200MLX_...=0) selects a non-default code path: the plan-shape assertions of the
    GPU tests hold for the default paths only, the numerical ones for every path."""
    import os
    return not any(k.startswith("B200MLX_") and v[:1] == "0" for k, v in os.environ.items())


def run_backend(pkg, backend, build, inputs, describe=False):
    builder = backend.Builder("test")
    f = builder.Main()
    params = [f.Parameter(f"p{i}", pkg.Shape(pkg.dtypes.from_numpy(a.dtype), a.shape)) for i, a in enumerate(inputs)]
    out = build(f, *params)
    outs = list(out) if isinstance(out, (list, tuple)) else [out]
    f.Return(outs, None)
    exe = builder.Compile()
    bufs = [backend.FromNumpy(a) for a in inputs]
    try:
        res = exe.Execute(bufs, None, 0)
        arrays = [backend.ToNumpy(r) for r in res]
        for r in res:
            backend.BufferFinalize(r)
    finally:
        for b in bufs:
            backend.BufferFinalize(b)
    plan = exe.Describe() if describe else None
    exe.Finalize()
    builder.Finalize()
    return (arrays, plan) if describe else arrays


def run_oracle(build, inputs):
    out = build(OracleFunction(), *inputs)
    return list(out) if isinstance(out, (list, tuple)) else [out]


def assert_parity(pkg, backend, build, inputs, rtol=1e-5, atol_scale=0.0, what=""):
    got = run_backend(pkg, backend, build, inputs)
    want = run_oracle(build, inputs)
    assert len(got) == len(want)
    for i, (g, w) in enumerate(zip(got, want)):
        w = np.asarray(w)
        assert g.shape == w.shape, f"{what}[{i}]: shape {g.shape} vs oracle {w.shape}"
        assert g.dtype == w.dtype, f"{what}[{i}]: dtype {g.dtype} vs oracle {w.dtype}"
        ok, viol = compare(g, w, rtol, atol_scale)
        assert ok, f"{what}[{i}]: differs from the oracle (worst violation {viol:.3e}, rtol {rtol})"
    return got


def rng_array(rng, shape, dtype, scale=1.0):
    import ml_dtypes
    if np.dtype(dtype).kind in "iu":
        info = np.iinfo(dtype)
        return rng.integers(max(info.min, -1000), min(info.max, 1000), size=shape, dtype=np.int64).astype(dtype)
    if np.dtype(dtype) == np.bool_:
        return rng.integers(0, 2, size=shape).astype(np.bool_)
    x = (rng.standard_normal(size=shape) * scale).astype(np.float32)
    return x.astype(dtype)
