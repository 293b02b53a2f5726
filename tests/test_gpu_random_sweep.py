"""Seeded random sweep over the shapes and layouts of the tensor-core paths: DotGeneral in its four storage forms
(aligned and ragged M / N, optional residual), FusedDense epilogues (bias, every activation, + / * with a same-shape
operand) and fused attention (odd sequence lengths, Sq != Sk, GQA ratios, both layouts), each against the CPU oracle."""
import ml_dtypes
import numpy as np
import pytest

from oracle.oracle import OracleFunction, compare
from tests.util import rng_array, run_backend, run_oracle

pytestmark = pytest.mark.gpu
BF16 = ml_dtypes.bfloat16


@pytest.mark.parametrize("seed", [11, 12])
def test_dot_general_random_shapes(b200, backend, seed):
    rng = np.random.default_rng(seed)
    for _ in range(12):
        B, M, N = int(rng.integers(1, 4)), int(rng.integers(1, 90)) * 8, int(rng.integers(1, 90)) * 8
        K = int(rng.choice([64, 200, 512, 1024, 1032, 2048]))
        if rng.random() < 0.3:
            N = int(rng.integers(8, 700))
        if rng.random() < 0.3:
            M = int(rng.integers(1, 700))
        form = str(rng.choice(["BMK_BKN", "BKM_BKN", "BMK_BNK", "BKM_BNK"]))
        dt = BF16 if rng.random() < 0.75 else np.float32
        a = rng_array(rng, (B, M, K) if form.startswith("BMK") else (B, K, M), dt)
        w = rng_array(rng, (B, K, N) if form.endswith("BKN") else (B, N, K), dt, 0.1)
        r = rng_array(rng, (B, M, N), dt)
        lc, rc = ([2] if form.startswith("BMK") else [1]), ([1] if form.endswith("BKN") else [2])
        use_res = bool(rng.random() < 0.5)

        def build(f, x, y, rr):
            d = f.DotGeneral(x, lc, [0], y, rc, [0])
            return f.Add(d, rr) if use_res else d

        (got,) = run_backend(b200, backend, build, [a, w, r])
        (want,) = run_oracle(build, [a, w, r])
        ok, viol = compare(got, want, 2e-2 if dt is BF16 else 1e-5, 1.0)
        assert ok, (B, M, N, K, form, np.dtype(dt).name, use_res, viol)


def test_dense_epilogues_random_shapes(b200, backend):
    rng = np.random.default_rng(13)
    for _ in range(14):
        M, N, K = int(rng.integers(1, 300)) * 8, int(rng.integers(1, 200)) * 8, int(rng.choice([128, 768, 1024, 3072]))
        if rng.random() < 0.3:
            N = int(rng.integers(8, 900))
        act, mode = int(rng.integers(0, 5)), int(rng.integers(0, 3))
        x, w = rng_array(rng, (M, K), BF16), rng_array(rng, (K, N), BF16, 0.05)
        bias, r = rng_array(rng, (N,), BF16), rng_array(rng, (M, N), BF16)

        def build(f, xx, ww, b_, rr):
            y = f.FusedDense(xx, ww, b_, act)
            return f.Add(rr, y) if mode == 1 else (f.Mul(y, rr) if mode == 2 else y)

        (got,) = run_backend(b200, backend, build, [x, w, bias, r])
        (want,) = run_oracle(build, [x, w, bias, r])
        ok, viol = compare(got, want, 2e-2, 1.0)
        assert ok, (M, N, K, act, mode, viol)


def test_attention_random_shapes(b200, backend):
    rng = np.random.default_rng(14)
    for _ in range(16):
        B, Hkv, rep = int(rng.integers(1, 4)), int(rng.choice([1, 2, 4])), int(rng.choice([1, 2, 4]))
        H = Hkv * rep
        Sq = int(rng.integers(1, 900))
        Sk = Sq if rng.random() < 0.7 else int(rng.integers(1, 900))
        causal = bool(rng.random() < 0.6) and Sq == Sk
        layout = int(rng.integers(0, 2))

        def shp(h, s):
            return (B, s, h, 64) if layout == 1 else (B, h, s, 64)

        q, k, v = rng_array(rng, shp(H, Sq), BF16), rng_array(rng, shp(Hkv, Sk), BF16), rng_array(rng, shp(Hkv, Sk), BF16)
        (got,) = run_backend(b200, backend, lambda f, qq, kk, vv: f.FusedScaledDotProductAttention(qq, kk, vv, None, H, Hkv, layout, 0.125, causal), [q, k, v])
        # the fused kernel keeps its scores in fp32: its reference is the oracle on fp32 copies of the inputs, rounded once
        want = OracleFunction().FusedScaledDotProductAttention(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), None, H, Hkv,
                                                               layout, 0.125, causal).astype(BF16)
        ok, viol = compare(got, want, 2e-2, 1.0)
        assert ok, (B, H, Hkv, Sq, Sk, causal, layout, viol)
