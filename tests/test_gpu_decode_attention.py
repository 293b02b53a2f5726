"""Attention of one query position over a key / value cache (a decoding step), with and without a mask tensor.

One launch reads the cache once; the scores stay in fp32.  The yardstick is the oracle on the same inputs in fp32,
rounded once at the end (the unfused lowering rounds the scores to the storage type before the softmax).
"""
import ml_dtypes
import numpy as np
import pytest

from oracle.oracle import OracleFunction, compare
from tests.util import default_switches, rng_array, run_backend

pytestmark = pytest.mark.gpu
BF16 = ml_dtypes.bfloat16
RTOL = 2e-2


def _case(b200, backend, B, H, Hkv, Sk, layout, dtype, mask, seed=0, scale=0.125, expect_fused=True):
    rng = np.random.default_rng(seed)
    D = 64
    shp = (lambda h, s: (B, h, s, D)) if layout == 0 else (lambda h, s: (B, s, h, D))
    q, k, v = rng_array(rng, shp(H, 1), dtype), rng_array(rng, shp(Hkv, Sk), dtype), rng_array(rng, shp(Hkv, Sk), dtype)
    inputs = [q, k, v] + ([mask] if mask is not None else [])
    build = lambda f, qq, kk, vv, mm=None: f.FusedScaledDotProductAttention(qq, kk, vv, mm, H, Hkv, layout, scale, False)
    (got,), plan = run_backend(b200, backend, build, inputs, describe=True)
    if expect_fused:
        assert (plan.startswith("attention_decode[") and plan.count("\n") == 1) or not default_switches(), plan
    m32 = None if mask is None else (mask if mask.dtype == np.bool_ else mask.astype(np.float32))
    want = OracleFunction().FusedScaledDotProductAttention(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), m32, H, Hkv,
                                                           layout, scale, False).astype(dtype)
    ok, viol = compare(got, want, RTOL, 1.0)
    assert ok, viol
    return got, plan


@pytest.mark.parametrize("layout", [0, 1], ids=["BHSD", "BSHD"])
@pytest.mark.parametrize("H,Hkv", [(2, 2), (4, 2), (8, 2), (8, 1), (12, 1)])   # groups of 1, 2, 4, 8 (shared K / V loads) and 12
@pytest.mark.parametrize("Sk", [1, 7, 64, 257, 1000, 1024, 5000])
def test_one_query_without_a_mask(b200, backend, layout, H, Hkv, Sk):
    _case(b200, backend, 2, H, Hkv, Sk, layout, BF16, None, seed=Sk)


@pytest.mark.parametrize("layout", [0, 1], ids=["BHSD", "BSHD"])
@pytest.mark.parametrize("mask_shape", ["k", "1k", "b11k", "bh1k", "1h1k", "111k"])
@pytest.mark.parametrize("kind", ["bool", "additive"])
def test_one_query_with_a_mask_of_every_broadcast_shape(b200, backend, layout, mask_shape, kind):
    B, H, Hkv, Sk = 3, 4, 2, 300
    rng = np.random.default_rng(11)
    # rank-4 masks follow the tensors' layout: [B, H, 1, Sk] in BHSD, [B, 1, H, Sk] in BSHD
    dims = {"k": (Sk,), "1k": (1, Sk), "b11k": (B, 1, 1, Sk), "111k": (1, 1, 1, Sk),
            "bh1k": (B, H, 1, Sk) if layout == 0 else (B, 1, H, Sk),
            "1h1k": (1, H, 1, Sk) if layout == 0 else (1, 1, H, Sk)}[mask_shape]
    if kind == "bool":
        mask = rng.integers(0, 4, size=dims) > 0
        mask[..., 0] = True    # no fully masked row here
    else:
        mask = (rng.standard_normal(size=dims) * 2).astype(BF16)
    _case(b200, backend, B, H, Hkv, Sk, layout, BF16, mask, seed=3)


def test_grouped_heads_with_a_mask_per_head(b200, backend):
    # the heads of a group share K and V but not the mask
    rng = np.random.default_rng(21)
    B, H, Hkv, Sk = 2, 8, 2, 700
    mask = rng.integers(0, 3, size=(B, H, 1, Sk)) > 0
    mask[..., 5] = True
    _case(b200, backend, B, H, Hkv, Sk, 0, BF16, mask, seed=22)
    add = (rng.standard_normal(size=(1, 1, H, Sk)) * 2).astype(BF16)   # BSHD: [B, 1, H, Sk]
    _case(b200, backend, B, H, Hkv, Sk, 1, BF16, add, seed=23)


def test_f16_tensors_and_an_f16_additive_mask(b200, backend):
    rng = np.random.default_rng(5)
    mask = (rng.standard_normal(size=(2, 1, 1, 777)) * 3).astype(np.float16)
    _case(b200, backend, 2, 8, 4, 777, 0, np.float16, mask, seed=6)
    _case(b200, backend, 2, 8, 4, 777, 1, np.float16, None, seed=7)


def test_position_mask_of_a_cache_filled_up_to_t(b200, backend):
    # the decoding workload's mask: key position <= t; everything past t holds garbage that must not leak
    B, H, Sk, t = 4, 12, 1024, 37
    rng = np.random.default_rng(9)
    q, k, v = rng_array(rng, (B, H, 1, 64), BF16), rng_array(rng, (B, H, Sk, 64), BF16), rng_array(rng, (B, H, Sk, 64), BF16)
    k[:, :, t + 1:, :] = BF16(1e30)
    v[:, :, t + 1:, :] = BF16(-1e30)
    mask = (np.arange(Sk) <= t).reshape(1, 1, 1, Sk)
    build = lambda f, qq, kk, vv, mm: f.FusedScaledDotProductAttention(qq, kk, vv, mm, H, H, 0, 0.125, False)
    (got,), plan = run_backend(b200, backend, build, [q, k, v, mask], describe=True)
    assert ("attention_decode[" in plan and "mask=Bool" in plan) or not default_switches(), plan
    want = OracleFunction().FusedScaledDotProductAttention(q.astype(np.float32)[...], k.astype(np.float32)[:, :, :t + 1], v.astype(np.float32)[:, :, :t + 1],
                                                           None, H, H, 0, 0.125, False).astype(BF16)
    ok, viol = compare(got, want, RTOL, 1.0)
    assert ok, viol


def test_fully_masked_rows_are_nan_and_the_others_are_not(b200, backend):
    B, H, Sk = 2, 4, 600
    mask = np.ones((B, H, 1, Sk), dtype=np.bool_)
    mask[1, 2] = False
    rng = np.random.default_rng(2)
    q, k, v = rng_array(rng, (B, H, 1, 64), BF16), rng_array(rng, (B, H, Sk, 64), BF16), rng_array(rng, (B, H, Sk, 64), BF16)
    build = lambda f, qq, kk, vv, mm: f.FusedScaledDotProductAttention(qq, kk, vv, mm, H, H, 0, 0.125, False)
    (got,) = run_backend(b200, backend, build, [q, k, v, mask])
    g = got.astype(np.float32)
    assert np.isnan(g[1, 2]).all()
    g[1, 2] = 0
    assert np.isfinite(g).all()


def test_masked_chunks_before_the_first_visible_key(b200, backend):
    # the running maximum stays -inf through whole 256-key chunks and across CTAs of the cluster
    B, H, Sk = 1, 2, 4096
    mask = np.zeros((1, 1, 1, Sk), dtype=np.bool_)
    mask[..., 3000:3010] = True
    _case(b200, backend, B, H, H, Sk, 0, BF16, mask, seed=8)


def test_large_scores_do_not_overflow(b200, backend):
    B, H, Sk = 2, 2, 513
    rng = np.random.default_rng(4)
    q = (rng.standard_normal((B, H, 1, 64)) * 30).astype(BF16)
    k = (rng.standard_normal((B, H, Sk, 64)) * 30).astype(BF16)
    v = rng_array(rng, (B, H, Sk, 64), BF16)
    build = lambda f, qq, kk, vv: f.FusedScaledDotProductAttention(qq, kk, vv, None, H, H, 0, 1.0, False)
    (got,) = run_backend(b200, backend, build, [q, k, v])
    want = OracleFunction().FusedScaledDotProductAttention(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), None, H, H, 0, 1.0,
                                                           False).astype(BF16)
    ok, viol = compare(got, want, RTOL, 1.0)
    assert ok, viol


def test_a_mask_with_several_query_positions_takes_the_general_lowering(b200, backend):
    B, H, Sq, Sk = 2, 2, 5, 40
    rng = np.random.default_rng(1)
    q, k, v = rng_array(rng, (B, H, Sq, 64), BF16), rng_array(rng, (B, H, Sk, 64), BF16), rng_array(rng, (B, H, Sk, 64), BF16)
    mask = rng.integers(0, 3, size=(Sq, Sk)) > 0
    mask[:, 0] = True
    build = lambda f, qq, kk, vv, mm: f.FusedScaledDotProductAttention(qq, kk, vv, mm, H, H, 0, 0.125, False)
    (got,), plan = run_backend(b200, backend, build, [q, k, v, mask], describe=True)
    assert "attention" not in plan and "softmax" in plan, plan
    want = OracleFunction().FusedScaledDotProductAttention(q, k, v, mask, H, H, 0, 0.125, False)
    ok, viol = compare(got, want, RTOL, 1.0)
    assert ok, viol


def test_query_and_cache_updates_are_read_in_place_inside_the_fused_projection(b200, backend):
    # a decoding step's attention block: one fused projection, K and V written into the caches at position t, the query
    # attended over the caches -- no Slice of the projection is ever copied
    B, H, S, D, t = 3, 4, 40, 64, 17
    d = H * D
    rng = np.random.default_rng(12)
    x = rng_array(rng, (B, 1, d), BF16)
    wqkv = rng_array(rng, (d, 3 * d), BF16, 1.0 / np.sqrt(d))
    kc, vc = rng_array(rng, (B, H, S, D), BF16), rng_array(rng, (B, H, S, D), BF16)
    mask = (np.arange(S) <= t).reshape(1, 1, 1, S)
    pos = np.array(t, dtype=np.int32)

    def build(f, xx, w, kcache, vcache, m, p):
        q, k, v = f.FusedAttentionQKVProjection(xx, w, None, None, None, d, d)
        heads = lambda a: f.Reshape(a, B, H, 1, D)
        zero = f.Constant(np.array([0], dtype=np.int32))
        kc2 = f.DynamicUpdateSlice(kcache, heads(k), [zero, zero, p, zero])
        vc2 = f.DynamicUpdateSlice(vcache, heads(v), [zero, zero, p, zero])
        o = f.FusedScaledDotProductAttention(heads(q), kc2, vc2, m, H, H, 0, 0.125, False)
        return [o, kc2, vc2]

    inputs = [x, wqkv, kc, vc, mask, pos]
    got, plan = run_backend(b200, backend, build, inputs, describe=True)
    # (the key and the value cache are updated by one step: the second update joins the first)
    assert ("move[Slice" not in plan and "update read in place + a second one, read in place" in plan and "attention_decode[" in plan) or not default_switches(), plan
    from tests.util import run_oracle
    want = run_oracle(build, inputs)
    np.testing.assert_array_equal(got[1].view(np.uint16), want[1].view(np.uint16))
    np.testing.assert_array_equal(got[2].view(np.uint16), want[2].view(np.uint16))
    # attention output against the fp32-scores yardstick on the updated caches
    qh = (x.astype(np.float32).reshape(B, d) @ wqkv.astype(np.float32))[:, :d].astype(BF16).reshape(B, H, 1, D)
    ref = OracleFunction().FusedScaledDotProductAttention(qh.astype(np.float32), want[1].astype(np.float32), want[2].astype(np.float32), mask, H, H, 0,
                                                          0.125, False).astype(BF16)
    ok, viol = compare(got[0], ref, RTOL, 1.0)
    assert ok, viol
