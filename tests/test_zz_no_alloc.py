"""The allocation-free sum reduction (b200_k_reduce_sum_f32_noalloc) against the regular entry point.

Some callers of this library cannot allocate device memory -- their memory budget is fixed at
start-up, or they sit in a loop that cannot pay for an allocation's implicit synchronisation --
so they cannot hand b200_k_reduce_sum_f32 the scratch buffer it wants.  The allocation-free entry
keeps that scratch in an array inside the library.  This file checks, through the C ABI, that it
returns what the regular entry returns, twice in a row (the array keeps the previous call's
partial sums, so the second call proves nothing stale leaks through), and that inputs beyond its
stated limit are refused.  The file name sorts last so that a run stopping at the first failure
has already run every other test.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _err(b200):
    from go_darwinml_b200 import _lib
    return _lib.B200Error()


def _check(b200, err):
    if err.code:
        raise AssertionError(b200.lib().take_string(err.message))


def _reduce_both_ways(b200, backend, x):
    L = b200.lib()
    n = x.size
    d_x = backend.FromNumpy(x)
    d_ref = backend.FromNumpy(np.zeros(1, dtype=np.float32))
    d_new = backend.FromNumpy(np.full(1, -123.0, dtype=np.float32))
    scratch_bytes = L.b200_k_reduce_sum_scratch_bytes(n)
    d_scratch = backend.FromNumpy(np.zeros(max(scratch_bytes, 4) // 4, dtype=np.float32))
    err = _err(b200)
    ok = L.b200_k_reduce_sum_f32(0, L.b200_buffer_device_ptr(d_x.handle), L.b200_buffer_device_ptr(d_ref.handle), n,
                                 L.b200_buffer_device_ptr(d_scratch.handle), scratch_bytes, ctypes.byref(err))
    _check(b200, err)
    assert ok
    err = _err(b200)
    ok = L.b200_k_reduce_sum_f32_noalloc(0, L.b200_buffer_device_ptr(d_x.handle), L.b200_buffer_device_ptr(d_new.handle), n,
                                         ctypes.byref(err))
    _check(b200, err)
    assert ok
    ref, new = backend.ToNumpy(d_ref)[0], backend.ToNumpy(d_new)[0]
    for b in (d_x, d_ref, d_new, d_scratch):
        backend.BufferFinalize(b)
    return float(ref), float(new), scratch_bytes


def test_noalloc_reduce_matches_regular_entry_twice_in_a_row(b200, backend):
    rng = np.random.default_rng(40)
    # first call: large enough to take the split path, so the built-in scratch is really used
    x1 = rng.standard_normal(3_000_000).astype(np.float32)
    ref1, new1, sb1 = _reduce_both_ways(b200, backend, x1)
    assert sb1 > 0
    np.testing.assert_allclose(new1, ref1, rtol=1e-5, atol=1e-3)
    np.testing.assert_allclose(new1, x1.astype(np.float64).sum(), rtol=1e-5, atol=1e-2)
    # second call, different size and data: the array still holds the first call's partial sums
    x2 = (rng.standard_normal(1_234_567) + 0.5).astype(np.float32)
    ref2, new2, sb2 = _reduce_both_ways(b200, backend, x2)
    assert sb2 > 0
    np.testing.assert_allclose(new2, ref2, rtol=1e-5, atol=1e-3)
    np.testing.assert_allclose(new2, x2.astype(np.float64).sum(), rtol=1e-5, atol=1e-2)


def test_noalloc_reduce_small_input_and_limit(b200, backend):
    x = np.arange(1000, dtype=np.float32)
    ref, new, _ = _reduce_both_ways(b200, backend, x)
    assert new == ref == float(x.sum())
    L = b200.lib()
    d = backend.FromNumpy(np.zeros(4, dtype=np.float32))
    err = _err(b200)
    ok = L.b200_k_reduce_sum_f32_noalloc(0, L.b200_buffer_device_ptr(d.handle), L.b200_buffer_device_ptr(d.handle), (1 << 30) + 1,
                                         ctypes.byref(err))
    assert not ok and err.code == 1
    assert "outside" in L.take_string(err.message)
    backend.BufferFinalize(d)


def test_noalloc_reduce_leaves_device_memory_untouched(b200, backend):
    """The point of the entry: a call on an initialised device takes no device memory, neither from the driver
    (free bytes as cudaMemGetInfo reports them) nor from this library's own pool (bytes reserved)."""
    import torch
    L = b200.lib()
    rng = np.random.default_rng(41)
    x = rng.standard_normal(2_000_000).astype(np.float32)
    d_x = backend.FromNumpy(x)
    d_out = backend.FromNumpy(np.zeros(1, dtype=np.float32))
    backend.Synchronize(0)
    free_before, _ = torch.cuda.mem_get_info(0)
    reserved_before = L.b200_device_bytes_reserved(0)
    for _ in range(3):
        err = _err(b200)
        ok = L.b200_k_reduce_sum_f32_noalloc(0, L.b200_buffer_device_ptr(d_x.handle), L.b200_buffer_device_ptr(d_out.handle), x.size,
                                             ctypes.byref(err))
        _check(b200, err)
        assert ok
    backend.Synchronize(0)
    free_after, _ = torch.cuda.mem_get_info(0)
    assert L.b200_device_bytes_reserved(0) == reserved_before
    assert free_after == free_before
    np.testing.assert_allclose(backend.ToNumpy(d_out)[0], x.astype(np.float64).sum(), rtol=1e-5, atol=1e-2)
    for b in (d_x, d_out):
        backend.BufferFinalize(b)
