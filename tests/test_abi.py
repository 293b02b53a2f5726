"""CPU-side checks of the C ABI: the library loads, exports everything the header declares,
and refuses to compute without a GPU (there is no CPU fallback)."""
import ctypes
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "go-darwinml_b200", "libb200mlx.so")


def test_header_is_plain_c():
    # the header must compile as C (a cgo preamble includes it as C, not C++)
    src = '#include "b200mlx.h"\nint main(void){return 0;}\n'
    r = subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), "-x", "c", "-"],
                       input=src, text=True, capture_output=True)
    assert r.returncode == 0, r.stderr


def test_library_exports_every_declared_symbol(b200):
    L = b200.lib()
    assert len(L.decls) > 100
    dll = ctypes.CDLL(LIB)
    for name in L.decls:
        assert hasattr(dll, name), name


def test_no_torch_types_in_signatures(b200):
    for name, (ret, params) in b200.lib().decls.items():
        for p in [ret] + params:
            assert "at::" not in p and "torch" not in p and "Tensor" not in p, (name, p)


def test_version_string(b200):
    L = b200.lib()
    assert b"sm_100a" in ctypes.string_at(L.b200_version())


def _has_gpu(b200):
    from go_darwinml_b200 import _lib
    err = _lib.B200Error()
    n = b200.lib().b200_device_count(ctypes.byref(err))
    if err.code:
        b200.lib().free(err.message)
    return n > 0


def test_fails_loudly_without_gpu(b200):
    if _has_gpu(b200):
        pytest.skip("a GPU is present")
    with pytest.raises(b200.BackendError) as e:
        b200.New("")
    assert e.value.code == 2  # B200_ERR_CUDA
    from go_darwinml_b200 import _lib
    err = _lib.B200Error()
    ctx = b200.lib().b200_create_context(0, ctypes.byref(err))
    assert not ctx and err.code == 2
    assert "no CPU fallback" in b200.lib().take_string(err.message)


def test_unknown_backend_option_is_an_error(b200):
    with pytest.raises(b200.BackendError):
        b200.New("frobnicate=1")


def test_capabilities_lists_the_hot_path_ops(b200):
    from go_darwinml_b200.capabilities import backend_capabilities
    caps = backend_capabilities()
    for op in ("DotGeneral", "FusedSoftmax", "FusedLayerNorm", "FusedGelu", "FusedDense", "FusedScaledDotProductAttention",
               "FusedAttentionQKVProjection", "Iota", "Gather", "ArgMinMax", "ReduceSum", "Where", "ConvertDType"):
        assert caps.Operations.get(op), op
    assert caps.DTypes[int(b200.dtypes.BFloat16)] and caps.DTypes[int(b200.dtypes.Float32)]
