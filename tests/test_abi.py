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


def test_go_bridge_names_only_declared_entry_points():
    """The Go plugin layer (go/b200) cannot be compiled where this library is built, so at least every C function its
    cgo bridge calls must be one include/b200mlx.h declares, with the argument count the header gives it."""
    import re

    from go_darwinml_b200 import _lib
    decls = _lib.parse_header()
    text = open(os.path.join(ROOT, "go", "b200", "internal", "bridge", "bridge.go")).read()
    preamble, body = text.split('import "C"', 1)
    called = set(re.findall(r"\bC\.(b200_\w+)\(", body)) | set(re.findall(r"\b(b200_\w+)\b", preamble.split("b200go_unary_fn", 1)[1]))
    called = {c for c in called if not c.startswith("b200go_")}
    assert called, "no C calls found"
    missing = sorted(c for c in called if c not in decls)
    assert not missing, f"bridge.go calls functions the header does not declare: {missing}"
    # argument counts of the direct calls (balanced-parenthesis scan of each call site)
    for m in re.finditer(r"\bC\.(b200_\w+)\(", body):
        name, i, depth, args, cur = m.group(1), m.end(), 1, 0, False
        while depth:
            ch = body[i]
            if ch == "(":
                depth += 1
            elif ch == ")":
                depth -= 1
            elif ch == "," and depth == 1:
                args += 1
            if not ch.isspace() and depth:
                cur = True
            i += 1
        nargs = args + 1 if cur else 0
        assert nargs == len(decls[name][1]), f"{name}: bridge.go passes {nargs} arguments, the header declares {len(decls[name][1])}"


def test_go_bridge_preamble_is_valid_c():
    """The C block of the cgo bridge (dispatch tables over the unary / binary entry points) compiles against the header."""
    text = open(os.path.join(ROOT, "go", "b200", "internal", "bridge", "bridge.go")).read()
    start = text.index("/*\n#cgo") + 3
    block = text[start:text.index("*/\nimport \"C\"")]
    src = "\n".join(l for l in block.splitlines() if not l.startswith("#cgo")) + "\nint main(void){(void)b200go_unary; (void)b200go_binary; return 0;}\n"
    r = subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), "-x", "c", "-"],
                       input=src, text=True, capture_output=True)
    assert r.returncode == 0, r.stderr
    # the op codes on the Go side index those tables: same lengths
    import re
    unary = re.search(r"b200go_unary_table\[\] = \{(.*?)\};", block, re.S).group(1).split(",")
    binary = re.search(r"b200go_binary_table\[\] = \{(.*?)\};", block, re.S).group(1).split(",")
    go_unary = re.search(r"const \(\n\tOpAbs = iota\n(.*?)\n\)", text, re.S).group(1).split()
    go_binary = re.search(r"const \(\n\tOpAdd = iota\n(.*?)\n\)", text, re.S).group(1).split()
    assert len(unary) == len(go_unary) + 1 and len(binary) == len(go_binary) + 1
