"""ctypes binding of libb200mlx.so: one Python callable per C-ABI entry point.

The signatures are read out of include/b200mlx.h at import time, so this file
cannot drift from the header: every function the header declares is bound, and
a symbol the header declares but the library does not export is an ImportError.
"""
from __future__ import annotations

import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "..", "include", "b200mlx.h")
LIB_PATH = os.path.join(HERE, "libb200mlx.so")


class B200Error(ctypes.Structure):
    _fields_ = [("code", ctypes.c_int), ("message", ctypes.c_void_p)]


_CTYPES = {
    "void": None,
    "bool": ctypes.c_bool,
    "int": ctypes.c_int,
    "float": ctypes.c_float,
    "double": ctypes.c_double,
    "int64_t": ctypes.c_int64,
    "unsigned": ctypes.c_ubyte,   # only "unsigned char" occurs
    "B200Context": ctypes.c_void_p,
    "B200Value": ctypes.c_void_p,
    "B200Exec": ctypes.c_void_p,
    "B200Buffer": ctypes.c_void_p,
}


def _ctype_of(decl: str):
    """Maps a C parameter/return type string to a ctypes type."""
    d = decl.replace("const", " ").strip()
    stars = d.count("*")
    base = d.replace("*", " ").split()[0]
    if base == "char" and stars == 1:
        return ctypes.c_void_p  # strings are read with string_at so malloc'd ones can be freed
    if base == "B200Error" and stars == 1:
        return ctypes.POINTER(B200Error)
    if stars == 0:
        return _CTYPES[base]
    if stars == 1:
        if base == "void":
            return ctypes.c_void_p
        if base == "float":
            return ctypes.c_void_p
        return ctypes.POINTER(_CTYPES[base])
    if stars == 2:
        if base == "void":
            return ctypes.POINTER(ctypes.c_void_p)
        return ctypes.POINTER(ctypes.POINTER(_CTYPES[base]))
    raise ValueError(decl)


def parse_header(path: str = HEADER):
    """Returns {name: (restype_decl, [param_decl, ...])} for every function the header declares."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    text = re.sub(r"^\s*#.*$", " ", text, flags=re.M)
    text = re.sub(r'extern\s+"C"\s*\{', " ", text)
    text = re.sub(r"typedef\s+(struct|enum)\s*\{.*?\}\s*\w+\s*;", " ", text, flags=re.S)
    text = re.sub(r"typedef[^;]*;", " ", text)
    out = {}
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(b200_\w+)\s*\(([^)]*)\)\s*;", text):
        ret, name, params = m.group(1).strip(), m.group(2), m.group(3).strip()
        plist = []
        if params and params != "void":
            for p in params.split(","):
                p = " ".join(p.split())
                # drop the parameter name (last identifier not followed by '*')
                pm = re.match(r"(.*?)(\w+)$", p)
                plist.append(pm.group(1).strip() if pm and pm.group(1).strip() else p)
        out[name] = (ret, plist)
    return out


class Library:
    def __init__(self, path: str = LIB_PATH):
        if not os.path.exists(path):
            raise ImportError(
                f"{path} is missing: build it with `python go-darwinml_b200/build.py` "
                "(there is no CPU fallback; the CUDA library is required)")
        self._dll = ctypes.CDLL(path)
        self._libc = ctypes.CDLL(None)
        self._libc.free.argtypes = [ctypes.c_void_p]
        self.decls = parse_header()
        for name, (ret, params) in self.decls.items():
            try:
                fn = getattr(self._dll, name)
            except AttributeError as e:
                raise ImportError(f"{path} does not export {name}, which include/b200mlx.h declares") from e
            fn.restype = _ctype_of(ret)
            fn.argtypes = [_ctype_of(p) for p in params]
            setattr(self, name, fn)

    def free(self, p):
        if p:
            self._libc.free(p)

    def take_string(self, p) -> str:
        """Reads and frees a malloc'd C string."""
        if not p:
            return ""
        s = ctypes.string_at(p).decode("utf-8", "replace")
        self.free(p)
        return s


_lib = None


def lib() -> Library:
    global _lib
    if _lib is None:
        _lib = Library()
    return _lib
