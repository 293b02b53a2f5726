"""Builds libb200mlx.so from csrc/ with nvcc for sm_100a.

Every .cu/.cpp file is compiled to an object in parallel, then linked into
one shared library next to this file.  Nothing here needs a GPU: nvcc
cross-compiles.  Run as `python go-darwinml_b200/build.py [--force] [--verbose]`.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libb200mlx.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-cudart", "static",
    "-DB200MLX_BUILD",
]


def sources():
    out = []
    for root, _, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith((".cu", ".cpp")):
                out.append(os.path.join(root, f))
    return sorted(out)


def headers_mtime():
    m = os.path.getmtime(os.path.join(HERE, "..", "include", "b200mlx.h"))
    for root, _, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".h", ".cuh")):
                m = max(m, os.path.getmtime(os.path.join(root, f)))
    return m


def compile_one(src, obj, verbose):
    cmd = ["nvcc", *NVCC_FLAGS, "-I", OBJ, "-x", "cu", "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    return src, r.returncode, r.stdout + r.stderr


def embed_sources():
    """csrc/kernels/ewise_ops.cuh as a C++ raw string literal (build/ewise_ops_src.inc): the run-time compiler of
    ewise_jit.cu hands that text to NVRTC in front of every generated kernel."""
    src = os.path.join(CSRC, "kernels", "ewise_ops.cuh")
    dst = os.path.join(OBJ, "ewise_ops_src.inc")
    text = 'R"EWOPS(' + open(src).read() + ')EWOPS"\n'
    if not os.path.exists(dst) or open(dst).read() != text:
        with open(dst, "w") as fh:
            fh.write(text)


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    embed_sources()
    hm = headers_mtime()
    jobs = []
    objs = []
    for src in sources():
        obj = os.path.join(OBJ, os.path.relpath(src, CSRC).replace(os.sep, "_") + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hm):
            jobs.append((src, obj))
    failed = False
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
            for src, rc, out in ex.map(lambda j: compile_one(j[0], j[1], verbose), jobs):
                if rc != 0 or verbose:
                    sys.stderr.write(f"--- {os.path.relpath(src, HERE)}\n{out}\n")
                failed |= rc != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if jobs or not os.path.exists(LIB):
        cmd = ["nvcc", "-shared", "-cudart", "static", "-o", LIB, *objs, "-Xlinker", "--no-undefined", "-ldl", "-lpthread", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
