"""Compiles the C restatement (oracle_c.c) into oracle/liboracle_c.so.

The reference itself cannot be compiled here: it is Go plus Objective-C against
Apple's MPSGraph / CoreML frameworks, so there is no oracle/_ref build.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "oracle_c.c")
LIB = os.path.join(HERE, "liboracle_c.so")


def build(force=False):
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(SRC):
        cmd = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-shared", "-fPIC", SRC, "-o", LIB, "-lm"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("gcc failed on oracle_c.c")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
