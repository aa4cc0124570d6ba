"""Compile ``oracle/neighbor_oracle.c`` into ``oracle/_build/libneighbor_oracle.so``.

``-ffp-contract=off`` keeps gcc from fusing anything but the explicit
``fma``/``fmaf`` calls, which is what makes the two rounding policies of the
oracle distinct.  ``python oracle/build.py`` (idempotent).
"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "neighbor_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libneighbor_oracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["gcc", "-std=c11", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
           "-Wall", "-Wno-unknown-pragmas", SRC, "-o", OUT, "-lm"]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
