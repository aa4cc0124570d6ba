"""Build recipe for ``oracle/_ref/ref_cluster_cpu.so`` (test infrastructure).

Compiles the reference's unmodified CPU neighbour search
(``csrc/cpu/knn_cpu.cpp``, ``csrc/cpu/radius_cpu.cpp`` with the vendored
nanoflann header under ``csrc/cpu/utils``) straight from the reference checkout
with g++, together with ``oracle/ref_shim.cpp`` which registers the two
functions as ``ref_cluster::knn_cpu`` / ``ref_cluster::radius_cpu``.  Flags
follow the reference's own build (``setup.py:47-59``: ``-O2``,
``-Wno-sign-compare``).  The reference's build system is not run.

Usage: ``python oracle/build_ref.py [--reference DIR] [--force]``.
The output is git-ignored; it is a checker and a timed CPU baseline, never part
of the product path.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "ref_cluster_cpu.so")


def torch_flags():
    import torch
    from torch.utils import cpp_extension as ce

    inc = [f"-I{p}" for p in ce.include_paths()]
    lib_dir = ce.library_paths()[0]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cflags = inc + [f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
    ldflags = [f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}", "-ltorch", "-ltorch_cpu", "-lc10"]
    return cflags, ldflags


def build(reference: str, force: bool = False, verbose: bool = True) -> str | None:
    """Compile the reference CPU path; returns the .so path, or None when the
    reference checkout is absent (then a previously built file is used as is)."""
    csrc = os.path.join(reference, "csrc")
    if not os.path.isdir(csrc):
        return OUT if os.path.exists(OUT) else None
    srcs = [
        os.path.join(csrc, "cpu", "knn_cpu.cpp"),
        os.path.join(csrc, "cpu", "radius_cpu.cpp"),
        os.path.join(HERE, "ref_shim.cpp"),
    ]
    if not force and os.path.exists(OUT) and all(
        os.path.getmtime(OUT) >= os.path.getmtime(s) for s in srcs
    ):
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    cflags, ldflags = torch_flags()
    objs = []
    procs = []
    for s in srcs:
        o = os.path.join(OUT_DIR, os.path.basename(s) + ".o")
        objs.append(o)
        cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-Wno-sign-compare", "-c", s, "-o", o,
               f"-I{csrc}"] + cflags
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append(subprocess.Popen(cmd))
    for p in procs:
        if p.wait() != 0:
            raise RuntimeError("compiling the reference CPU path failed")
    cmd = ["g++", "-shared", "-o", OUT] + objs + ldflags
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("REFERENCE_DIR", "/root/reference"))
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    out = build(a.reference, a.force)
    print(out or "reference checkout not found; nothing built")
    sys.exit(0 if out else 1)
