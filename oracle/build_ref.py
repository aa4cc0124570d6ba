"""Build recipe for ``oracle/_ref/ref_cluster_cpu.so`` (test infrastructure).

Compiles the reference's unmodified CPU neighbour search
(``csrc/cpu/knn_cpu.cpp``, ``csrc/cpu/radius_cpu.cpp``, ``csrc/cpu/fps_cpu.cpp`` with the vendored
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
OUT_CUDA = os.path.join(OUT_DIR, "ref_cluster_cuda.so")


def default_reference_dir() -> str:
    """Where the reference checkout is looked for: ``$REFERENCE_DIR``, else a directory named
    ``reference`` beside this repository."""
    return os.environ.get("REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


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
        os.path.join(csrc, "cpu", "fps_cpu.cpp"),
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


def build_cuda(reference: str, force: bool = False, verbose: bool = True) -> str | None:
    """Compile the reference's unmodified CUDA kernels of this path
    (``csrc/cuda/knn_cuda.cu``, ``radius_cuda.cu``, ``nearest_cuda.cu``, ``fps_cuda.cu``) for sm_100a with nvcc, plus
    ``oracle/ref_shim_cuda.cpp``, into ``oracle/_ref/ref_cluster_cuda.so``.  Returns the path,
    or None when neither the reference checkout nor a previously built file exists."""
    import shutil

    csrc = os.path.join(reference, "csrc")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isdir(csrc) or not os.path.exists(nvcc):
        return OUT_CUDA if os.path.exists(OUT_CUDA) else None
    cu = [os.path.join(csrc, "cuda", f) for f in ("knn_cuda.cu", "radius_cuda.cu", "nearest_cuda.cu", "fps_cuda.cu")]
    shim = os.path.join(HERE, "ref_shim_cuda.cpp")
    if not force and os.path.exists(OUT_CUDA) and all(
        os.path.getmtime(OUT_CUDA) >= os.path.getmtime(s) for s in cu + [shim]
    ):
        return OUT_CUDA
    os.makedirs(OUT_DIR, exist_ok=True)
    cflags, ldflags = torch_flags()
    cuda_home = os.path.dirname(os.path.dirname(nvcc))
    cflags = cflags + [f"-I{cuda_home}/include"]
    procs, objs = [], []
    for s in cu:
        o = os.path.join(OUT_DIR, os.path.basename(s) + ".o")
        objs.append(o)
        cmd = [nvcc, "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a",
               "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-c", s, "-o", o, f"-I{csrc}"] + cflags + [
                   # what torch.utils.cpp_extension adds to every nvcc command of a CUDAExtension
                   "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
                   "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__"]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append(subprocess.Popen(cmd))
    o = os.path.join(OUT_DIR, "ref_shim_cuda.cpp.o")
    objs.append(o)
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-Wno-sign-compare", "-c", shim, "-o", o, f"-I{csrc}"] + cflags
    if verbose:
        print(" ".join(cmd), flush=True)
    procs.append(subprocess.Popen(cmd))
    for p in procs:
        if p.wait() != 0:
            raise RuntimeError("compiling the reference CUDA path failed")
    lib_dir = [f for f in ldflags if f.startswith("-L")][0][2:]
    cmd = ["g++", "-shared", "-o", OUT_CUDA] + objs + ldflags + [
        "-ltorch_cuda", "-lc10_cuda", f"-L{cuda_home}/lib64", "-lcudart"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return OUT_CUDA


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=default_reference_dir())
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    out = build(a.reference, a.force)
    print(out or "reference checkout not found; nothing built")
    print(build_cuda(a.reference, a.force) or "reference CUDA path not built")
    sys.exit(0 if out else 1)
