"""In-tree build of the two native libraries (no JIT cache, no pip):

``libb200cluster.so``   the C ABI of ``include/b200_cluster.h``: hand-written sm_100a CUDA
                        kernels, compiled by nvcc with
                        ``-gencode arch=compute_100a,code=sm_100a``; no torch dependency.
``_torch_ops.so``       the torch operator layer (``torch_cluster::knn`` / ``radius``),
                        compiled by g++ against libtorch and linked to the first.

``python pytorch_cluster_b200/build.py`` builds both (incremental by mtime).  Run it as a script:
importing the package needs the libraries this step produces.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")
OBJ_DIR = os.path.join(PKG, "build")
LIB_CABI = os.path.join(PKG, "libb200cluster.so")
LIB_OPS = os.path.join(PKG, "_torch_ops.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", f"-I{INCLUDE}", f"-I{CSRC}"]


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"command failed ({r.returncode}): {' '.join(cmd)}\n{r.stdout}")
    return r.stdout


def build_cabi(force: bool = False, verbose: bool = False, ptxas_v: bool = False) -> str:
    nvcc = os.path.join(_cuda_home(), "bin", "nvcc")
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        glob.glob(os.path.join(INCLUDE, "*.h"))
    os.makedirs(OBJ_DIR, exist_ok=True)
    jobs, objs = [], []
    for s in sources:
        o = os.path.join(OBJ_DIR, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or not _newer(o, [s] + headers):
            jobs.append([nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_v else []) + ["-c", s, "-o", o])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        outs = list(ex.map(lambda c: _run(c, verbose), jobs))
    if ptxas_v:
        print("\n".join(outs))
    if jobs or not os.path.exists(LIB_CABI):
        _run([nvcc, "-shared", "-o", LIB_CABI] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"], verbose)
    return LIB_CABI


def build_ops(force: bool = False, verbose: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce

    src = os.path.join(CSRC, "torch_ops.cpp")
    deps = [src, os.path.join(INCLUDE, "b200_cluster.h"), os.path.join(INCLUDE, "b200_cluster_torch.h"), LIB_CABI]
    if not force and _newer(LIB_OPS, deps):
        return LIB_OPS
    lib_dir = ce.library_paths()[0]
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-Wno-sign-compare", src, "-o", LIB_OPS,
           f"-I{INCLUDE}", f"-I{os.path.join(_cuda_home(), 'include')}"]
    cmd += [f"-I{p}" for p in ce.include_paths()]
    cmd += [f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += [f"-L{PKG}", "-lb200cluster", "-Wl,-rpath,$ORIGIN", f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}",
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ldl"]
    _run(cmd, verbose)
    return LIB_OPS


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cabi(force, verbose)
    build_ops(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print(LIB_CABI)
    print(LIB_OPS)
