"""CPU-side checks of the boundary: the C ABI library loads without a GPU and exports every
function that include/b200_cluster.h declares; the operator library registers the reference's
operator names and schemas; the Python functions keep the reference's signatures."""
import ctypes
import inspect
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "b200_cluster.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200c_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("b200c_knn", "b200c_radius_count", "b200c_radius_fill", "b200c_exclusive_scan",
                 "b200c_segment_ptr", "b200c_knn_compact", "b200c_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from pytorch_cluster_b200 import _native

    lib = ctypes.CDLL(_native.LIB_CABI)
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"
    assert lib.b200c_version() >= 100


def test_no_compute_entry_point_runs_without_valid_arguments():
    # argument checks come before any CUDA call, so this is safe without a GPU
    from pytorch_cluster_b200 import _native

    lib = _native.cabi()
    st = lib.b200c_knn(None, None, None, None, 1, 10, 10, 3, 5, 0, 0, None, None, None, 0, None, 0, None)
    assert st == 1 and b"CUDA tensors" in lib.b200c_last_error()
    st = lib.b200c_radius_count(None, None, None, None, 1, 10, 10, 3, 1.0, 32, 0, 0, None, None, 0, None)
    assert st == 1
    assert lib.b200c_scan_workspace_bytes(5000) == 8 * 3


def test_operator_schemas_match_the_reference():
    import pytorch_cluster_b200  # noqa: F401

    knn = str(torch.ops.torch_cluster.knn.default._schema)
    rad = str(torch.ops.torch_cluster.radius.default._schema)
    assert knn.startswith("torch_cluster::knn(Tensor _0, Tensor _1, Tensor? _2, Tensor? _3, int _4, bool _5, int _6) -> Tensor")
    assert rad.startswith("torch_cluster::radius(Tensor _0, Tensor _1, Tensor? _2, Tensor? _3, float _4, int _5, int _6, bool _7) -> Tensor")


def test_python_signatures_match_the_reference():
    import pytorch_cluster_b200 as pc
    import torch_cluster as shim

    def params(f):
        return [(p.name, p.default) for p in inspect.signature(f).parameters.values()]

    E = inspect.Parameter.empty
    assert params(pc.knn) == [("x", E), ("y", E), ("k", E), ("batch_x", None), ("batch_y", None), ("cosine", False),
                              ("num_workers", 1), ("batch_size", None)]
    assert params(pc.knn_graph) == [("x", E), ("k", E), ("batch", None), ("loop", False),
                                    ("flow", "source_to_target"), ("cosine", False), ("num_workers", 1),
                                    ("batch_size", None)]
    assert params(pc.radius) == [("x", E), ("y", E), ("r", E), ("batch_x", None), ("batch_y", None),
                                 ("max_num_neighbors", 32), ("num_workers", 1), ("batch_size", None),
                                 ("ignore_same_index", False)]
    assert params(pc.radius_graph) == [("x", E), ("r", E), ("batch", None), ("loop", False),
                                       ("max_num_neighbors", 32), ("flow", "source_to_target"), ("num_workers", 1),
                                       ("batch_size", None)]
    assert shim.knn is pc.knn and shim.radius_graph is pc.radius_graph
    for f in (pc.knn, pc.knn_graph, pc.radius, pc.radius_graph):
        torch.jit.script(f)


def test_cpu_tensors_are_refused_not_served():
    import pytorch_cluster_b200 as pc

    with pytest.raises(RuntimeError, match="must be CUDA tensor"):
        pc.knn(torch.rand(8, 3), torch.rand(2, 3), 2)
    with pytest.raises(RuntimeError, match="must be CUDA tensor"):
        pc.radius_graph(torch.rand(8, 3), 0.5)
    # empty inputs never reach the operator (torch_cluster/knn.py:55-56)
    assert pc.knn(torch.empty(0, 3), torch.rand(2, 3), 2).shape == (2, 0)


def test_fps_segment_classification():
    """Which fps kernel a segment goes to: the common call (0), the many-SM kernel (1: more points than
    one thread block keeps in registers, at most what all SMs hold) or a call of its own from global
    memory (2: more than that).  Segments without samples stay in the common call."""
    import pytorch_cluster_b200  # noqa: F401

    ptr = torch.tensor([0, 10, 8202, 8202, 30000, 30010, 1300000, 1300005])
    out = torch.tensor([0, 1, 3, 3, 4, 5, 6, 6])
    cls = torch.ops.torch_cluster.fps_segment_classes(ptr, out, 8192, 1212416)
    #            10 pts  8192   0 pts  21798  10   1269990  5 pts / no sample
    assert cls.tolist() == [0, 0, 0, 1, 0, 2, 0]
    cls = torch.ops.torch_cluster.fps_segment_classes(ptr, out, 8192, 20000)
    assert cls.tolist() == [0, 0, 0, 2, 0, 2, 0]
    big = torch.tensor([0, 8193]), torch.tensor([0, 0])
    assert torch.ops.torch_cluster.fps_segment_classes(big[0], big[1], 8192, 100000).tolist() == [0]


def test_cpp_api_header_links_against_the_operator_library(tmp_path):
    """A libtorch program includes include/b200_cluster_torch.h, links _torch_ops.so and calls the free
    functions `knn` and `radius` (the reference's C++ API, csrc/cluster.h:23-32).  Without a GPU the
    calls must end in c10::Error "x must be CUDA tensor": there is no CPU branch."""
    import subprocess

    from torch.utils import cpp_extension as ce

    from pytorch_cluster_b200 import _native

    src = tmp_path / "use_api.cpp"
    src.write_text('''
#include "b200_cluster_torch.h"
#include <iostream>
int main() {
  auto x = torch::rand({16, 3});
  int caught = 0;
  try { knn(x, x, std::nullopt, std::nullopt, 4, false, 1); } catch (const c10::Error &e) {
    caught += std::string(e.what()).find("x must be CUDA tensor") != std::string::npos;
  }
  try { radius(x, x, std::nullopt, std::nullopt, 0.5, 8, 1, false); } catch (const c10::Error &e) {
    caught += std::string(e.what()).find("x must be CUDA tensor") != std::string::npos;
  }
  try { nearest(x, x, torch::tensor({0, 16}), torch::tensor({0, 16})); } catch (const c10::Error &e) { caught += 1; }
  try { fps(x, torch::tensor({0, 16}), torch::tensor(0.5), false); } catch (const c10::Error &e) { caught += 1; }
  std::cout << "caught " << caught << std::endl;
  return caught == 4 ? 0 : 1;
}
''')
    exe = tmp_path / "use_api"
    pkg = os.path.dirname(_native.LIB_OPS)
    lib_dir = ce.library_paths()[0]
    cmd = ["g++", "-std=c++17", "-O0", str(src), "-o", str(exe), f"-I{os.path.join(ROOT, 'include')}"]
    cmd += [f"-I{p}" for p in ce.include_paths()]
    cmd += [f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", f"-L{pkg}", "-l:_torch_ops.so",
            "-lb200cluster", f"-Wl,-rpath,{pkg}", f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}", "-ltorch", "-ltorch_cpu",
            "-lc10"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
