// Test infrastructure only: registers the reference's own CPU neighbour-search
// functions (csrc/cpu/knn_cpu.cpp:7, csrc/cpu/radius_cpu.cpp:7, csrc/cpu/fps_cpu.cpp:11) under the
// separate operator namespace `ref_cluster`, so that they can be loaded next to
// the library under test (which owns the `torch_cluster::knn` /
// `torch_cluster::radius` names, csrc/knn.cpp:39-40, csrc/radius.cpp:38-39).
// The reference sources are compiled where they lie; nothing of them is copied.
#include <torch/script.h>

#include "cpu/fps_cpu.h"
#include "cpu/knn_cpu.h"
#include "cpu/radius_cpu.h"

TORCH_LIBRARY(ref_cluster, m) {
  m.def("knn_cpu(Tensor x, Tensor y, Tensor? ptr_x, Tensor? ptr_y, int k, "
        "int num_workers) -> Tensor",
        &knn_cpu);
  m.def("radius_cpu(Tensor x, Tensor y, Tensor? ptr_x, Tensor? ptr_y, float r, "
        "int max_num_neighbors, int num_workers, bool ignore_same_index) -> "
        "Tensor",
        &radius_cpu);
  m.def("fps_cpu(Tensor src, Tensor ptr, Tensor ratio, bool random_start) -> Tensor", &fps_cpu);
}
