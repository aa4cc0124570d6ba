// Test infrastructure only: registers the reference's own CUDA neighbour-search
// functions (csrc/cuda/knn_cuda.cu:86, csrc/cuda/radius_cuda.cu:44, csrc/cuda/nearest_cuda.cu:63,
// csrc/cuda/fps_cuda.cu:70) under the
// separate operator namespace `ref_cluster_cuda`, so that they can be loaded next
// to the library under test (which owns `torch_cluster::knn` / `torch_cluster::radius`).
// The reference sources are compiled where they lie, for sm_100a; nothing of them is
// copied.  They serve as a second parity checker on the GPU and as the timed
// "kernel to beat"; no product code path loads this library.
#include <torch/script.h>

#include "cuda/knn_cuda.h"
#include "cuda/fps_cuda.h"
#include "cuda/nearest_cuda.h"
#include "cuda/radius_cuda.h"

TORCH_LIBRARY(ref_cluster_cuda, m) {
  m.def("knn_cuda(Tensor x, Tensor y, Tensor? ptr_x, Tensor? ptr_y, int k, "
        "bool cosine) -> Tensor",
        &knn_cuda);
  m.def("radius_cuda(Tensor x, Tensor y, Tensor? ptr_x, Tensor? ptr_y, float r, "
        "int max_num_neighbors, bool ignore_same_index) -> Tensor",
        &radius_cuda);
  m.def("nearest_cuda(Tensor x, Tensor y, Tensor ptr_x, Tensor ptr_y) -> Tensor", &nearest_cuda);
  m.def("fps_cuda(Tensor src, Tensor ptr, Tensor ratio, bool random_start) -> Tensor", &fps_cuda);
}
