/*
 * b200_cluster_torch.h — C++ API for libtorch programs.
 *
 * The free functions a C++ user of torch_cluster calls (csrc/cluster.h:23-32 of the reference,
 * "C++ API" in its README), implemented by the operator library of this package
 * (`pytorch_cluster_b200/_torch_ops.so`): link against it, include this header and call them with
 * CUDA tensors.  Signatures follow the reference's definitions (csrc/knn.cpp:22-25,
 * csrc/radius.cpp:22-26, csrc/nearest.cpp:22-23, csrc/fps.cpp:22-23); its header still declares
 * `radius` with the six arguments of an older version, the definition — and the registered
 * operator — take eight.  The same functions are registered as `torch_cluster::knn`, `radius`,
 * `nearest` and `fps`, so `torch::jit` programs find them by name once the library is loaded.
 *
 * There is no CPU branch: a CPU tensor raises c10::Error ("x must be CUDA tensor").
 */
#pragma once

#include <torch/script.h>

#include <optional>

#if defined(__GNUC__)
#define B200C_TORCH_API __attribute__((visibility("default")))
#else
#define B200C_TORCH_API
#endif

/* int64 [2, E]: row 0 = row of y, row 1 = one of its k nearest rows of x (same segment),
 * ascending by (distance, index) per query. */
B200C_TORCH_API torch::Tensor knn(torch::Tensor x, torch::Tensor y, std::optional<torch::Tensor> ptr_x,
                                  std::optional<torch::Tensor> ptr_y, int64_t k, bool cosine,
                                  int64_t num_workers);

/* int64 [2, E]: row 0 = row of y, row 1 = a row of x (same segment) closer than r; at most
 * max_num_neighbors per query, the lowest x rows first. */
B200C_TORCH_API torch::Tensor radius(torch::Tensor x, torch::Tensor y, std::optional<torch::Tensor> ptr_x,
                                     std::optional<torch::Tensor> ptr_y, double r, int64_t max_num_neighbors,
                                     int64_t num_workers, bool ignore_same_index);

/* int64 [n]: for every row of x the nearest row of y of the same segment. */
B200C_TORCH_API torch::Tensor nearest(torch::Tensor x, torch::Tensor y, torch::Tensor ptr_x,
                                      torch::Tensor ptr_y);

/* int64 [S]: farthest point samples, ceil(ratio * n_b) per segment. */
B200C_TORCH_API torch::Tensor fps(torch::Tensor src, torch::Tensor ptr, torch::Tensor ratio,
                                  bool random_start);
