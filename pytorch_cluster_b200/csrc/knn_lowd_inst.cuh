// Dispatch of knn_lowd_kernel over (DIM, KP); included once per data type.
#pragma once

#include "knn_lowd.cuh"
#include "launchers.h"

namespace b200c {

template <typename T, int DIM, int KP>
static int launch_knn_lowd_one(const KnnArgs &a) {
  using Cfg = KnnLowD<T, DIM, KP>;
  auto kern = knn_lowd_kernel<T, DIM, KP>;
  static unsigned long long configured = 0ull;  // devices on which the shared-memory opt-in is done
  B200C_CUDA(opt_in_shared_memory(kern, Cfg::SMEM_BYTES, configured));
  const int64_t tiles = (a.m + Cfg::TQ - 1) / Cfg::TQ;
  if (tiles > 0x7fffffffLL) {
    set_error("too many query tiles");
    return B200C_ERR_INVALID;
  }
  kern<<<(unsigned)tiles, CTA_THREADS, Cfg::SMEM_BYTES, a.stream>>>(
      (const T *)a.x, (const T *)a.y, a.ptr_x, a.ptr_y, a.num_segments, a.n, a.m, a.k, a.out_row,
      a.out_col, a.counts, a.num_valid, a.graph_out, a.graph_row_stride, a.graph_index_base, a.graph_s2t,
      a.graph_irregular);
  B200C_LAUNCH_CHECK("knn_lowd_kernel");
  return B200C_OK;
}

template <typename T, int DIM>
static int launch_knn_lowd_dim(const KnnArgs &a) {
  if (a.k <= 32) return launch_knn_lowd_one<T, DIM, 32>(a);
  if (a.k <= 64) return launch_knn_lowd_one<T, DIM, 64>(a);
  return launch_knn_lowd_one<T, DIM, 128>(a);
}

template <typename T>
static int launch_knn_lowd(const KnnArgs &a) {
  switch (a.dim) {
    case 1: return launch_knn_lowd_dim<T, 1>(a);
    case 2: return launch_knn_lowd_dim<T, 2>(a);
    case 3: return launch_knn_lowd_dim<T, 3>(a);
    case 4: return launch_knn_lowd_dim<T, 4>(a);
    case 5: return launch_knn_lowd_dim<T, 5>(a);
    case 6: return launch_knn_lowd_dim<T, 6>(a);
    case 7: return launch_knn_lowd_dim<T, 7>(a);
    case 8: return launch_knn_lowd_dim<T, 8>(a);
  }
  set_error("low-dimensional kNN kernel called with dim=%d", a.dim);
  return B200C_ERR_INVALID;
}

}  // namespace b200c
