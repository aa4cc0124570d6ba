// Dispatch of radius_lowd_kernel over DIM; included once per data type.
#pragma once

#include "launchers.h"
#include "radius_lowd.cuh"

namespace b200c {

template <typename T, int DIM, int MODE>
static int launch_radius_lowd_one(const RadiusArgs &a) {
  using Cfg = RadiusLowD<T, DIM>;
  auto kern = radius_lowd_kernel<T, DIM, MODE>;
  static unsigned long long configured = 0ull;  // devices on which the shared-memory opt-in is done
  B200C_CUDA(opt_in_shared_memory(kern, Cfg::SMEM_BYTES, configured));
  const int64_t tiles = (a.m + Cfg::TQ - 1) / Cfg::TQ;
  if (tiles > 0x7fffffffLL) {
    set_error("too many query tiles");
    return B200C_ERR_INVALID;
  }
  const T r2 = (T)(a.r * a.r);  // formed in double, narrowed once (csrc/cuda/radius_cuda.cu:90)
  kern<<<(unsigned)tiles, CTA_THREADS, Cfg::SMEM_BYTES, a.stream>>>(
      (const T *)a.x, (const T *)a.y, a.ptr_x, a.ptr_y, a.num_segments, a.n, a.m, r2, a.max_nn,
      a.ignore_same, a.counts, a.offsets, a.out_row, a.out_col, a.direct_rows, a.mask_base, a.mask_words,
      a.query_base);
  B200C_LAUNCH_CHECK("radius_lowd_kernel");
  return B200C_OK;
}

// fill == false: pass 1 (counts; with direct_rows also the hits themselves).
// fill == true : pass 2 (edges from a second scan, or from direct_rows by a compaction copy).
template <typename T, int DIM>
static int launch_radius_lowd_dim(const RadiusArgs &a, bool fill) {
  if (!fill) {
    if (a.mask_words) return launch_radius_lowd_one<T, DIM, RADIUS_COUNT_MASK>(a);
    return a.direct_rows ? launch_radius_lowd_one<T, DIM, RADIUS_DIRECT>(a)
                         : launch_radius_lowd_one<T, DIM, RADIUS_COUNT>(a);
  }
  if (a.mask_words) {
    const int64_t threads = a.m * 32;
    radius_mask_fill_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, a.stream>>>(
        a.mask_words, a.mask_base, a.ptr_x, a.ptr_y, a.num_segments, a.n, a.m, LowD<T, DIM>::XC, a.counts, a.offsets,
        a.out_row, a.out_col);
    B200C_LAUNCH_CHECK("radius_mask_fill_kernel");
    return B200C_OK;
  }
  if (!a.direct_rows) return launch_radius_lowd_one<T, DIM, RADIUS_FILL>(a);
  const int64_t threads = (a.m + 3) / 4 * 32;  // a warp per four queries
  radius_direct_compact_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, a.stream>>>(
      a.direct_rows, a.counts, a.offsets, a.m, a.max_nn, a.out_row, a.out_col);
  B200C_LAUNCH_CHECK("radius_direct_compact_kernel");
  return B200C_OK;
}

template <typename T>
static int launch_radius_lowd(const RadiusArgs &a, bool fill) {
  switch (a.dim) {
    case 1: return launch_radius_lowd_dim<T, 1>(a, fill);
    case 2: return launch_radius_lowd_dim<T, 2>(a, fill);
    case 3: return launch_radius_lowd_dim<T, 3>(a, fill);
    case 4: return launch_radius_lowd_dim<T, 4>(a, fill);
    case 5: return launch_radius_lowd_dim<T, 5>(a, fill);
    case 6: return launch_radius_lowd_dim<T, 6>(a, fill);
    case 7: return launch_radius_lowd_dim<T, 7>(a, fill);
    case 8: return launch_radius_lowd_dim<T, 8>(a, fill);
  }
  set_error("low-dimensional radius kernel called with dim=%d", a.dim);
  return B200C_ERR_INVALID;
}

template <typename T>
static int radius_lowd_chunk_points_t(int dim) {
  switch (dim) {
    case 1: return LowD<T, 1>::XC;
    case 2: return LowD<T, 2>::XC;
    case 3: return LowD<T, 3>::XC;
    case 4: return LowD<T, 4>::XC;
    case 5: return LowD<T, 5>::XC;
    case 6: return LowD<T, 6>::XC;
    case 7: return LowD<T, 7>::XC;
    case 8: return LowD<T, 8>::XC;
  }
  return 0;
}

}  // namespace b200c
