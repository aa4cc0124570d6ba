// Dispatch of generic_kernel; included once per data type.
#pragma once

#include "generic.cuh"
#include "launchers.h"

namespace b200c {

template <typename T, int MODE, int KP, bool COSINE, int RND>
static int launch_generic_one(const KnnArgs *ka, const RadiusArgs *ra) {
  using S = GenSmem<T, KP>;
  using G = GenD<T>;
  auto kern = generic_kernel<T, MODE, KP, COSINE, RND>;
  static unsigned long long configured = 0ull;  // devices on which the shared-memory opt-in is done
  B200C_CUDA(opt_in_shared_memory(kern, S::SMEM_BYTES, configured));
  const int64_t m = ka ? ka->m : ra->m;
  const int64_t tiles = (m + G::TQ - 1) / G::TQ;
  if (tiles > 0x7fffffffLL) {
    set_error("too many query tiles");
    return B200C_ERR_INVALID;
  }
  if (ka) {
    kern<<<(unsigned)tiles, CTA_THREADS, S::SMEM_BYTES, ka->stream>>>(
        (const T *)ka->x, (const T *)ka->y, ka->ptr_x, ka->ptr_y, ka->num_segments, ka->n, ka->m, ka->dim,
        ka->k, (T)0, (int64_t)0, 0, (const T *)ka->norms_x, (const T *)ka->norms_y, nullptr, ka->out_row,
        ka->out_col, ka->counts, ka->num_valid, (int64_t)0);
  } else {
    // formed in double, narrowed once (csrc/cuda/radius_cuda.cu:90); the 16-bit types narrow through
    // float, as the conversion constructors of c10::Half / c10::BFloat16 do
    T r2 = (T)(ra->r * ra->r);
    if (RND == 1) r2 = (T)__half2float(__float2half_rn((float)r2));
    if (RND == 2) r2 = (T)__bfloat162float(__float2bfloat16_rn((float)r2));
    kern<<<(unsigned)tiles, CTA_THREADS, S::SMEM_BYTES, ra->stream>>>(
        (const T *)ra->x, (const T *)ra->y, ra->ptr_x, ra->ptr_y, ra->num_segments, ra->n, ra->m, ra->dim, 0,
        r2, ra->max_nn, ra->ignore_same, nullptr, nullptr, ra->offsets, ra->out_row, ra->out_col, ra->counts,
        nullptr, ra->query_base);
  }
  B200C_LAUNCH_CHECK("generic_kernel");
  return B200C_OK;
}

template <typename T, bool COSINE, int RND>
static int launch_knn_generic_k(const KnnArgs &a) {
  if (a.k <= 32) return launch_generic_one<T, GEN_KNN, 32, COSINE, RND>(&a, nullptr);
  if (a.k <= 64) return launch_generic_one<T, GEN_KNN, 64, COSINE, RND>(&a, nullptr);
  return launch_generic_one<T, GEN_KNN, 128, COSINE, RND>(&a, nullptr);
}

template <typename T, int RND = 0>
static int launch_knn_generic(const KnnArgs &a) {
  return a.cosine ? launch_knn_generic_k<T, true, RND>(a) : launch_knn_generic_k<T, false, RND>(a);
}

template <typename T, int RND = 0>
static int launch_radius_generic(const RadiusArgs &a, bool fill) {
  return fill ? launch_generic_one<T, GEN_RADIUS_FILL, 0, false, RND>(nullptr, &a)
              : launch_generic_one<T, GEN_RADIUS_COUNT, 0, false, RND>(nullptr, &a);
}

// nearest: a.x / a.ptr_x describe the points searched, a.y / a.ptr_y the rows assigned; a.out_col [a.m]
template <typename T, int RND = 0>
static int launch_nearest_generic(const KnnArgs &a) {
  return launch_generic_one<T, GEN_NEAREST, 0, false, RND>(&a, nullptr);
}

template <typename T, int RND = 0>
static int launch_row_norms_t(const void *a, int64_t rows, int dim, void *out, cudaStream_t stream) {
  if (rows == 0) return B200C_OK;
  row_norms_kernel<T, RND><<<(unsigned)((rows + 127) / 128), 128, 0, stream>>>((const T *)a, rows, dim, (T *)out);
  B200C_LAUNCH_CHECK("row_norms_kernel");
  return B200C_OK;
}

}  // namespace b200c
